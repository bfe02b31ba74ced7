// Stand-alone forms of the indexer operators that the shipped flows chain: GeMM, Softmax, Normalize, the
// RAGGED reductions, the (BATCHED, PAGED) binary operators, Transpose and Save / Load.
//
// The shipped flows run these operators as links of one fused kernel (indexer_body.cuh); the kernels here are
// what a flow gets when it composes them differently or reads an intermediate.  They compute the same bits as
// the fused forms (one canonical order per reduction, one rounding to bf16 per operator output) and stream
// their operands once: HBM-bound, a few bytes per element, not on the measured path.
//
// Every kernel works on the candidate window of each segment - packed positions
// [dense_kv_indptr[s] + bos, dense_kv_indptr[s + 1] - eos) of segments with more than topk_val candidates -
// which is where the reference's workload list sends its Triton programs (csrc/utils_sglang.cu:219-251).
// One CTA per segment; bf16 only (as the reference's kernels are).
//
// Canonical orders (shared with the CPU checker):
//   dot / sum over the last axis  the axis is cut in chunks of 8 (padded with +0.0), L = min(32, pow2ceil(chunks))
//                                 partial sums, partial l adds chunks l, l + L, ... element by element in fp32
//                                 (no FMA), partials folded v[i] += v[i + w], w = L/2 .. 1;
//   sum over the page axis        128 partial sums (candidate i goes to partial i % 128, ascending), folded in
//                                 halves w = 64 .. 1;
//   sum over axis 1               sequential in ascending order from +0.0.
#include "vtx_common.cuh"

namespace {

constexpr int kThreads = 128;

__device__ __forceinline__ float ld_bf16(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// exp(x) for x <= 0 as a fixed sequence of fp32 operations (the same sequence as the fused indexer's softmax)
__device__ __forceinline__ float exp_canonical(float x) {
    if (x < -87.0f) return 0.f;
    const float k = rintf(__fmul_rn(x, 1.44269504f));
    float r = __fsub_rn(x, __fmul_rn(k, 0.693145751953125f));
    r = __fsub_rn(r, __fmul_rn(k, 1.42860677e-6f));
    float p = (float)(1.0 / 720.0);
    p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 120.0));
    p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 24.0));
    p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 6.0));
    p = __fadd_rn(__fmul_rn(p, r), 0.5f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f);
    return __fmul_rn(p, __int_as_float(((int)k + 127) << 23));
}

struct Window {
    int beg, cnt;  // first packed position and number of candidates; cnt == 0: nothing to do
};

__device__ __forceinline__ Window window_of(const int32_t* indptr, int s, int K, int bos, int eos) {
    const int a = indptr[s] + bos, b = indptr[s + 1] - eos;
    Window w;
    w.beg = a;
    w.cnt = b - a > K ? b - a : 0;
    return w;
}

__device__ __forceinline__ int lanes_for(int n) {  // min(32, pow2ceil(ceil(n / 8)))
    int nch = (n + 7) / 8, L = 1;
    while (L < nch && L < 32) L <<= 1;
    return L;
}

// Canonical sum of f(j), j < n, over the last axis, by one thread.
template <typename F>
__device__ __forceinline__ float canonical_sum_thread(int n, F f) {
    const int nch = (n + 7) / 8, L = lanes_for(n);
    float part[32];
#pragma unroll
    for (int l = 0; l < 32; ++l) part[l] = 0.f;
    for (int c0 = 0; c0 < nch; c0 += L)
        for (int l = 0; l < L && c0 + l < nch; ++l)
            for (int j = 0; j < 8; ++j) {
                const int idx = (c0 + l) * 8 + j;
                part[l] = __fadd_rn(part[l], idx < n ? f(idx) : 0.f);
            }
    for (int w = L >> 1; w > 0; w >>= 1)
        for (int i = 0; i < w; ++i) part[i] = __fadd_rn(part[i], part[i + w]);
    return part[0];
}

// Canonical sum over the CTA's candidates: thread t holds the partial of candidates t, t + 128, ...
__device__ __forceinline__ float fold128(float mine, float* red) {
    red[threadIdx.x] = mine;
    __syncthreads();
    for (int w = kThreads / 2; w > 0; w >>= 1) {
        if (threadIdx.x < w) red[threadIdx.x] = __fadd_rn(red[threadIdx.x], red[threadIdx.x + w]);
        __syncthreads();
    }
    const float total = red[0];
    __syncthreads();
    return total;
}

__device__ __forceinline__ float max128(float mine, float* red) {
    red[threadIdx.x] = mine;
    __syncthreads();
    float m = red[0];
    for (int t = 1; t < kThreads; ++t) m = fmaxf(m, red[t]);
    __syncthreads();
    return m;
}

// ---- GeMM on (BATCHED, PAGED): out[p, c, g] = table[row_p, c, :] . q[s, g, :], fp32 products and sum ----
// One warp per (candidate, c): lane l < L owns the partial sums' chunks l, l + L, ...
__global__ void __launch_bounds__(kThreads) gemm_bpr_kernel(const __nv_bfloat16* __restrict__ q,
                                                           const __nv_bfloat16* __restrict__ table,
                                                           __nv_bfloat16* __restrict__ out,
                                                           const int32_t* __restrict__ indptr,
                                                           const int32_t* __restrict__ indices, int G, int C, int D, int K,
                                                           int bos, int eos) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int s = blockIdx.x;
    const Window w = window_of(indptr, s, K, bos, eos);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nch = D / 8, L = lanes_for(D);
    const __nv_bfloat16* qs = q + (int64_t)s * G * D;
    for (int item = warp; item < w.cnt * C; item += kThreads / 32) {
        const int i = item / C, c = item - i * C;
        const int p = w.beg + i;
        const __nv_bfloat16* row = table + ((int64_t)VTX_CHECK_SUMMARY_ROW(indices[p]) * C + c) * D;
        for (int g = 0; g < G; ++g) {
            float acc = 0.f;
            if (lane < L)
                for (int ch = lane; ch < nch; ch += L) {
                    vtx::Vec8<__nv_bfloat16> rv, qv;
                    rv.load_cached(row + ch * 8);
                    qv.load_cached(qs + (int64_t)g * D + ch * 8);
                    float rf[8], qf[8];
                    rv.unpack(rf);
                    qv.unpack(qf);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc = __fadd_rn(acc, __fmul_rn(rf[j], qf[j]));
                }
            for (int ww = L >> 1; ww > 0; ww >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, ww));
            if (lane == 0) out[((int64_t)p * C + c) * G + g] = __float2bfloat16_rn(acc);
        }
    }
}

// ---- Softmax(dim=0, scale) / Normalize(dim=0) in place over the candidates of a segment, per inner element ----
template <bool NORMALIZE>
__global__ void __launch_bounds__(kThreads) scan_ragged_kernel(__nv_bfloat16* __restrict__ x,
                                                              const int32_t* __restrict__ indptr, int inner, int K,
                                                              int bos, int eos, float scale, float eps) {
    __shared__ float red[kThreads];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const Window w = window_of(indptr, blockIdx.x, K, bos, eos);
    if (w.cnt == 0) return;
    for (int e = 0; e < inner; ++e) {
        __nv_bfloat16* col = x + (int64_t)w.beg * inner + e;
        if (NORMALIZE) {
            float part = 0.f;
            for (int i = threadIdx.x; i < w.cnt; i += kThreads) {
                const float v = ld_bf16(col + (int64_t)i * inner);
                part = __fadd_rn(part, __fmul_rn(v, v));
            }
            const float nrm = fmaxf(__fsqrt_rn(fold128(part, red)), eps);
            for (int i = threadIdx.x; i < w.cnt; i += kThreads)
                col[(int64_t)i * inner] = __float2bfloat16_rn(__fdiv_rn(ld_bf16(col + (int64_t)i * inner), nrm));
        } else {
            float mx = -INFINITY;
            for (int i = threadIdx.x; i < w.cnt; i += kThreads)
                mx = fmaxf(mx, __fmul_rn(ld_bf16(col + (int64_t)i * inner), scale));
            mx = max128(mx, red);
            float part = 0.f;
            for (int i = threadIdx.x; i < w.cnt; i += kThreads)
                part = __fadd_rn(part, exp_canonical(__fsub_rn(__fmul_rn(ld_bf16(col + (int64_t)i * inner), scale), mx)));
            const float l = fold128(part, red);
            for (int i = threadIdx.x; i < w.cnt; i += kThreads) {
                const float t = __fmul_rn(ld_bf16(col + (int64_t)i * inner), scale);
                col[(int64_t)i * inner] = __float2bfloat16_rn(__fdiv_rn(exp_canonical(__fsub_rn(t, mx)), l));
            }
        }
        __syncthreads();
    }
}

// ---- RAGGED reductions over axis 1 or 2 of [N, R, C]; kind: 0 mean, 1 max, 2 min, 3 l2norm, 4 sum ----
__global__ void __launch_bounds__(kThreads) reduce_ragged_kernel(const __nv_bfloat16* __restrict__ x,
                                                                __nv_bfloat16* __restrict__ out,
                                                                const int32_t* __restrict__ indptr, int R, int C, int dim,
                                                                int kind, int K, int bos, int eos) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const Window w = window_of(indptr, blockIdx.x, K, bos, eos);
    const int keep = dim == 1 ? C : R, len = dim == 1 ? R : C;
    for (int item = threadIdx.x; item < w.cnt * keep; item += kThreads) {
        const int i = item / keep, o = item - i * keep;
        const int64_t p = w.beg + i;
        const __nv_bfloat16* base = x + p * R * C;
        auto at = [&](int j) { return dim == 1 ? ld_bf16(base + (int64_t)j * C + o) : ld_bf16(base + (int64_t)o * C + j); };
        float r;
        if (kind == 1 || kind == 2) {
            r = at(0);
            for (int j = 1; j < len; ++j) r = kind == 1 ? fmaxf(r, at(j)) : fminf(r, at(j));
        } else {
            auto term = [&](int j) {
                const float v = at(j);
                return kind == 3 ? __fmul_rn(v, v) : v;
            };
            if (dim == 2) {
                r = canonical_sum_thread(len, term);
            } else {
                r = 0.f;
                for (int j = 0; j < len; ++j) r = __fadd_rn(r, term(j));
            }
            if (kind == 0) r = __fdiv_rn(r, (float)len);
            else if (kind == 3) r = __fsqrt_rn(r);
        }
        out[p * keep + o] = __float2bfloat16_rn(r);
    }
}

// ---- binary operators on (BATCHED, PAGED): out[p] = op(q[s], table[row_p]), inner dims broadcast; with x_ragged
// the left operand is the RAGGED row q[p] instead (the (RAGGED, PAGED) form) ----
// op 0 max, 1 min, 2 bf16(alpha x) + bf16(beta y), 3 x y; one rounding per bf16 operation
__global__ void __launch_bounds__(kThreads) binary_bpr_kernel(const __nv_bfloat16* __restrict__ q,
                                                             const __nv_bfloat16* __restrict__ table,
                                                             __nv_bfloat16* __restrict__ out,
                                                             const int32_t* __restrict__ indptr,
                                                             const int32_t* __restrict__ indices, int a0, int a1, int b0,
                                                             int b1, int op, float alpha, float beta, int K, int bos,
                                                             int eos, int x_ragged) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int s = blockIdx.x;
    const Window w = window_of(indptr, s, K, bos, eos);
    const int o0 = a0 > b0 ? a0 : b0, o1 = a1 > b1 ? a1 : b1, inner = o0 * o1;
    const __nv_bfloat16* qs = q + (int64_t)s * a0 * a1;
    for (int64_t item = threadIdx.x; item < (int64_t)w.cnt * inner; item += kThreads) {
        const int i = (int)(item / inner), e = (int)(item - (int64_t)i * inner), c = e / o1, d = e - c * o1;
        const int64_t p = w.beg + i;
        const __nv_bfloat16* xs = x_ragged ? q + p * a0 * a1 : qs;  // left operand: the row itself or the segment's query
        const float a = ld_bf16(xs + (a0 == 1 ? 0 : c) * a1 + (a1 == 1 ? 0 : d));
        const float b = ld_bf16(table + ((int64_t)VTX_CHECK_SUMMARY_ROW(indices[p]) * b0 + (b0 == 1 ? 0 : c)) * b1 + (b1 == 1 ? 0 : d));
        float o;
        if (op == 0) o = fmaxf(a, b);
        else if (op == 1) o = fminf(a, b);
        else if (op == 2) o = __fadd_rn(bf16_round(__fmul_rn(alpha, a)), bf16_round(__fmul_rn(beta, b)));
        else o = __fmul_rn(a, b);
        out[p * inner + e] = __float2bfloat16_rn(o);
    }
}

// ---- Transpose of the inner dims: out[p, c, r] = x[p, r, c] ----
__global__ void __launch_bounds__(kThreads) transpose_ragged_kernel(const __nv_bfloat16* __restrict__ x,
                                                                   __nv_bfloat16* __restrict__ out,
                                                                   const int32_t* __restrict__ indptr, int R, int C, int K,
                                                                   int bos, int eos) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const Window w = window_of(indptr, blockIdx.x, K, bos, eos);
    const int inner = R * C;
    for (int64_t item = threadIdx.x; item < (int64_t)w.cnt * inner; item += kThreads) {
        const int i = (int)(item / inner), e = (int)(item - (int64_t)i * inner), c = e / R, r = e - c * R;
        const int64_t p = w.beg + i;
        out[p * inner + e] = x[p * inner + (int64_t)r * C + c];
    }
}

// ---- Save (RAGGED -> PAGED: paged[row_p] = x[p]) and Load (PAGED -> RAGGED: out[p] = paged[row_p]) ----
template <bool SAVE>
__global__ void __launch_bounds__(kThreads) save_load_kernel(__nv_bfloat16* __restrict__ ragged,
                                                            __nv_bfloat16* __restrict__ paged,
                                                            const int32_t* __restrict__ indptr,
                                                            const int32_t* __restrict__ indices, int inner, int K, int bos,
                                                            int eos) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const Window w = window_of(indptr, blockIdx.x, K, bos, eos);
    for (int64_t item = threadIdx.x; item < (int64_t)w.cnt * inner; item += kThreads) {
        const int i = (int)(item / inner), e = (int)(item - (int64_t)i * inner);
        const int64_t p = w.beg + i;
        const int64_t r = VTX_CHECK_SUMMARY_ROW(indices[p]);
        if (SAVE) paged[r * inner + e] = ragged[p * inner + e];
        else ragged[p * inner + e] = paged[r * inner + e];
    }
}

int check(const int32_t* indptr, int eff_bs, int K, int bos, int eos, int dtype) {
    if (!indptr || eff_bs < 0 || K < 1 || bos < 0 || eos < 0) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16) return VTX_ERR_UNSUPPORTED;
    return VTX_OK;
}

}  // namespace

extern "C" int vtx_gemm_bpr(const void* q, const void* table, void* out, const int32_t* dense_kv_indptr,
                            const int32_t* dense_kv_indices, int eff_batch_size, int group_size, int table_rows,
                            int head_dim, int topk_val, int page_reserved_bos, int page_reserved_eos, int dtype,
                            void* stream) {
    int rc = check(dense_kv_indptr, eff_batch_size, topk_val, page_reserved_bos, page_reserved_eos, dtype);
    if (rc != VTX_OK) return rc;
    if (!q || !table || !out || !dense_kv_indices || group_size < 1 || table_rows < 1 || head_dim < 1)
        return VTX_ERR_INVALID_ARGUMENT;
    if (head_dim % 8 != 0) return VTX_ERR_UNSUPPORTED;
    if (eff_batch_size == 0) return VTX_OK;
    return vtx::launch(gemm_bpr_kernel, dim3(eff_batch_size), dim3(kThreads), 0, (cudaStream_t)stream,
                       (const __nv_bfloat16*)q, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, dense_kv_indptr,
                       dense_kv_indices, group_size, table_rows, head_dim, topk_val, page_reserved_bos, page_reserved_eos);
}

extern "C" int vtx_softmax_ragged(void* x, const int32_t* dense_kv_indptr, int eff_batch_size, int inner_size,
                                  int topk_val, int page_reserved_bos, int page_reserved_eos, float scale, int dtype,
                                  void* stream) {
    int rc = check(dense_kv_indptr, eff_batch_size, topk_val, page_reserved_bos, page_reserved_eos, dtype);
    if (rc != VTX_OK) return rc;
    if (!x || inner_size < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    return vtx::launch(scan_ragged_kernel<false>, dim3(eff_batch_size), dim3(kThreads), 0, (cudaStream_t)stream,
                       (__nv_bfloat16*)x, dense_kv_indptr, inner_size, topk_val, page_reserved_bos, page_reserved_eos,
                       scale, 0.f);
}

extern "C" int vtx_normalize_ragged(void* x, const int32_t* dense_kv_indptr, int eff_batch_size, int inner_size,
                                    int topk_val, int page_reserved_bos, int page_reserved_eos, float eps, int dtype,
                                    void* stream) {
    int rc = check(dense_kv_indptr, eff_batch_size, topk_val, page_reserved_bos, page_reserved_eos, dtype);
    if (rc != VTX_OK) return rc;
    if (!x || inner_size < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    return vtx::launch(scan_ragged_kernel<true>, dim3(eff_batch_size), dim3(kThreads), 0, (cudaStream_t)stream,
                       (__nv_bfloat16*)x, dense_kv_indptr, inner_size, topk_val, page_reserved_bos, page_reserved_eos,
                       1.f, eps);
}

extern "C" int vtx_reduce_ragged(const void* x, void* out, const int32_t* dense_kv_indptr, int eff_batch_size,
                                 int rows, int cols, int dim, int kind, int topk_val, int page_reserved_bos,
                                 int page_reserved_eos, int dtype, void* stream) {
    int rc = check(dense_kv_indptr, eff_batch_size, topk_val, page_reserved_bos, page_reserved_eos, dtype);
    if (rc != VTX_OK) return rc;
    if (!x || !out || rows < 1 || cols < 1 || (dim != 1 && dim != 2) || kind < 0 || kind > 4)
        return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    return vtx::launch(reduce_ragged_kernel, dim3(eff_batch_size), dim3(kThreads), 0, (cudaStream_t)stream,
                       (const __nv_bfloat16*)x, (__nv_bfloat16*)out, dense_kv_indptr, rows, cols, dim, kind, topk_val,
                       page_reserved_bos, page_reserved_eos);
}

extern "C" int vtx_binary_bpr(const void* q, const void* table, void* out, const int32_t* dense_kv_indptr,
                              const int32_t* dense_kv_indices, int eff_batch_size, int q_c, int q_d, int table_c,
                              int table_d, int op, float alpha, float beta, int x_is_ragged, int topk_val,
                              int page_reserved_bos, int page_reserved_eos, int dtype, void* stream) {
    int rc = check(dense_kv_indptr, eff_batch_size, topk_val, page_reserved_bos, page_reserved_eos, dtype);
    if (rc != VTX_OK) return rc;
    if (!q || !table || !out || !dense_kv_indices || q_c < 1 || q_d < 1 || table_c < 1 || table_d < 1 || op < 0 || op > 3)
        return VTX_ERR_INVALID_ARGUMENT;
    if ((q_c != table_c && q_c != 1 && table_c != 1) || (q_d != table_d && q_d != 1 && table_d != 1))
        return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    const float a = __bfloat162float(__float2bfloat16_rn(alpha)), b = __bfloat162float(__float2bfloat16_rn(beta));
    return vtx::launch(binary_bpr_kernel, dim3(eff_batch_size), dim3(kThreads), 0, (cudaStream_t)stream,
                       (const __nv_bfloat16*)q, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, dense_kv_indptr,
                       dense_kv_indices, q_c, q_d, table_c, table_d, op, a, b, topk_val, page_reserved_bos,
                       page_reserved_eos, x_is_ragged ? 1 : 0);
}

extern "C" int vtx_transpose_ragged(const void* x, void* out, const int32_t* dense_kv_indptr, int eff_batch_size,
                                    int rows, int cols, int topk_val, int page_reserved_bos, int page_reserved_eos,
                                    int dtype, void* stream) {
    int rc = check(dense_kv_indptr, eff_batch_size, topk_val, page_reserved_bos, page_reserved_eos, dtype);
    if (rc != VTX_OK) return rc;
    if (!x || !out || rows < 1 || cols < 1 || x == out) return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    return vtx::launch(transpose_ragged_kernel, dim3(eff_batch_size), dim3(kThreads), 0, (cudaStream_t)stream,
                       (const __nv_bfloat16*)x, (__nv_bfloat16*)out, dense_kv_indptr, rows, cols, topk_val,
                       page_reserved_bos, page_reserved_eos);
}

extern "C" int vtx_save_load_ragged(void* ragged, void* paged, const int32_t* dense_kv_indptr,
                                    const int32_t* dense_kv_indices, int eff_batch_size, int inner_size, int save,
                                    int topk_val, int page_reserved_bos, int page_reserved_eos, int dtype,
                                    void* stream) {
    int rc = check(dense_kv_indptr, eff_batch_size, topk_val, page_reserved_bos, page_reserved_eos, dtype);
    if (rc != VTX_OK) return rc;
    if (!ragged || !paged || !dense_kv_indices || inner_size < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    auto* r = (__nv_bfloat16*)ragged;
    auto* p = (__nv_bfloat16*)paged;
    cudaStream_t st = (cudaStream_t)stream;
    if (save)
        return vtx::launch(save_load_kernel<true>, dim3(eff_batch_size), dim3(kThreads), 0, st, r, p, dense_kv_indptr,
                           dense_kv_indices, inner_size, topk_val, page_reserved_bos, page_reserved_eos);
    return vtx::launch(save_load_kernel<false>, dim3(eff_batch_size), dim3(kThreads), 0, st, r, p, dense_kv_indptr,
                       dense_kv_indices, inner_size, topk_val, page_reserved_bos, page_reserved_eos);
}
