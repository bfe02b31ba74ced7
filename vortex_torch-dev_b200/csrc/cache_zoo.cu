// Cache-side operators beyond the page mean: reductions in every layout, GeMM, unary and binary elementwise.
//
// All of them are page-completion operators: for every new token slot t of `loc` with (t + 1) % page_size == 0
// and every KV head h, one [rows, cols] block per operand is read and one block (or vector) is written.  An
// operand is either PAGED - its block sits at row (t / page_size) * H + h of a [num_pages * H, ...] cache - or
// RAGGED - at row i * H + h of a [num_tokens * H, ...] tensor, i being the token's index in `loc`
// (cache/triton_kernels/reduce_impl.py:119-508 of the reference spell out the four layouts of the reduction;
// its GeMM and elementwise kernels address their operands the same way).  No shipped flow uses these
// operators; they let user flows keep other per-page summaries than the mean.  One warp per (token, head)
// item, bf16 in and out, fp32 arithmetic with one rounding per output, sums in a fixed order:
//   over rows (dim 1)     sequential in ascending order from +0.0;
//   over columns (dim 2)  the canonical chunked order of the indexer (chunks of 8, min(32, pow2ceil(chunks))
//                         partial sums, folded in halves) - also the order of the GeMM's dot products.
#include <algorithm>

#include "vtx_common.cuh"

namespace {

constexpr int kThreads = 256;

struct Item {
    bool active;
    int64_t paged_row, ragged_row;
};

__device__ __forceinline__ Item item_of(const int64_t* loc, int64_t it, int H, int P) {
    const vtx::DivMod ih = vtx::divmod(it, H);
    const int64_t i = ih.q;
    const int h = ih.r;
    const int64_t t = VTX_CHECK_LOC(loc[i]);
    Item r;
    const vtx::PageSlot ps = vtx::page_slot(t, P);
    r.active = ps.row == P - 1;
    r.paged_row = ps.page * H + h;
    r.ragged_row = i * H + h;
    return r;
}

__device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float exp_canonical(float x) {
    if (x > 88.f) return __int_as_float(0x7f800000);
    if (x < -87.0f) return 0.f;
    const float k = rintf(__fmul_rn(x, 1.44269504f));
    float r = __fsub_rn(x, __fmul_rn(k, 0.693145751953125f));
    r = __fsub_rn(r, __fmul_rn(k, 1.42860677e-6f));
    float p = (float)(1.0 / 720.0);
    p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 120.0));
    p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 24.0));
    p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 6.0));
    p = __fadd_rn(__fmul_rn(p, r), 0.5f);
    p = __fadd_rn(__fmul_rn(p, r), 1.f);
    p = __fadd_rn(__fmul_rn(p, r), 1.f);
    return __fmul_rn(p, __int_as_float(((int)k + 127) << 23));
}

// canonical sum of f(j), j < n, by one thread
template <typename F>
__device__ __forceinline__ float canonical_sum(int n, F f) {
    const int nch = (n + 7) / 8;
    int L = 1;
    while (L < nch && L < 32) L <<= 1;
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

// kind: 0 mean, 1 max, 2 min, 3 l2norm
__global__ void __launch_bounds__(kThreads) cache_reduce_kernel(const __nv_bfloat16* __restrict__ x,
                                                               __nv_bfloat16* __restrict__ out,
                                                               const int64_t* __restrict__ loc, int64_t nnz, int H, int R,
                                                               int C, int P, int dim, int kind, int x_ragged,
                                                               int out_ragged) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int64_t items = nnz * H;
    for (int64_t it = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); it < items;
         it += (int64_t)gridDim.x * (kThreads / 32)) {
        const Item m = item_of(loc, it, H, P);
        if (!m.active) continue;
        const __nv_bfloat16* src = x + (x_ragged ? m.ragged_row : m.paged_row) * (int64_t)R * C;
        const int keep = dim == 1 ? C : R, len = dim == 1 ? R : C;
        __nv_bfloat16* dst = out + (out_ragged ? m.ragged_row : m.paged_row) * (int64_t)keep;
        for (int o = lane; o < keep; o += 32) {
            auto at = [&](int j) { return dim == 1 ? ld(src + (int64_t)j * C + o) : ld(src + (int64_t)o * C + j); };
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
                    r = canonical_sum(len, term);
                } else {
                    r = 0.f;
                    for (int j = 0; j < len; ++j) r = __fadd_rn(r, term(j));
                }
                r = kind == 0 ? __fdiv_rn(r, (float)len) : __fsqrt_rn(r);
            }
            dst[o] = __float2bfloat16_rn(r);
        }
    }
}

// unary op: 0 x >= alpha ? x : beta; 1 1/(1+exp(beta x+alpha)); 2 x/(1+exp(beta x+alpha)); 3 |beta x+alpha|; 4 beta x+alpha;
// 5 alpha (a fill: x is not read)
__device__ __forceinline__ float unary(int op, float x, float alpha, float beta) {
    if (op == 0) return x >= alpha ? x : beta;
    if (op == 5) return alpha;
    const float z = bf16_round(__fadd_rn(bf16_round(__fmul_rn(beta, x)), alpha));
    if (op == 1) return __fdiv_rn(1.f, __fadd_rn(1.f, exp_canonical(z)));
    if (op == 2) return __fdiv_rn(x, __fadd_rn(1.f, exp_canonical(z)));
    if (op == 3) return fabsf(z);
    return z;
}

__global__ void __launch_bounds__(kThreads) cache_elementwise_kernel(const __nv_bfloat16* __restrict__ x,
                                                                    __nv_bfloat16* __restrict__ out,
                                                                    const int64_t* __restrict__ loc, int64_t nnz, int H,
                                                                    int inner, int P, int op, float alpha, float beta,
                                                                    int x_ragged, int out_ragged) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int64_t items = nnz * H;
    for (int64_t it = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); it < items;
         it += (int64_t)gridDim.x * (kThreads / 32)) {
        const Item m = item_of(loc, it, H, P);
        if (!m.active) continue;
        const __nv_bfloat16* src = x + (x_ragged ? m.ragged_row : m.paged_row) * (int64_t)inner;
        __nv_bfloat16* dst = out + (out_ragged ? m.ragged_row : m.paged_row) * (int64_t)inner;
        for (int e = lane; e < inner; e += 32)
            dst[e] = __float2bfloat16_rn(unary(op, op == 5 ? 0.f : ld(src + e), alpha, beta));
    }
}

// binary op: 0 max, 1 min, 2 bf16(alpha x) + bf16(beta y), 3 x y; inner dims broadcast
__global__ void __launch_bounds__(kThreads) cache_binary_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ y,
                                                               __nv_bfloat16* __restrict__ out,
                                                               const int64_t* __restrict__ loc, int64_t nnz, int H, int a0,
                                                               int a1, int b0, int b1, int P, int op, float alpha,
                                                               float beta, int xy_ragged, int out_ragged) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int64_t items = nnz * H;
    const int o0 = a0 > b0 ? a0 : b0, o1 = a1 > b1 ? a1 : b1, inner = o0 * o1;
    for (int64_t it = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); it < items;
         it += (int64_t)gridDim.x * (kThreads / 32)) {
        const Item m = item_of(loc, it, H, P);
        if (!m.active) continue;
        const int64_t in_row = xy_ragged ? m.ragged_row : m.paged_row;
        const __nv_bfloat16* xs = x + in_row * a0 * a1;
        const __nv_bfloat16* ys = y + in_row * b0 * b1;
        __nv_bfloat16* dst = out + (out_ragged ? m.ragged_row : m.paged_row) * (int64_t)inner;
        for (int e = lane; e < inner; e += 32) {
            const int c = e / o1, d = e - c * o1;
            const float a = ld(xs + (a0 == 1 ? 0 : c) * a1 + (a1 == 1 ? 0 : d));
            const float b = ld(ys + (b0 == 1 ? 0 : c) * b1 + (b1 == 1 ? 0 : d));
            float o;
            if (op == 0) o = fmaxf(a, b);
            else if (op == 1) o = fminf(a, b);
            else if (op == 2) o = __fadd_rn(bf16_round(__fmul_rn(alpha, a)), bf16_round(__fmul_rn(beta, b)));
            else o = __fmul_rn(a, b);
            dst[e] = __float2bfloat16_rn(o);
        }
    }
}

// O = Y X^T per block: x [nx, k], y [ny, k] -> out [ny, nx], fp32 products and canonical sum over k
__global__ void __launch_bounds__(kThreads) cache_gemm_kernel(const __nv_bfloat16* __restrict__ x,
                                                             const __nv_bfloat16* __restrict__ y,
                                                             __nv_bfloat16* __restrict__ out,
                                                             const int64_t* __restrict__ loc, int64_t nnz, int H, int nx,
                                                             int ny, int k, int P, int xy_ragged, int out_ragged) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int64_t items = nnz * H;
    for (int64_t it = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); it < items;
         it += (int64_t)gridDim.x * (kThreads / 32)) {
        const Item m = item_of(loc, it, H, P);
        if (!m.active) continue;
        const int64_t in_row = xy_ragged ? m.ragged_row : m.paged_row;
        const __nv_bfloat16* xs = x + in_row * nx * k;
        const __nv_bfloat16* ys = y + in_row * ny * k;
        __nv_bfloat16* dst = out + (out_ragged ? m.ragged_row : m.paged_row) * (int64_t)ny * nx;
        for (int e = lane; e < ny * nx; e += 32) {
            const int yr = e / nx, xr = e - yr * nx;
            const float s = canonical_sum(k, [&](int j) { return __fmul_rn(ld(ys + (int64_t)yr * k + j), ld(xs + (int64_t)xr * k + j)); });
            dst[e] = __float2bfloat16_rn(s);
        }
    }
}

int common_check(const void* a, const void* b, const int64_t* loc, int64_t nnz, int H, int P, int dtype) {
    if (!a || !b || !loc) return VTX_ERR_INVALID_ARGUMENT;
    if (nnz < 0 || H < 1 || P < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16) return VTX_ERR_UNSUPPORTED;
    return VTX_OK;
}

unsigned grid_for(int64_t items) {
    const int64_t blocks = (items + kThreads / 32 - 1) / (kThreads / 32);
    return (unsigned)std::max<int64_t>(1, std::min<int64_t>(blocks, 148 * 16));
}

}  // namespace

extern "C" int vtx_cache_reduce(const void* x, void* out, const int64_t* loc, int64_t nnz, int num_kv_heads,
                                int rows, int cols, int page_size, int dim, int kind, int x_is_ragged,
                                int out_is_ragged, int dtype, void* stream) {
    int rc = common_check(x, out, loc, nnz, num_kv_heads, page_size, dtype);
    if (rc != VTX_OK) return rc;
    if (rows < 1 || cols < 1 || (dim != 1 && dim != 2) || kind < 0 || kind > 3) return VTX_ERR_INVALID_ARGUMENT;
    if (nnz == 0) return VTX_OK;
    return vtx::launch(cache_reduce_kernel, dim3(grid_for(nnz * num_kv_heads)), dim3(kThreads), 0, (cudaStream_t)stream,
                       (const __nv_bfloat16*)x, (__nv_bfloat16*)out, loc, nnz, num_kv_heads, rows, cols, page_size, dim,
                       kind, x_is_ragged ? 1 : 0, out_is_ragged ? 1 : 0);
}

extern "C" int vtx_cache_elementwise(const void* x, void* out, const int64_t* loc, int64_t nnz, int num_kv_heads,
                                     int inner_size, int page_size, int op, float alpha, float beta, int x_is_ragged,
                                     int out_is_ragged, int dtype, void* stream) {
    int rc = common_check(x, out, loc, nnz, num_kv_heads, page_size, dtype);
    if (rc != VTX_OK) return rc;
    if (inner_size < 1 || op < 0 || op > 5) return VTX_ERR_INVALID_ARGUMENT;
    if (nnz == 0) return VTX_OK;
    const float a = __bfloat162float(__float2bfloat16_rn(alpha)), b = __bfloat162float(__float2bfloat16_rn(beta));
    return vtx::launch(cache_elementwise_kernel, dim3(grid_for(nnz * num_kv_heads)), dim3(kThreads), 0,
                       (cudaStream_t)stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, loc, nnz, num_kv_heads,
                       inner_size, page_size, op, a, b, x_is_ragged ? 1 : 0, out_is_ragged ? 1 : 0);
}

extern "C" int vtx_cache_binary(const void* x, const void* y, void* out, const int64_t* loc, int64_t nnz,
                                int num_kv_heads, int x_c, int x_d, int y_c, int y_d, int page_size, int op, float alpha,
                                float beta, int inputs_are_ragged, int out_is_ragged, int dtype, void* stream) {
    int rc = common_check(x, out, loc, nnz, num_kv_heads, page_size, dtype);
    if (rc != VTX_OK) return rc;
    if (!y || x_c < 1 || x_d < 1 || y_c < 1 || y_d < 1 || op < 0 || op > 3) return VTX_ERR_INVALID_ARGUMENT;
    if ((x_c != y_c && x_c != 1 && y_c != 1) || (x_d != y_d && x_d != 1 && y_d != 1)) return VTX_ERR_INVALID_ARGUMENT;
    if (nnz == 0) return VTX_OK;
    const float a = __bfloat162float(__float2bfloat16_rn(alpha)), b = __bfloat162float(__float2bfloat16_rn(beta));
    return vtx::launch(cache_binary_kernel, dim3(grid_for(nnz * num_kv_heads)), dim3(kThreads), 0, (cudaStream_t)stream,
                       (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, (__nv_bfloat16*)out, loc, nnz, num_kv_heads, x_c,
                       x_d, y_c, y_d, page_size, op, a, b, inputs_are_ragged ? 1 : 0, out_is_ragged ? 1 : 0);
}

extern "C" int vtx_cache_gemm(const void* x, const void* y, void* out, const int64_t* loc, int64_t nnz,
                              int num_kv_heads, int x_rows, int y_rows, int inner_dim, int page_size,
                              int inputs_are_ragged, int out_is_ragged, int dtype, void* stream) {
    int rc = common_check(x, out, loc, nnz, num_kv_heads, page_size, dtype);
    if (rc != VTX_OK) return rc;
    if (!y || x_rows < 1 || y_rows < 1 || inner_dim < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (nnz == 0) return VTX_OK;
    return vtx::launch(cache_gemm_kernel, dim3(grid_for(nnz * num_kv_heads)), dim3(kThreads), 0, (cudaStream_t)stream,
                       (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, (__nv_bfloat16*)out, loc, nnz, num_kv_heads,
                       x_rows, y_rows, inner_dim, page_size, inputs_are_ragged ? 1 : 0, out_is_ragged ? 1 : 0);
}
