// Prefill-side helpers of the attention backend: planners (page lists, query offsets, token -> request
// table) and the per-request token-major <-> head-major shuffles of q / (o, lse).
//
// Behaviour follows csrc/utils_sglang.cu of the reference: Sgl_Prefill_Plan_Indptr_Kernel :462-509,
// Sgl_Prefill_Plan_IndicesBatchTable_Kernel :511-551, the block-table planner :797-869 and the three
// chunk-wise transposes :623-695, :698-793, :872-946.  Design: as for the decode planner, one CTA per
// (request, head) recomputes the prefix sums it needs from the length arrays, so planning is one launch
// with no batch limit; the shuffles are one grid-stride copy kernel with 16-byte (or 8-byte) vectors.
#include <algorithm>

#include "vtx_common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ int2 block_sum2(int2 v, int2* smem) {
    for (int o = 16; o > 0; o >>= 1) {
        v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
        v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    int2 t = make_int2(0, 0);
    for (int w = 0; w < kThreads / 32; ++w) {
        t.x += smem[w].x;
        t.y += smem[w].y;
    }
    return t;
}

__global__ void __launch_bounds__(kThreads) prefill_plan_kernel(
    const int32_t* __restrict__ cached, const int32_t* __restrict__ input_lens, const int32_t* __restrict__ r2t,
    int64_t r2t_stride, const int64_t* __restrict__ req_indices, int32_t* __restrict__ kv_indptr,
    int32_t* __restrict__ kv_indices, int32_t* __restrict__ qo_ragged, int32_t* __restrict__ qo_paged,
    int32_t* __restrict__ last_len, uint16_t* __restrict__ batch_table, int bs, int P, int H) {
    __shared__ int2 red[kThreads / 32];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int r = blockIdx.x, h = blockIdx.y, tx = threadIdx.x;
    int2 part = make_int2(0, 0);
    for (int i = tx; i < r; i += kThreads) {
        part.x += input_lens[i];
        part.y += (cached[i] + P - 1) / P;
    }
    const int2 before = block_sum2(part, red);
    const int in_r = input_lens[r];
    const int np = (cached[r] + P - 1) / P;
    const int s = r * H + h;
    const int kv0 = H * before.y + h * np;
    if (tx == 0) {
        kv_indptr[s] = kv0;
        qo_paged[s] = H * before.x + h * in_r;
        const int rem = cached[r] % P;
        last_len[s] = rem == 0 ? P : rem;
        if (h == 0) qo_ragged[r] = before.x;
        if (r == bs - 1 && h == H - 1) {
            kv_indptr[s + 1] = kv0 + np;
            qo_paged[s + 1] = H * before.x + H * in_r;
            qo_ragged[bs] = before.x + in_r;
        }
    }
    const int32_t* toks = r2t + VTX_CHECK_REQ_ROW(req_indices[r]) * r2t_stride;
    for (int p = tx; p < np; p += kThreads) kv_indices[kv0 + p] = (VTX_CHECK_LOC(toks[(int64_t)p * P]) / P) * H + h;
    if (h == 0)
        for (int p = tx; p < in_r; p += kThreads) batch_table[before.x + p] = (uint16_t)r;
}

__global__ void __launch_bounds__(kThreads) prefill_plan_fa3_kernel(
    const int32_t* __restrict__ cached_per_seg, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ r2t,
    int64_t r2t_stride, const int64_t* __restrict__ req_indices, int32_t* __restrict__ page_table,
    int64_t pt_stride, uint16_t* __restrict__ batch_table, int P, int H) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int r = blockIdx.x, h = blockIdx.y, tx = threadIdx.x;
    const int s = r * H + h;
    const int np = (cached_per_seg[s] + P - 1) / P;
    const int32_t* toks = r2t + VTX_CHECK_REQ_ROW(req_indices[r]) * r2t_stride;
    int32_t* out = page_table + (int64_t)s * pt_stride;
    for (int p = tx; p < np; p += kThreads) out[p] = (VTX_CHECK_LOC(toks[(int64_t)p * P]) / P) * H + h;
    if (h == 0) {
        const int q_len = cu_q[s + 1] - cu_q[s];
        uint16_t* bt = batch_table + cu_q[s] / H;
        for (int p = tx; p < q_len; p += kThreads) bt[p] = (uint16_t)r;
    }
}

// Token-major [N, H, G, D] <-> per-request head-major [H][L_b][G][D] (requests packed by indptr).
// TO_HEAD_MAJOR: dst is head-major.  One thread moves one vector of VEC bytes; y (optional, fp32 per
// (token, head, g)) travels the same way in the head-major -> token-major direction.
template <typename V, bool TO_HEAD_MAJOR>
__global__ void __launch_bounds__(kThreads) chunkwise_transpose_kernel(
    const V* __restrict__ x, V* __restrict__ x_out, const float* __restrict__ y, float* __restrict__ y_out,
    const int32_t* __restrict__ indptr, const uint16_t* __restrict__ batch_table, int64_t n_tokens, int H, int G,
    int vec_per_row) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int64_t total = n_tokens * H * G * vec_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int v = (int)(i % vec_per_row);
        int64_t rest = i / vec_per_row;
        const int g = (int)(rest % G);
        rest /= G;
        const int h = (int)(rest % H);
        const int64_t tok = rest / H;
        const int b = batch_table[tok];
        const int64_t off = indptr[b], len = indptr[b + 1] - off;
        const int64_t row_tm = (tok * H + h) * G + g;                                  // token-major row
        const int64_t row_hm = off * H * G + ((int64_t)h * len + (tok - off)) * G + g;  // head-major row
        if (TO_HEAD_MAJOR) {
            x_out[row_hm * vec_per_row + v] = x[row_tm * vec_per_row + v];
        } else {
            x_out[row_tm * vec_per_row + v] = x[row_hm * vec_per_row + v];
            if (y != nullptr && v == 0) y_out[row_tm] = y[row_hm];
        }
    }
}

template <bool TO_HEAD_MAJOR>
int launch_transpose(const void* x, void* x_out, const float* y, float* y_out, const int32_t* indptr,
                     const uint16_t* batch_table, int64_t n_tokens, int H, int G, int head_dim, cudaStream_t st) {
    const int row_bytes = head_dim * 2;
    if (row_bytes % 8 != 0) return VTX_ERR_UNSUPPORTED;
    const bool wide = row_bytes % 16 == 0;
    const int vec_per_row = row_bytes / (wide ? 16 : 8);
    const int64_t total = n_tokens * H * G * vec_per_row;
    const unsigned blocks = (unsigned)std::min<int64_t>((total + kThreads - 1) / kThreads, 148 * 16);
    if (wide)
        return vtx::launch(chunkwise_transpose_kernel<uint4, TO_HEAD_MAJOR>, dim3(blocks), dim3(kThreads), 0, st,
                           (const uint4*)x, (uint4*)x_out, y, y_out, indptr, batch_table, n_tokens, H, G, vec_per_row);
    return vtx::launch(chunkwise_transpose_kernel<uint2, TO_HEAD_MAJOR>, dim3(blocks), dim3(kThreads), 0, st,
                       (const uint2*)x, (uint2*)x_out, y, y_out, indptr, batch_table, n_tokens, H, G, vec_per_row);
}

}  // namespace

extern "C" int vtx_plan_prefill(const int32_t* cached_seq_lens, const int32_t* input_seq_lens,
                                const int32_t* req_to_token, int64_t req_to_token_stride,
                                const int64_t* req_indices, int32_t* dense_kv_indptr, int32_t* dense_kv_indices,
                                int32_t* qo_indptr_ragged, int32_t* qo_indptr_paged, int32_t* kv_last_page_len,
                                uint16_t* batch_table, int batch_size, int page_size, int num_kv_heads,
                                void* stream) {
    if (!cached_seq_lens || !input_seq_lens || !req_to_token || !req_indices || !dense_kv_indptr ||
        !dense_kv_indices || !qo_indptr_ragged || !qo_indptr_paged || !kv_last_page_len || !batch_table)
        return VTX_ERR_INVALID_ARGUMENT;
    if (batch_size < 0 || page_size < 1 || num_kv_heads < 1 || req_to_token_stride < 0) return VTX_ERR_INVALID_ARGUMENT;
    if (num_kv_heads > 65535 || batch_size > 65536) return VTX_ERR_UNSUPPORTED;  // the table holds 16-bit request ids
    if (batch_size == 0) return VTX_OK;
    return vtx::launch(prefill_plan_kernel, dim3(batch_size, num_kv_heads), dim3(kThreads), 0, (cudaStream_t)stream,
                       cached_seq_lens, input_seq_lens, req_to_token, req_to_token_stride, req_indices,
                       dense_kv_indptr, dense_kv_indices, qo_indptr_ragged, qo_indptr_paged, kv_last_page_len,
                       batch_table, batch_size, page_size, num_kv_heads);
}

extern "C" int vtx_plan_prefill_fa3(const int32_t* cached_seq_lens, const int32_t* cu_seqlens_q,
                                    const int32_t* req_to_token, int64_t req_to_token_stride,
                                    const int64_t* req_indices, int32_t* page_table, int64_t page_table_stride,
                                    uint16_t* batch_table, int batch_size, int page_size, int num_kv_heads,
                                    void* stream) {
    if (!cached_seq_lens || !cu_seqlens_q || !req_to_token || !req_indices || !page_table || !batch_table)
        return VTX_ERR_INVALID_ARGUMENT;
    if (batch_size < 0 || page_size < 1 || num_kv_heads < 1 || req_to_token_stride < 0 || page_table_stride < 1)
        return VTX_ERR_INVALID_ARGUMENT;
    if (num_kv_heads > 65535 || batch_size > 65536) return VTX_ERR_UNSUPPORTED;
    if (batch_size == 0) return VTX_OK;
    return vtx::launch(prefill_plan_fa3_kernel, dim3(batch_size, num_kv_heads), dim3(kThreads), 0,
                       (cudaStream_t)stream, cached_seq_lens, cu_seqlens_q, req_to_token, req_to_token_stride,
                       req_indices, page_table, page_table_stride, batch_table, page_size, num_kv_heads);
}

extern "C" int vtx_chunkwise_nh2hn(const void* x, void* x_out, const int32_t* indptr, const uint16_t* batch_table,
                                   int64_t num_tokens, int num_kv_heads, int group_size, int head_dim,
                                   void* stream) {
    if (!x || !x_out || !indptr || !batch_table) return VTX_ERR_INVALID_ARGUMENT;
    if (num_tokens < 0 || num_kv_heads < 1 || group_size < 1 || head_dim < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (num_tokens == 0) return VTX_OK;
    return launch_transpose<true>(x, x_out, nullptr, nullptr, indptr, batch_table, num_tokens, num_kv_heads,
                                  group_size, head_dim, (cudaStream_t)stream);
}

extern "C" int vtx_chunkwise_hn2nh(const void* x, void* x_out, const float* y, float* y_out, const int32_t* indptr,
                                   const uint16_t* batch_table, int64_t num_tokens, int num_kv_heads,
                                   int group_size, int head_dim, void* stream) {
    if (!x || !x_out || !indptr || !batch_table || ((y == nullptr) != (y_out == nullptr)))
        return VTX_ERR_INVALID_ARGUMENT;
    if (num_tokens < 0 || num_kv_heads < 1 || group_size < 1 || head_dim < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (num_tokens == 0) return VTX_OK;
    return launch_transpose<false>(x, x_out, y, y_out, indptr, batch_table, num_tokens, num_kv_heads, group_size,
                                   head_dim, (cudaStream_t)stream);
}
