// Block-table builder for one decode step: indptr scans, dense and sparse page lists,
// last-page lengths, the workload list and (optionally) the block-table form, in one launch.
//
// Behaviour follows the reference's three-kernel planner (csrc/utils_sglang.cu:123-184,
// :188-254, :257-309) and its block-table twin (:949-1083).  Design: one CTA per
// (request, head) segment.  Instead of a single-CTA scan followed by dependent launches,
// each CTA recomputes the three prefix sums it needs (pages, sparse slots, workload chunks
// of the requests before it) straight from cached_seq_lens, which stays L2-resident, so
// there is no inter-CTA dependency and no batch-size limit.
#include "vtx_common.cuh"

namespace {

constexpr int kPlanThreads = 256;

struct PlanArgs {
    const int32_t* seq_lens;
    const int32_t* req_to_token;
    int64_t r2t_stride;
    const int64_t* req_indices;
    int32_t* dense_indptr;
    int32_t* dense_indices;
    int32_t* sparse_indptr;
    int32_t* sparse_indices;
    int32_t* last_page_len;
    int32_t* w_q;
    int32_t* w_off;
    int32_t* w_len;
    int32_t* w_num;
    int32_t* w_chunk;
    int32_t* dense_pt;
    int32_t* dense_sl;
    int32_t* sparse_pt;
    int32_t* sparse_sl;
    int64_t pt_stride;
    int bs, P, H, K, bos, eos, max_chunk;
};

__device__ __forceinline__ int3 block_sum3(int3 v, int3* smem) {
    for (int o = 16; o > 0; o >>= 1) {
        v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
        v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
        v.z += __shfl_xor_sync(0xffffffffu, v.z, o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    int3 t = make_int3(0, 0, 0);
    for (int w = 0; w < kPlanThreads / 32; ++w) {
        t.x += smem[w].x;
        t.y += smem[w].y;
        t.z += smem[w].z;
    }
    return t;
}

__device__ __forceinline__ int chunks_of(int pages, int bos, int eos, int K, int max_chunk) {
    const int w = pages - bos - eos;
    return (w > K) ? (w + max_chunk - 1) / max_chunk : 0;
}

__global__ void __launch_bounds__(kPlanThreads) plan_decode_kernel(PlanArgs a) {
    __shared__ int3 red[kPlanThreads / 32];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int r = blockIdx.x, h = blockIdx.y, tx = threadIdx.x;
    const int budget = a.K + a.bos + a.eos;

    // The segment's first kPre * kPlanThreads page entries are requested before the prefix sums below: the request
    // row and the token slots depend only on r, so their two round trips overlap the sums and the block barrier.
    constexpr int kPre = 8;
    const int seq_early = a.seq_lens[r];
    const int n_early = (seq_early + a.P - 1) / a.P;
    const int32_t* toks_early = a.req_to_token + VTX_CHECK_REQ_ROW(a.req_indices[r]) * a.r2t_stride;
    int32_t pre[kPre];
#pragma unroll
    for (int u = 0; u < kPre; ++u) {
        const int p = tx + u * kPlanThreads;
        pre[u] = p < n_early ? toks_early[(int64_t)p * a.P] : 0;
    }

    int3 part = make_int3(0, 0, 0);
    for (int i = tx; i < r; i += kPlanThreads) {
        const int n = (a.seq_lens[i] + a.P - 1) / a.P;
        part.x += n;
        part.y += min(budget, n);
        part.z += chunks_of(n, a.bos, a.eos, a.K, a.max_chunk);
    }
    const int3 before = block_sum3(part, red);

    const int seq = a.seq_lens[r];
    const int n = (seq + a.P - 1) / a.P;
    const int m = min(budget, n);
    const int nch = chunks_of(n, a.bos, a.eos, a.K, a.max_chunk);
    const int s = r * a.H + h;
    const int d0 = a.H * before.x + h * n;
    const int s0 = a.H * before.y + h * m;
    const int w0 = a.H * before.z + h * nch;
    const int rem = seq % a.P;
    const int last_len = rem == 0 ? a.P : rem;

    if (tx == 0) {
        a.dense_indptr[s] = d0;
        a.sparse_indptr[s] = s0;
        if (a.last_page_len) a.last_page_len[s] = last_len;
        if (a.dense_sl) {
            a.dense_sl[s] = seq;
            a.sparse_sl[s] = min((budget - 1) * a.P + last_len, seq);
        }
        if (r == a.bs - 1 && h == a.H - 1) {
            a.dense_indptr[s + 1] = d0 + n;
            a.sparse_indptr[s + 1] = s0 + m;
            *a.w_num = w0 + nch;
            *a.w_chunk = a.max_chunk;
        }
    }

    const int32_t* toks = a.req_to_token + VTX_CHECK_REQ_ROW(a.req_indices[r]) * a.r2t_stride;
    int32_t* dense = a.dense_indices + d0;
    int32_t* sparse = a.sparse_indices + s0;
    int32_t* dpt = a.dense_pt ? a.dense_pt + (int64_t)s * a.pt_stride : nullptr;
    int32_t* spt = a.sparse_pt ? a.sparse_pt + (int64_t)s * a.pt_stride : nullptr;
    const bool copy_all = n <= budget;

    for (int p = tx, u = 0; p < n; p += kPlanThreads, ++u) {
        int32_t tok = 0;
        if (u < kPre) {
#pragma unroll
            for (int w = 0; w < kPre; ++w)
                if (w == u) tok = pre[w];
        } else {
            tok = toks[(int64_t)p * a.P];
        }
        const int row = (VTX_CHECK_LOC(tok) / a.P) * a.H + h;
        dense[p] = row;
        if (dpt) dpt[p] = row;
        int slot = -1;
        if (copy_all) slot = p;
        else if (p < a.bos) slot = p;
        else if (p >= n - a.eos) slot = budget - (n - p);
        if (slot >= 0) {
            sparse[slot] = row;
            if (spt) spt[slot] = row;
        }
    }

    // workload chunks of this segment (consumed only by chunk-list style operators)
    const int cand = n - a.bos - a.eos;
    for (int j = tx; j < nch; j += kPlanThreads) {
        int len = cand - j * a.max_chunk;
        if (len > a.max_chunk) len = a.max_chunk;
        a.w_q[w0 + j] = s;
        a.w_len[w0 + j] = len;
        a.w_off[w0 + j] = d0 + j * a.max_chunk + a.bos;
    }
}

}  // namespace

extern "C" int vtx_plan_decode(const int32_t* cached_seq_lens, const int32_t* req_to_token,
                               int64_t req_to_token_stride, const int64_t* req_indices,
                               int32_t* dense_kv_indptr, int32_t* dense_kv_indices,
                               int32_t* sparse_kv_indptr, int32_t* sparse_kv_indices,
                               int32_t* kv_last_page_len, int32_t* winfo_q_indices,
                               int32_t* winfo_kv_offsets, int32_t* winfo_kv_lens,
                               int32_t* winfo_num_workloads, int32_t* winfo_chunk_size,
                               int32_t* dense_page_table, int32_t* dense_cache_seqlens,
                               int32_t* sparse_page_table, int32_t* sparse_cache_seqlens,
                               int64_t page_table_stride, int batch_size, int page_size,
                               int num_kv_heads, int topk_val, int page_reserved_bos,
                               int page_reserved_eos, int max_chunk_size, int min_chunk_size,
                               void* stream) {
    // the two per-request inputs are empty (and may be null) for an empty batch
    if (batch_size != 0 && (!cached_seq_lens || !req_indices)) return VTX_ERR_INVALID_ARGUMENT;
    if (!req_to_token || !dense_kv_indptr || !dense_kv_indices ||
        !sparse_kv_indptr || !sparse_kv_indices || !winfo_q_indices ||
        !winfo_kv_offsets || !winfo_kv_lens || !winfo_num_workloads || !winfo_chunk_size)
        return VTX_ERR_INVALID_ARGUMENT;
    // Same argument rules as the reference's debug checks (csrc/utils_sglang.cu:349-356).
    if (batch_size < 0 || page_size < 1 || num_kv_heads < 1 || topk_val < 1 || page_reserved_bos < 0 ||
        page_reserved_eos < 1 || min_chunk_size < 1 || max_chunk_size < 1 || req_to_token_stride < 0)
        return VTX_ERR_INVALID_ARGUMENT;
    const int tables = (dense_page_table != nullptr) + (dense_cache_seqlens != nullptr) +
                       (sparse_page_table != nullptr) + (sparse_cache_seqlens != nullptr);
    if (tables != 0 && tables != 4) return VTX_ERR_INVALID_ARGUMENT;
    if (tables == 4 && page_table_stride < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (!kv_last_page_len && tables != 4) return VTX_ERR_INVALID_ARGUMENT;  // optional only in table form
    if (num_kv_heads > 65535) return VTX_ERR_UNSUPPORTED;
    if (batch_size == 0) return VTX_OK;

    PlanArgs a;
    a.seq_lens = cached_seq_lens;
    a.req_to_token = req_to_token;
    a.r2t_stride = req_to_token_stride;
    a.req_indices = req_indices;
    a.dense_indptr = dense_kv_indptr;
    a.dense_indices = dense_kv_indices;
    a.sparse_indptr = sparse_kv_indptr;
    a.sparse_indices = sparse_kv_indices;
    a.last_page_len = kv_last_page_len;
    a.w_q = winfo_q_indices;
    a.w_off = winfo_kv_offsets;
    a.w_len = winfo_kv_lens;
    a.w_num = winfo_num_workloads;
    a.w_chunk = winfo_chunk_size;
    a.dense_pt = dense_page_table;
    a.dense_sl = dense_cache_seqlens;
    a.sparse_pt = sparse_page_table;
    a.sparse_sl = sparse_cache_seqlens;
    a.pt_stride = page_table_stride;
    a.bs = batch_size;
    a.P = page_size;
    a.H = num_kv_heads;
    a.K = topk_val;
    a.bos = page_reserved_bos;
    a.eos = page_reserved_eos;
    a.max_chunk = max_chunk_size;
    dim3 grid(batch_size, num_kv_heads);
    return vtx::launch(plan_decode_kernel, grid, dim3(kPlanThreads), 0, (cudaStream_t)stream, a);
}
