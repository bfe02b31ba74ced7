// Indexer kernels: grouped-query mean, centroid GeMV and top-k page selection (stand-alone launches).
// The device code and the description of the arithmetic live in indexer_body.cuh.
#include "indexer_body.cuh"

namespace {

template <typename T, int D, int MODE>
__global__ void __launch_bounds__(kThreads, 4) indexer_kernel(IndexerArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    indexer_body<T, D, MODE>(a, smem_raw, blockIdx.x, blockIdx.y);
}

// gqa_block_sparse_attention indexer: GeMM -> Softmax over pages -> Max over heads -> top-k, one launch.
template <int D, int GQ>
__global__ void __launch_bounds__(kThreads, 4) indexer_gqa_kernel(IndexerArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    indexer_body<__nv_bfloat16, D, 2, NoHooks, GQ>(a, smem_raw, blockIdx.x, blockIdx.y);
}

// gqa_quest_sparse_attention indexer: envelope bound per head -> Max over heads -> top-k, one launch.
template <int D, int GQ>
__global__ void __launch_bounds__(kThreads, 2) indexer_quest_kernel(IndexerArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    indexer_body<__nv_bfloat16, D, 3, NoHooks, GQ>(a, smem_raw, blockIdx.x, blockIdx.y);
}

template <typename T>
__global__ void __launch_bounds__(kThreads) topk_kernel(const T* __restrict__ scores, IndexerArgs a) {
    using Key = typename KeyOf<T>::type;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // layout: [scratch for the register sort][keys][ids]
    Key* xbuf = reinterpret_cast<Key*>(smem_raw);
    const int scratch_keys = 2 * (a.key_cap < 512 ? 512 : (a.key_cap < 2048 ? a.key_cap : 2048));
    Key* keys = xbuf + scratch_keys;
    int32_t* ids = reinterpret_cast<int32_t*>(keys + a.key_cap);
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int s = blockIdx.x;
    const int beg = a.dense_indptr[s] + a.bos;
    const int c = a.dense_indptr[s + 1] - a.eos - beg;
    if (c <= a.K) return;
    const int o0 = a.sparse_indptr[s] + a.bos;
    if (c > a.key_cap) {  // more candidates than promised: flag it, keep the list well defined
        if (threadIdx.x == 0 && a.status) atomicOr(a.status, (uint32_t)VTX_STATUS_CANDIDATE_OVERFLOW);
        for (int e = threadIdx.x; e < a.K; e += kThreads) a.sparse_indices[o0 + e] = a.dense_indices[beg + e];
        return;
    }
    for (int i = threadIdx.x; i < c; i += kThreads) {
        ids[i] = a.dense_indices[beg + i];
        keys[i] = KeyOf<T>::make(load_score<T>(scores + beg + i), i);
    }
    __syncthreads();
    EmitSelection<T> emit;
    emit.to_scratch = false;
    emit.part = nullptr;
    emit.ids = ids;
    emit.out = a.sparse_indices + o0;
    emit.out_pt = nullptr;
    sort_emit<Key>(keys, c, a.K, xbuf, emit);
}

template <typename T, int D, int MODE>
int launch_indexer_cfg(const IndexerArgs& a, int eff_bs, cudaStream_t st) {
    using Gm = Geom<T, D>;
    using Key = typename KeyOf<T>::type;
    size_t bytes = Gm::ring_bytes + (size_t)q_stage_bytes<T, D, MODE, 1>();
    if (MODE == 0) bytes += (size_t)a.key_cap * (sizeof(Key) + sizeof(int32_t));
    if (bytes > 227 * 1024) return VTX_ERR_UNSUPPORTED;
    auto kern = indexer_kernel<T, D, MODE>;
    int rc = set_smem(kern, bytes);
    if (rc != VTX_OK) return rc;
    return vtx::launch(kern, dim3(eff_bs, a.nch_max), dim3(kThreads), bytes, st, a);
}

template <typename T, int MODE>
int launch_indexer(const IndexerArgs& a, int eff_bs, cudaStream_t st) {
    switch (a.D) {
        case 64: return launch_indexer_cfg<T, 64, MODE>(a, eff_bs, st);
        case 128: return launch_indexer_cfg<T, 128, MODE>(a, eff_bs, st);
        case 256: return launch_indexer_cfg<T, 256, MODE>(a, eff_bs, st);
        case 512: return launch_indexer_cfg<T, 512, MODE>(a, eff_bs, st);
        case 576: return launch_indexer_cfg<T, 576, MODE>(a, eff_bs, st);
        default: return VTX_ERR_UNSUPPORTED;
    }
}

template <typename T>
int launch_topk(const void* scores, const IndexerArgs& a, int eff_bs, cudaStream_t st) {
    using Key = typename KeyOf<T>::type;
    const int scratch_keys = 2 * (a.key_cap < 512 ? 512 : (a.key_cap < 2048 ? a.key_cap : 2048));
    const size_t bytes = (size_t)scratch_keys * sizeof(Key) + (size_t)a.key_cap * (sizeof(Key) + sizeof(int32_t));
    if (bytes > 227 * 1024) return VTX_ERR_UNSUPPORTED;
    int rc = set_smem(topk_kernel<T>, bytes);
    if (rc != VTX_OK) return rc;
    return vtx::launch(topk_kernel<T>, dim3(eff_bs), dim3(kThreads), bytes, st, (const T*)scores, a);
}

template <int D, int GQ>
int launch_indexer_gqa_cfg(const IndexerArgs& a, int eff_bs, cudaStream_t st) {
    using Gm = Geom<__nv_bfloat16, D>;
    const size_t bytes = Gm::ring_bytes + (size_t)GQ * D * 4 +
                         (size_t)a.key_cap * (sizeof(uint32_t) + sizeof(int32_t) + GQ * sizeof(__nv_bfloat16));
    if (bytes > 227 * 1024) return VTX_ERR_UNSUPPORTED;
    auto kern = indexer_gqa_kernel<D, GQ>;
    int rc = set_smem(kern, bytes);
    if (rc != VTX_OK) return rc;
    return vtx::launch(kern, dim3(eff_bs, a.nch_max), dim3(kThreads), bytes, st, a);
}

int launch_indexer_gqa(const IndexerArgs& a, int eff_bs, cudaStream_t st) {
#define VTX_GQA_CASE(D_, G_) \
    if (a.D == D_ && a.G == G_) return launch_indexer_gqa_cfg<D_, G_>(a, eff_bs, st);
    VTX_GQA_CASE(64, 1) VTX_GQA_CASE(64, 2) VTX_GQA_CASE(64, 4) VTX_GQA_CASE(64, 8)
    VTX_GQA_CASE(128, 1) VTX_GQA_CASE(128, 2) VTX_GQA_CASE(128, 4) VTX_GQA_CASE(128, 8)
#undef VTX_GQA_CASE
    return VTX_ERR_UNSUPPORTED;
}

template <int D, int GQ>
int launch_indexer_quest_cfg(const IndexerArgs& a, int eff_bs, cudaStream_t st) {
    using Gm = Geom<__nv_bfloat16, D>;
    constexpr int slot_b = 2 * Gm::slot_bytes;
    constexpr int slots = ring_slots(slot_b);
    const size_t bytes = (size_t)kWarps * slots * slot_b + (size_t)GQ * D * 2 +
                         (size_t)a.key_cap * (sizeof(uint32_t) + sizeof(int32_t));
    if (bytes > 227 * 1024) return VTX_ERR_UNSUPPORTED;
    auto kern = indexer_quest_kernel<D, GQ>;
    int rc = set_smem(kern, bytes);
    if (rc != VTX_OK) return rc;
    return vtx::launch(kern, dim3(eff_bs, a.nch_max), dim3(kThreads), bytes, st, a);
}

int launch_indexer_quest(const IndexerArgs& a, int eff_bs, cudaStream_t st) {
#define VTX_QUEST_CASE(D_, G_) \
    if (a.D == D_ && a.G == G_) return launch_indexer_quest_cfg<D_, G_>(a, eff_bs, st);
    VTX_QUEST_CASE(64, 1) VTX_QUEST_CASE(64, 2) VTX_QUEST_CASE(64, 4) VTX_QUEST_CASE(64, 8)
    VTX_QUEST_CASE(128, 1) VTX_QUEST_CASE(128, 2) VTX_QUEST_CASE(128, 4) VTX_QUEST_CASE(128, 8)
#undef VTX_QUEST_CASE
    return VTX_ERR_UNSUPPORTED;
}

}  // namespace

extern "C" int vtx_gemv(const void* q_mean, const void* centroids, void* scores,
                        const int32_t* dense_kv_indptr, const int32_t* dense_kv_indices, int eff_batch_size,
                        int head_dim, int topk_val, int page_reserved_bos, int page_reserved_eos, int dtype,
                        void* stream) {
    int rc = check_common(dense_kv_indptr, dense_kv_indices, eff_batch_size, topk_val, page_reserved_bos,
                          page_reserved_eos, 1, dtype);
    if (rc != VTX_OK) return rc;
    if (!q_mean || !centroids || !scores) return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    IndexerArgs a{};
    a.q = q_mean;
    a.centroids = centroids;
    a.scores = scores;
    a.dense_indptr = dense_kv_indptr;
    a.dense_indices = dense_kv_indices;
    a.G = 1;
    a.D = head_dim;
    a.K = topk_val;
    a.bos = page_reserved_bos;
    a.eos = page_reserved_eos;
    a.key_cap = 0;  // GeMV mode keeps no keys in shared memory
    a.status = vtx::device_status_word();
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == VTX_BF16 ? launch_indexer<__nv_bfloat16, 1>(a, eff_batch_size, st)
                             : launch_indexer<float, 1>(a, eff_batch_size, st);
}

extern "C" int vtx_topk(const void* scores, const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                        const int32_t* dense_kv_indices, int32_t* sparse_kv_indices, int eff_batch_size,
                        int topk_val, int page_reserved_bos, int page_reserved_eos,
                        int max_num_pages_per_request, int dtype, void* stream) {
    int rc = check_common(dense_kv_indptr, dense_kv_indices, eff_batch_size, topk_val, page_reserved_bos,
                          page_reserved_eos, max_num_pages_per_request, dtype);
    if (rc != VTX_OK) return rc;
    if (!scores || !sparse_kv_indptr || !sparse_kv_indices) return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    IndexerArgs a{};
    a.dense_indptr = dense_kv_indptr;
    a.sparse_indptr = sparse_kv_indptr;
    a.dense_indices = dense_kv_indices;
    a.sparse_indices = sparse_kv_indices;
    a.K = topk_val;
    a.bos = page_reserved_bos;
    a.eos = page_reserved_eos;
    a.key_cap = key_capacity(max_num_pages_per_request);
    a.status = vtx::device_status_word();
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == VTX_BF16 ? launch_topk<__nv_bfloat16>(scores, a, eff_batch_size, st)
                             : launch_topk<float>(scores, a, eff_batch_size, st);
}

extern "C" int vtx_indexer_fused(const void* q, const void* centroids, const int32_t* dense_kv_indptr,
                                 const int32_t* sparse_kv_indptr, const int32_t* dense_kv_indices,
                                 int32_t* sparse_kv_indices, int32_t* sparse_page_table,
                                 int64_t page_table_stride, int eff_batch_size, int group_size, int head_dim,
                                 int topk_val, int page_reserved_bos, int page_reserved_eos,
                                 int max_num_pages_per_request, int dtype, void* stream) {
    int rc = check_common(dense_kv_indptr, dense_kv_indices, eff_batch_size, topk_val, page_reserved_bos,
                          page_reserved_eos, max_num_pages_per_request, dtype);
    if (rc != VTX_OK) return rc;
    if (!q || !centroids || !sparse_kv_indptr || !sparse_kv_indices) return VTX_ERR_INVALID_ARGUMENT;
    if (group_size < 1 || (sparse_page_table && page_table_stride < 1)) return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    IndexerArgs a{};
    a.q = q;
    a.centroids = centroids;
    a.dense_indptr = dense_kv_indptr;
    a.sparse_indptr = sparse_kv_indptr;
    a.dense_indices = dense_kv_indices;
    a.sparse_indices = sparse_kv_indices;
    a.sparse_pt = sparse_page_table;
    a.pt_stride = page_table_stride;
    a.G = group_size;
    a.D = head_dim;
    a.K = topk_val;
    a.bos = page_reserved_bos;
    a.eos = page_reserved_eos;
    a.key_cap = key_capacity(max_num_pages_per_request);
    a.status = vtx::device_status_word();
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == VTX_BF16 ? launch_indexer<__nv_bfloat16, 0>(a, eff_batch_size, st)
                             : launch_indexer<float, 0>(a, eff_batch_size, st);
}

extern "C" int vtx_indexer_gqa_softmax_fused(const void* q, const void* centroids, const int32_t* dense_kv_indptr,
                                             const int32_t* sparse_kv_indptr, const int32_t* dense_kv_indices,
                                             int32_t* sparse_kv_indices, int32_t* sparse_page_table,
                                             int64_t page_table_stride, int eff_batch_size, int group_size,
                                             int head_dim, int topk_val, int page_reserved_bos,
                                             int page_reserved_eos, int max_num_pages_per_request,
                                             float softmax_scale, int dtype, void* stream) {
    int rc = check_common(dense_kv_indptr, dense_kv_indices, eff_batch_size, topk_val, page_reserved_bos,
                          page_reserved_eos, max_num_pages_per_request, dtype);
    if (rc != VTX_OK) return rc;
    if (!q || !centroids || !sparse_kv_indptr || !sparse_kv_indices) return VTX_ERR_INVALID_ARGUMENT;
    if (group_size < 1 || (sparse_page_table && page_table_stride < 1)) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16) return VTX_ERR_UNSUPPORTED;
    if (eff_batch_size == 0) return VTX_OK;
    IndexerArgs a{};
    a.q = q;
    a.centroids = centroids;
    a.dense_indptr = dense_kv_indptr;
    a.sparse_indptr = sparse_kv_indptr;
    a.dense_indices = dense_kv_indices;
    a.sparse_indices = sparse_kv_indices;
    a.sparse_pt = sparse_page_table;
    a.pt_stride = page_table_stride;
    a.G = group_size;
    a.D = head_dim;
    a.K = topk_val;
    a.bos = page_reserved_bos;
    a.eos = page_reserved_eos;
    a.key_cap = key_capacity(max_num_pages_per_request);
    a.scale = softmax_scale;
    a.status = vtx::device_status_word();
    return launch_indexer_gqa(a, eff_batch_size, (cudaStream_t)stream);
}

extern "C" int vtx_indexer_quest_fused(const void* q, const void* cache_max, const void* cache_min,
                                       const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                                       const int32_t* dense_kv_indices, int32_t* sparse_kv_indices,
                                       int32_t* sparse_page_table, int64_t page_table_stride, int eff_batch_size,
                                       int group_size, int head_dim, int topk_val, int page_reserved_bos,
                                       int page_reserved_eos, int max_num_pages_per_request, int dtype,
                                       void* stream) {
    int rc = check_common(dense_kv_indptr, dense_kv_indices, eff_batch_size, topk_val, page_reserved_bos,
                          page_reserved_eos, max_num_pages_per_request, dtype);
    if (rc != VTX_OK) return rc;
    if (!q || !cache_max || !cache_min || !sparse_kv_indptr || !sparse_kv_indices) return VTX_ERR_INVALID_ARGUMENT;
    if (group_size < 1 || (sparse_page_table && page_table_stride < 1)) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16) return VTX_ERR_UNSUPPORTED;
    if (eff_batch_size == 0) return VTX_OK;
    IndexerArgs a{};
    a.q = q;
    a.centroids = cache_max;
    a.centroids2 = cache_min;
    a.dense_indptr = dense_kv_indptr;
    a.sparse_indptr = sparse_kv_indptr;
    a.dense_indices = dense_kv_indices;
    a.sparse_indices = sparse_kv_indices;
    a.sparse_pt = sparse_page_table;
    a.pt_stride = page_table_stride;
    a.G = group_size;
    a.D = head_dim;
    a.K = topk_val;
    a.bos = page_reserved_bos;
    a.eos = page_reserved_eos;
    a.key_cap = key_capacity(max_num_pages_per_request);
    a.status = vtx::device_status_word();
    return launch_indexer_quest(a, eff_batch_size, (cudaStream_t)stream);
}
