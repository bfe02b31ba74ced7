// Entry points of the one-launch sparse layer (see sparse_layer_kernel.cuh for the kernel).
#include "indexer_body.cuh"

namespace vtx {
int launch_sparse_layer_m0(const vtxidx::IndexerArgs&, const vtxdec::DecodeArgs&, const vtxidx::AppendArgs&, int, int, bool,
                           cudaStream_t);
int launch_sparse_layer_m2(const vtxidx::IndexerArgs&, const vtxdec::DecodeArgs&, const vtxidx::AppendArgs&, int, int, bool,
                           cudaStream_t);
int launch_sparse_layer_m3(const vtxidx::IndexerArgs&, const vtxdec::DecodeArgs&, const vtxidx::AppendArgs&, int, int, bool,
                           cudaStream_t);
}  // namespace vtx

extern "C" int64_t vtx_sparse_layer_workspace_bytes(int eff_batch_size, int max_num_pages_per_request, int topk_val,
                                                    int page_reserved_bos, int page_reserved_eos) {
    if (eff_batch_size < 0 || max_num_pages_per_request < 1 || topk_val < 1 || page_reserved_bos < 0 ||
        page_reserved_eos < 0)
        return -1;
    return split_workspace_bytes(eff_batch_size, max_num_pages_per_request, topk_val, page_reserved_bos,
                                 page_reserved_eos);
}

extern "C" int vtx_sparse_layer(const vtx_sparse_layer_params* p, void* stream) {
    if (!p) return VTX_ERR_INVALID_ARGUMENT;
    int rc = check_common(p->dense_kv_indptr, p->dense_kv_indices, p->eff_batch_size, p->topk_val,
                          p->page_reserved_bos, p->page_reserved_eos, p->max_num_pages_per_request, p->dtype);
    if (rc != VTX_OK) return rc;
    if (!p->q || !p->summary || !p->k_cache || !p->v_cache || !p->out || !p->sparse_kv_indptr ||
        !p->sparse_kv_indices || !p->kv_last_page_len)
        return VTX_ERR_INVALID_ARGUMENT;
    if (p->group_size < 1 || p->page_size < 1 || p->workspace_bytes < 0) return VTX_ERR_INVALID_ARGUMENT;
    if (p->score_mode != VTX_SCORE_MEAN_DOT && p->score_mode != VTX_SCORE_GQA_SOFTMAX && p->score_mode != VTX_SCORE_QUEST)
        return VTX_ERR_INVALID_ARGUMENT;
    if (p->score_mode == VTX_SCORE_QUEST && !p->summary2) return VTX_ERR_INVALID_ARGUMENT;
    const int appends = (p->new_k != nullptr) + (p->new_v != nullptr) + (p->loc != nullptr);
    if (appends != 0 && appends != 3) return VTX_ERR_INVALID_ARGUMENT;
    if (appends == 3 && (p->num_kv_heads < 1 || p->eff_batch_size % p->num_kv_heads != 0 || p->page_reserved_eos < 1))
        return VTX_ERR_INVALID_ARGUMENT;  // the written page must be a reserved (never scanned) one
    if (p->dtype != VTX_BF16) return VTX_ERR_UNSUPPORTED;
    if (p->eff_batch_size == 0) return VTX_OK;
    AppendArgs ap{};
    if (appends == 3) {
        ap.k_cache = (__nv_bfloat16*)const_cast<void*>(p->k_cache);
        ap.v_cache = (__nv_bfloat16*)const_cast<void*>(p->v_cache);
        ap.centroids = (__nv_bfloat16*)const_cast<void*>(p->summary);
        ap.centroids2 = (__nv_bfloat16*)const_cast<void*>(p->summary2);
        ap.new_k = (const __nv_bfloat16*)p->new_k;
        ap.new_v = (const __nv_bfloat16*)p->new_v;
        ap.loc = p->loc;
        ap.H = p->num_kv_heads;
        ap.P = p->page_size;
    }
    IndexerArgs ia{};
    ia.q = p->q;
    ia.centroids = p->summary;
    ia.centroids2 = p->summary2;
    ia.dense_indptr = p->dense_kv_indptr;
    ia.sparse_indptr = p->sparse_kv_indptr;
    ia.dense_indices = p->dense_kv_indices;
    ia.sparse_indices = p->sparse_kv_indices;
    ia.G = p->group_size;
    ia.D = p->head_dim;
    ia.K = p->topk_val;
    ia.bos = p->page_reserved_bos;
    ia.eos = p->page_reserved_eos;
    ia.key_cap = key_capacity(p->max_num_pages_per_request);
    ia.scale = p->softmax_scale;
    plan_split(ia, p->eff_batch_size, p->max_num_pages_per_request,
               p->score_mode == VTX_SCORE_GQA_SOFTMAX ? nullptr : p->workspace, p->workspace_bytes);
    vtxdec::DecodeArgs da;
    da.q = p->q;
    da.k = p->k_cache;
    da.v = p->v_cache;
    da.out = p->out;
    da.indptr = p->sparse_kv_indptr;
    da.indices = p->sparse_kv_indices;
    da.last_len = p->kv_last_page_len;
    da.P = p->page_size;
    da.scale_log2 = p->sm_scale * 1.4426950408889634f;
    cudaStream_t st = (cudaStream_t)stream;
    const bool early = (p->flags & VTX_LAYER_EARLY_PROLOGUE) != 0 && vtx::programmatic_launch_enabled();
    const int eff = p->eff_batch_size, grp = p->group_size;
    if (p->score_mode == VTX_SCORE_QUEST) return vtx::launch_sparse_layer_m3(ia, da, ap, eff, grp, early, st);
    if (p->score_mode == VTX_SCORE_GQA_SOFTMAX) return vtx::launch_sparse_layer_m2(ia, da, ap, eff, grp, early, st);
    return vtx::launch_sparse_layer_m0(ia, da, ap, eff, grp, early, st);
}

namespace {
vtx_sparse_layer_params layer_params(const void* q, const void* summary, const void* summary2, const void* k_cache,
                                     const void* v_cache, void* out, const void* new_k, const void* new_v,
                                     const int64_t* loc, int num_kv_heads, const int32_t* dense_kv_indptr,
                                     const int32_t* sparse_kv_indptr, const int32_t* dense_kv_indices,
                                     int32_t* sparse_kv_indices, const int32_t* kv_last_page_len, int eff_batch_size,
                                     int group_size, int head_dim, int page_size, int topk_val, int page_reserved_bos,
                                     int page_reserved_eos, int max_num_pages_per_request, float sm_scale, int dtype,
                                     int score_mode, float softmax_scale) {
    vtx_sparse_layer_params p{};
    p.q = q; p.summary = summary; p.summary2 = summary2; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out;
    p.new_k = new_k; p.new_v = new_v; p.loc = loc;
    p.dense_kv_indptr = dense_kv_indptr; p.sparse_kv_indptr = sparse_kv_indptr;
    p.dense_kv_indices = dense_kv_indices; p.sparse_kv_indices = sparse_kv_indices;
    p.kv_last_page_len = kv_last_page_len;
    p.eff_batch_size = eff_batch_size; p.group_size = group_size; p.head_dim = head_dim; p.page_size = page_size;
    p.num_kv_heads = num_kv_heads; p.topk_val = topk_val; p.page_reserved_bos = page_reserved_bos;
    p.page_reserved_eos = page_reserved_eos; p.max_num_pages_per_request = max_num_pages_per_request;
    p.sm_scale = sm_scale; p.softmax_scale = softmax_scale; p.score_mode = score_mode; p.dtype = dtype;
    return p;
}
}  // namespace

extern "C" int vtx_sparse_layer_fused(const void* q, const void* centroids, const void* k_cache, const void* v_cache,
                                      void* out, const void* new_k, const void* new_v, const int64_t* loc,
                                      int num_kv_heads, const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                                      const int32_t* dense_kv_indices, int32_t* sparse_kv_indices,
                                      const int32_t* kv_last_page_len, int eff_batch_size, int group_size,
                                      int head_dim, int page_size, int topk_val, int page_reserved_bos,
                                      int page_reserved_eos, int max_num_pages_per_request, float sm_scale,
                                      int dtype, void* stream) {
    const vtx_sparse_layer_params p = layer_params(
        q, centroids, nullptr, k_cache, v_cache, out, new_k, new_v, loc, num_kv_heads, dense_kv_indptr,
        sparse_kv_indptr, dense_kv_indices, sparse_kv_indices, kv_last_page_len, eff_batch_size, group_size, head_dim,
        page_size, topk_val, page_reserved_bos, page_reserved_eos, max_num_pages_per_request, sm_scale, dtype,
        VTX_SCORE_MEAN_DOT, 0.f);
    return vtx_sparse_layer(&p, stream);
}

extern "C" int vtx_sparse_layer_fused_quest(const void* q, const void* cache_max, const void* cache_min,
                                            const void* k_cache, const void* v_cache, void* out, const void* new_k,
                                            const void* new_v, const int64_t* loc, int num_kv_heads,
                                            const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                                            const int32_t* dense_kv_indices, int32_t* sparse_kv_indices,
                                            const int32_t* kv_last_page_len, int eff_batch_size, int group_size,
                                            int head_dim, int page_size, int topk_val, int page_reserved_bos,
                                            int page_reserved_eos, int max_num_pages_per_request, float sm_scale,
                                            int dtype, void* stream) {
    const vtx_sparse_layer_params p = layer_params(
        q, cache_max, cache_min, k_cache, v_cache, out, new_k, new_v, loc, num_kv_heads, dense_kv_indptr,
        sparse_kv_indptr, dense_kv_indices, sparse_kv_indices, kv_last_page_len, eff_batch_size, group_size, head_dim,
        page_size, topk_val, page_reserved_bos, page_reserved_eos, max_num_pages_per_request, sm_scale, dtype,
        VTX_SCORE_QUEST, 0.f);
    return vtx_sparse_layer(&p, stream);
}

extern "C" int vtx_sparse_layer_fused_gqa_softmax(const void* q, const void* centroids, const void* k_cache,
                                                  const void* v_cache, void* out, const void* new_k, const void* new_v,
                                                  const int64_t* loc, int num_kv_heads, const int32_t* dense_kv_indptr,
                                                  const int32_t* sparse_kv_indptr, const int32_t* dense_kv_indices,
                                                  int32_t* sparse_kv_indices, const int32_t* kv_last_page_len,
                                                  int eff_batch_size, int group_size, int head_dim, int page_size,
                                                  int topk_val, int page_reserved_bos, int page_reserved_eos,
                                                  int max_num_pages_per_request, float sm_scale, float softmax_scale,
                                                  int dtype, void* stream) {
    const vtx_sparse_layer_params p = layer_params(
        q, centroids, nullptr, k_cache, v_cache, out, new_k, new_v, loc, num_kv_heads, dense_kv_indptr,
        sparse_kv_indptr, dense_kv_indices, sparse_kv_indices, kv_last_page_len, eff_batch_size, group_size, head_dim,
        page_size, topk_val, page_reserved_bos, page_reserved_eos, max_num_pages_per_request, sm_scale, dtype,
        VTX_SCORE_GQA_SOFTMAX, softmax_scale);
    return vtx_sparse_layer(&p, stream);
}
