// The one-launch sparse layer kernel (token write + page selection + attention); instantiated per score
// mode in sparse_layer_m0.cu / _m2.cu / _m3.cu so that the modes compile in parallel.
#pragma once
#include "indexer_body.cuh"

namespace {

// What the fused layer kernel adds to the indexer body (see NoHooks for the protocol): the wait for the
// preceding launch, the new-token write by the last warp of the segment's first CTA - with the older rows of
// the page the token closes copied into that warp's spare ring slot ahead of time - and the early start of
// the decode phase under the final key merge.
template <int D, int G, int MODE>
struct LayerHooks {
    using Regs = AppendRegs;
    const IndexerArgs& ia;
    const vtxdec::DecodeArgs& da;
    const AppendArgs& ap;
    unsigned char* smem_raw;
    const int* s_pre;  // pages listed, tokens of the last page, row of the last / first list entry
    int seg, chunk_no;
    bool early;
    bool pre_issued;

    __device__ __forceinline__ bool appends(int warp) const {
        return ap.loc != nullptr && chunk_no == 0 && warp == kWarps - 1;
    }
    // the page's older rows fit the spare slot (P - 1 <= kRowsPerSlot rows of D bf16)
    __device__ __forceinline__ bool needs_spare(int warp) const { return appends(warp) && ap.P - 1 <= kRowsPerSlot; }
    __device__ __forceinline__ void issue_extra(int warp, int lane, uint32_t spare) const {
        if (!needs_spare(warp)) return;
        // loc is an input of the step that is final before the step's first launch, like the page lists
        const int64_t t = VTX_CHECK_LOC(ap.loc[seg / ap.H]);
        const vtx::PageSlot ps = vtx::page_slot(t, ap.P);
        if (ps.row != ap.P - 1) return;  // the token does not close its page: nothing to average
        const unsigned char* page = reinterpret_cast<const unsigned char*>(ap.k_cache) +
                                    (ps.page * ap.H + seg % ap.H) * (int64_t)ap.P * (D * 2);
        constexpr int pieces = D * 2 / 16;
        for (int pc = lane; pc < (ap.P - 1) * pieces; pc += 32) cp_async16(spare + pc * 16, page + (size_t)pc * 16, true);
    }
    __device__ __forceinline__ void wait() const {
        if (early) vtx::pdl_wait();
    }
    __device__ __forceinline__ Regs load(int warp, int lane) const {
        return appends(warp) ? append_load<D>(ap, seg, lane) : Regs{};
    }
    __device__ __forceinline__ void finish(int warp, int lane, const Regs& r, const unsigned char* spare) const {
        if (appends(warp)) append_finish<D, MODE == 3>(ap, seg, lane, r, needs_spare(warp) ? spare : nullptr);
    }
    __device__ __forceinline__ int pre_sort(int n_sort) {
        constexpr int kTile = vtxdec::kDecTileTokens * D * 2;
        constexpr int kFree = 2 * vtxdec::kDecSlots * kTile;  // ring space of decode warps 2 and 3
        if (2 * sort_width(n_sort) * (int)sizeof(uint32_t) > kFree) return 0;
        pre_issued = vtxdec::decode_mma_prefetch<G, D>(da, smem_raw, s_pre[0], s_pre[1], s_pre[2], s_pre[3],
                                                       ia.eos >= 1, ia.bos >= 1);
        return kFree;
    }
};

// One launch per sparse layer: page selection, then attention over the selected pages, by the same CTA.
// The decode phase of one segment overlaps the scan phase of its neighbours on the SM, so neither phase
// pays its own launch and ramp-up; the selected rows still go to the sparse page list (the decode reads
// them back after the block barrier).  bf16 only (the decode phase is the tensor-core body).
// Grid (chunks, segments): a segment with more than ia.chunk candidates is scanned by several CTAs and the
// one that arrives last merges their best keys and runs the decode phase (see IndexerArgs); the others exit.
// With a token to append (ap.loc set) the last warp of the segment's first CTA writes the new token and the
// summary of the page it closes: the page is the segment's last one, which is never a candidate (eos >= 1),
// and the decode phase reads it only after block barriers (and, across CTAs, after the arrival counter), so
// the write needs no kernel of its own.  The older rows of that page are copied into the warp's spare ring
// slot together with its first gather batches, so the warp is not behind the others when scoring starts.
// With `early` set the CTA stages its row ids, starts its first summary-row gathers and that page copy before
// it waits for the preceding launch: those reads touch only the block-table builder's outputs, `loc`, this
// layer's summary rows of non-reserved pages and K rows written by earlier steps, none of which a launch
// between the builder and this one writes.  Everything else (q, the new token, the sparse list, the scratch
// of a split segment, the output) comes after the wait.
// Every warp keeps the best keys of the rows it scores sorted in registers, so selection ends with a short
// merge by one warp; under that merge the CTA that will run the decode phase already has the K and V tiles of
// the reserved pages it knows (the list's last and first entry) in flight.
// MODE 0: scores of the block_sparse_attention flow (group mean . centroid); MODE 2: scores of the
// gqa_block_sparse_attention flow (per-head product, softmax over pages, maximum over heads) on the same
// centroid cache, so the token write is the same too; MODE 3: scores of the gqa_quest_sparse_attention flow
// from the per-page maximum and minimum caches, which the token write then maintains instead of the mean
// (twice the summary bytes per page: two CTAs per SM instead of four).
template <int D, int G, int MODE = 0>
__global__ void __launch_bounds__(kThreads, 4) sparse_layer_kernel(IndexerArgs ia, vtxdec::DecodeArgs da,
                                                                  AppendArgs ap, const int early) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    if (!early) vtx::pdl_wait();
    vtx::pdl_trigger();
    const int seg = blockIdx.x, chunk_no = blockIdx.y;
    // What the early start of the decode phase needs, all of it written by the block-table builder; fetched
    // now (off the critical path) and parked in shared memory so that it costs no registers until the sort.
    __shared__ int s_pre[4];  // pages listed, tokens of the last page, row of the last / first list entry
    if (threadIdx.x == 0) {
        const int dbeg = ia.dense_indptr[seg], dend = ia.dense_indptr[seg + 1];
        s_pre[0] = da.indptr[seg + 1] - da.indptr[seg];
        s_pre[1] = da.last_len[seg];
        s_pre[2] = dend > dbeg ? VTX_CHECK_KV_ROW(ia.dense_indices[dend - 1]) : 0;
        s_pre[3] = dend > dbeg ? VTX_CHECK_KV_ROW(ia.dense_indices[dbeg]) : 0;
    }
    LayerHooks<D, G, MODE> hooks{ia, da, ap, smem_raw, s_pre, seg, chunk_no, early != 0, false};
    // quest mode gathers two summary rows per page: four lanes per row (8-row batches) keep its ring at the size
    // of the other modes', so that four CTAs fit an SM in every mode
    const bool owner = indexer_body<__nv_bfloat16, D, MODE, LayerHooks<D, G, MODE>&, (MODE >= 2 ? G : 1), 0, 0,
                                    (MODE == 3 ? 4 : 2)>(ia, smem_raw, seg, chunk_no, hooks);
    const bool pre_issued = hooks.pre_issued;
    if (!owner) return;
    __syncthreads();  // the list is complete and visible to the CTA; rings and sort scratch are idle
    vtxdec::decode_mma_body<G, D>(da, smem_raw, seg, 0, -1, nullptr, pre_issued);
}

template <int D, int G, int MODE>
int launch_sparse_layer_cfg(const IndexerArgs& ia, const vtxdec::DecodeArgs& da, const AppendArgs& ap, int eff_bs,
                            bool early, cudaStream_t st) {
    using Gm = Geom<__nv_bfloat16, D>;
    static_assert(vtxdec::kDecWarps * 32 == kThreads, "both phases use the same CTA shape");
    constexpr int quest_slot_b = 2 * Geom<__nv_bfloat16, D, 4>::slot_bytes;
    constexpr int quest_slots = ring_slots(quest_slot_b);
    size_t bytes = MODE == 2 ? Gm::ring_bytes + (size_t)G * D * 4 +
                                   (size_t)ia.key_cap * (sizeof(uint32_t) + sizeof(int32_t) + G * sizeof(__nv_bfloat16))
                   : MODE == 3 ? (size_t)kWarps * quest_slots * quest_slot_b + (size_t)G * D * 2 +
                                     (size_t)ia.key_cap * (sizeof(uint32_t) + sizeof(int32_t))
                               : Gm::ring_bytes + (size_t)kWarps * Gm::row_bytes +
                                     (size_t)ia.key_cap * (sizeof(uint32_t) + sizeof(int32_t));
    const size_t dec = vtxdec::decode_mma_smem_bytes<G, D>();
    if (dec > bytes) bytes = dec;
    if (bytes > 227 * 1024) return VTX_ERR_UNSUPPORTED;
    auto kern = sparse_layer_kernel<D, G, MODE>;
    int rc = set_smem(kern, bytes);
    if (rc != VTX_OK) return rc;
    return vtx::launch(kern, dim3(eff_bs, ia.nch_max), dim3(kThreads), bytes, st, ia, da, ap, early ? 1 : 0);
}

template <int D, int MODE>
int launch_sparse_layer_d(const IndexerArgs& ia, const vtxdec::DecodeArgs& da, const AppendArgs& ap, int eff_bs,
                          int group, bool early, cudaStream_t st) {
    switch (group) {
        case 1: return launch_sparse_layer_cfg<D, 1, MODE>(ia, da, ap, eff_bs, early, st);
        case 2: return launch_sparse_layer_cfg<D, 2, MODE>(ia, da, ap, eff_bs, early, st);
        case 4: return launch_sparse_layer_cfg<D, 4, MODE>(ia, da, ap, eff_bs, early, st);
        case 8: return launch_sparse_layer_cfg<D, 8, MODE>(ia, da, ap, eff_bs, early, st);
        default: return VTX_ERR_UNSUPPORTED;
    }
}

}  // namespace
