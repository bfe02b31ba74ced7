// Tensor-core body of the paged GQA decode (bf16), shared by the stand-alone decode kernel and the
// fused sparse-layer kernel.  See decode_gqa.cu for the description of the algorithm.
#pragma once

#include "vtx_common.cuh"

namespace vtxdec {

constexpr int kDecWarps = 4;
constexpr int kDecSlots = 3;        // ring slots per warp
constexpr int kDecTileTokens = 16;  // token rows per tile

struct DecodeArgs {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    const int32_t* indptr;
    const int32_t* indices;
    const int32_t* last_len;
    int P;
    float scale_log2;
};

template <int G, int D>
constexpr size_t decode_mma_smem_bytes() {
    constexpr size_t ring = (size_t)kDecWarps * kDecSlots * kDecTileTokens * D * 2;
    constexpr size_t merge = (size_t)(kDecWarps * G * D + 2 * kDecWarps * G) * sizeof(float);
    return ring > merge ? ring : merge;
}

// Order in which a whole page list of np entries is walked: the last entry first (the only page that can
// be partial, and - like the first entry - one the block-table builder fixes before any page is selected),
// then entries 0 .. np-2.  Position p of that order is taken by warp p % kDecWarps.
__device__ __forceinline__ int list_slot(int p, int np) { return p == 0 ? np - 1 : p - 1; }

// Copy of one K or V tile (kDecTileTokens token rows of page `row`, from token tok0) into a ring slot,
// rows past nvalid_page zero-filled, 16-byte chunks swizzled by (chunk ^ (row & 7)).  One warp.
template <int D>
__device__ __forceinline__ void issue_tile(const unsigned char* cache, int row, int P, int tok0, int nvalid_page,
                                           uint32_t dst, int lane) {
    constexpr int ROWB = D * 2, CH_PER_ROW = ROWB / 16, CPL = kDecTileTokens * ROWB / 16 / 32;
    const unsigned char* src = cache + ((int64_t)row * P + tok0) * ROWB;
    if constexpr (D == 128) {
        // 256-byte rows: a lane takes one 16-byte chunk of eight consecutive token rows (lanes 0-15 rows 0-7,
        // lanes 16-31 rows 8-15), so that the swizzle of its c-th row is a constant of the unrolled loop
        const int tbase = (lane >> 4) * 8, cr = lane & 15;
        const unsigned char* s0 = src + tbase * ROWB + cr * 16;
        const uint32_t d0 = dst + (uint32_t)(tbase * ROWB);
#pragma unroll
        for (int c = 0; c < 8; ++c)
            vtx::cp_async16(d0 + c * ROWB + ((cr ^ c) << 4), s0 + c * ROWB, tok0 + tbase + c < nvalid_page);
        return;
    }
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
        const int ch = c * 32 + lane;
        const int t = ch / CH_PER_ROW, cr = ch % CH_PER_ROW;
        vtx::cp_async16(dst + t * ROWB + ((cr ^ (t & 7)) << 4), src + (size_t)ch * 16, tok0 + t < nvalid_page);
    }
}

// Early start of decode_mma_body for a caller that knows the rows of the list's last entry (row_last)
// and first entry (row_first) before the rest of the list exists: warp 0 (position 0 = last entry) and
// warp 1 (position 1 = first entry) put the first K and V tiles of those pages in flight, exactly the two
// copy groups the body would otherwise start with.  have_last / have_first say which of the two rows is
// already final.  Returns true for a warp that issued (pass it on as `pre_issued`).  The caller must not
// touch the first two ring slots of warps 0 and 1, nor commit or wait for copy groups, until the body runs.
template <int G, int D>
__device__ __forceinline__ bool decode_mma_prefetch(const DecodeArgs& a, unsigned char* smem_raw, const int np,
                                                    const int last_len, const int row_last, const int row_first,
                                                    const bool have_last, const bool have_first) {
    constexpr int TILE_BYTES = kDecTileTokens * D * 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp >= 2 || np < 2) return false;
    if (warp == 0 ? !have_last : !have_first) return false;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem_raw + (size_t)warp * kDecSlots * TILE_BYTES);
    const int row = warp == 0 ? row_last : row_first;
    const int nvalid_page = warp == 0 ? last_len : a.P;
    issue_tile<D>(reinterpret_cast<const unsigned char*>(a.k), row, a.P, 0, nvalid_page, ring, lane);
    vtx::cp_async_commit();
    issue_tile<D>(reinterpret_cast<const unsigned char*>(a.v), row, a.P, 0, nvalid_page, ring + TILE_BYTES, lane);
    vtx::cp_async_commit();
    return true;
}

// Body of the bf16 tensor-core decode for segment s; smem_raw: the CTA's dynamic shared memory
// (decode_mma_smem_bytes<G, D>() bytes, 128-byte aligned).  Called by all kDecWarps * 32 threads.
// pg_lo / pg_cnt: the part of the segment's page list this CTA attends to (whole list: 0 / -1; a whole
// list is walked in the order of list_slot, a part in list order).
// partial: null -> the normalised result goes to a.out; else the CTA's un-normalised state goes to
// partial[g * (D + 2) + {0..D-1: sum of p*V, D: running max (log2 domain), D+1: sum of p}] (split-KV).
// pre_issued (warp-uniform): this warp's first two copy groups were started by decode_mma_prefetch.
template <int G, int D>
__device__ __forceinline__ void decode_mma_body(const DecodeArgs& a, unsigned char* smem_raw, const int s,
                                                const int pg_lo = 0, const int pg_cnt = -1,
                                                float* partial = nullptr, const bool pre_issued = false) {
    using T = __nv_bfloat16;
    constexpr int KSTEPS = D / 16;                 // k-steps of QK^T == 16-dim tiles of the output
    constexpr int ROWB = D * 2;                    // bytes per token row
    constexpr int TILE_BYTES = kDecTileTokens * ROWB;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tid = lane & 3;
    const int beg = a.indptr[s];
    const int npages = a.indptr[s + 1] - beg;
    const int last_len = a.last_len[s];
    const int P = a.P;
    const int tiles_per_page = (P + kDecTileTokens - 1) / kDecTileTokens;
    // page ordinal of a (K, V) pair: a division by a run-time value per item is ~20 instructions, three times per
    // item; the usual page sizes give a power of two (16 tokens: one tile per page), which is a shift
    const bool tpp_pow2 = (tiles_per_page & (tiles_per_page - 1)) == 0;
    const int tpp_shift = 31 - __clz(tiles_per_page);
    auto page_of = [&](int pair) { return tpp_pow2 ? (pair >> tpp_shift) : pair / tiles_per_page; };

    unsigned char* my_ring = smem_raw + (size_t)warp * kDecSlots * TILE_BYTES;
    const uint32_t my_ring_addr = (uint32_t)__cvta_generic_to_shared(my_ring);

    // q as the A operand: row gid (zero for gid >= G), 16 dims per k-step
    uint32_t qa[KSTEPS][2];
    {
        const uint32_t* qs = reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(a.q) +
                                                               ((int64_t)s * G + gid) * D);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            qa[ks][0] = gid < G ? qs[ks * 8 + tid] : 0u;
            qa[ks][1] = gid < G ? qs[ks * 8 + 4 + tid] : 0u;
        }
    }
    float o[KSTEPS][4];  // O^T: [16 dims of tile mt] x [8 heads]
#pragma unroll
    for (int mt = 0; mt < KSTEPS; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[mt][i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;  // running max / partial sum of head `gid`
    float a0 = 1.f, a1 = 1.f;              // pending rescale of the O^T columns this lane holds
    bool rescale = false;                  // warp-uniform: some factor of the pending rescale differs from 1
    uint32_t pb0 = 0u, pb1 = 0u;           // P^T of the current tile as the B operand

    const bool whole = pg_cnt < 0;
    const int np_local = whole ? npages : pg_cnt;
    const int my_pages = np_local > warp ? (np_local - warp + kDecWarps - 1) / kDecWarps : 0;
    const int n_items = my_pages * tiles_per_page * 2;
    const unsigned char* kc = reinterpret_cast<const unsigned char*>(a.k);
    const unsigned char* vc = reinterpret_cast<const unsigned char*>(a.v);
    // list entry of this warp's page number po
    auto entry_of = [&](int po) { return whole ? list_slot(warp + kDecWarps * po, npages) : pg_lo + warp + kDecWarps * po; };
    int id_base = 0;
    int id_reg = (lane < my_pages) ? VTX_CHECK_KV_ROW(a.indices[beg + entry_of(lane)]) : 0;

    auto issue = [&](int item) {
        const int pair = item >> 1;
        const int po = page_of(pair), tile = pair - po * tiles_per_page;
        const int row = __shfl_sync(0xffffffffu, id_reg, (po - id_base) & 31);
        const int nvalid_page = (entry_of(po) == npages - 1) ? last_len : P;
        issue_tile<D>((item & 1) ? vc : kc, row, P, tile * kDecTileTokens, nvalid_page,
                      my_ring_addr + (uint32_t)((item % kDecSlots) * TILE_BYTES), lane);
    };

    if (!pre_issued) {
#pragma unroll
        for (int i = 0; i < kDecSlots - 1; ++i) {
            if (i < n_items) issue(i);
            vtx::cp_async_commit();
        }
    }

    // ldmatrix row address of this lane inside a tile: token row and which chunk of the pair
    const int lm_t = ((lane >> 4) << 3) + (lane & 7);
    const int lm_c = (lane >> 3) & 1;

    for (int item = 0; item < n_items; ++item) {
        vtx::cp_async_wait<kDecSlots - 2>();
        __syncwarp();
        {
            const int nxt = item + kDecSlots - 1;
            if (nxt < n_items) {
                const int po = page_of(nxt >> 1);
                if (po - id_base >= 32) {
                    id_base += 32;
                    id_reg = (id_base + lane < my_pages) ? VTX_CHECK_KV_ROW(a.indices[beg + entry_of(id_base + lane)]) : 0;
                }
                issue(nxt);
            }
            vtx::cp_async_commit();
        }
        const uint32_t tile_addr = my_ring_addr + (uint32_t)((item % kDecSlots) * TILE_BYTES) + lm_t * ROWB;
        if ((item & 1) == 0) {
            const int pair = item >> 1;
            const int po = page_of(pair), tile = pair - po * tiles_per_page;
            const int nvalid = ((entry_of(po) == npages - 1) ? last_len : P) - tile * kDecTileTokens;
            float st[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) st[j][i] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t kb[4];
                vtx::ldmatrix_x4(kb, tile_addr + ((((ks << 1) + lm_c) ^ (lm_t & 7)) << 4));
                vtx::mma_bf16(st[0], qa[ks][0], 0u, qa[ks][1], 0u, kb[0], kb[1]);
                vtx::mma_bf16(st[1], qa[ks][0], 0u, qa[ks][1], 0u, kb[2], kb[3]);
            }
            // this lane: head gid, tokens tid*2 + {0,1} (+8 for the second n-tile)
            float sv[4];
            sv[0] = (tid * 2 < nvalid) ? st[0][0] * a.scale_log2 : -INFINITY;
            sv[1] = (tid * 2 + 1 < nvalid) ? st[0][1] * a.scale_log2 : -INFINITY;
            sv[2] = (tid * 2 + 8 < nvalid) ? st[1][0] * a.scale_log2 : -INFINITY;
            sv[3] = (tid * 2 + 9 < nvalid) ? st[1][1] * a.scale_log2 : -INFINITY;
            float tmax = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            const float mn = fmaxf(m_run, tmax);
            // mn stays -inf only while nothing valid was seen (tiles past the end of a short last page)
            const float alpha = (mn == -INFINITY) ? 1.f : exp2f(m_run - mn);
            const float base = (mn == -INFINITY) ? 0.f : mn;
            m_run = mn;
            const float p0 = exp2f(sv[0] - base), p1 = exp2f(sv[1] - base);
            const float p2 = exp2f(sv[2] - base), p3 = exp2f(sv[3] - base);
            l_run = l_run * alpha + (p0 + p1) + (p2 + p3);
            pb0 = vtx::pack_bf16x2(p0, p1);
            pb1 = vtx::pack_bf16x2(p2, p3);
            // the O^T columns of this lane are heads tid*2 and tid*2+1
            a0 = __shfl_sync(0xffffffffu, alpha, (tid * 2) << 2);
            a1 = __shfl_sync(0xffffffffu, alpha, (tid * 2 + 1) << 2);
            // once the running maxima have settled every factor is exactly 1: the rescaling below is skipped
            rescale = !__all_sync(0xffffffffu, alpha == 1.f);
        } else {
#pragma unroll
            for (int mt = 0; mt < KSTEPS; ++mt) {
                uint32_t va[4];
                vtx::ldmatrix_x4_trans(va, tile_addr + ((((mt << 1) + lm_c) ^ (lm_t & 7)) << 4));
                if (rescale) { o[mt][0] *= a0; o[mt][1] *= a1; o[mt][2] *= a0; o[mt][3] *= a1; }
                // A regs: (dims 0-7, tok 0-7), (dims 8-15, tok 0-7), (dims 0-7, tok 8-15), (dims 8-15, tok 8-15)
                vtx::mma_bf16(o[mt], va[0], va[1], va[2], va[3], pb0, pb1);
            }
        }
    }
    vtx::cp_async_wait<0>();
    __syncthreads();

    float* sm_acc = reinterpret_cast<float*>(smem_raw);  // [kDecWarps][G][D]
    float* sm_m = sm_acc + kDecWarps * G * D;               // [kDecWarps][G]
    float* sm_l = sm_m + kDecWarps * G;
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (tid == 0 && gid < G) {
        sm_m[warp * G + gid] = m_run;
        sm_l[warp * G + gid] = l_run;
    }
#pragma unroll
    for (int mt = 0; mt < KSTEPS; ++mt) {
        const int h0 = tid * 2, d0 = mt * 16 + gid;
        if (h0 < G) {
            sm_acc[(warp * G + h0) * D + d0] = o[mt][0];
            sm_acc[(warp * G + h0) * D + d0 + 8] = o[mt][2];
        }
        if (h0 + 1 < G) {
            sm_acc[(warp * G + h0 + 1) * D + d0] = o[mt][1];
            sm_acc[(warp * G + h0 + 1) * D + d0 + 8] = o[mt][3];
        }
    }
    __syncthreads();
    T* out = reinterpret_cast<T*>(a.out) + (int64_t)s * G * D;
    for (int idx = threadIdx.x; idx < G * D; idx += kDecWarps * 32) {
        const int g = idx / D, d = idx % D;
        float mx = sm_m[g];
#pragma unroll
        for (int w = 1; w < kDecWarps; ++w) mx = fmaxf(mx, sm_m[w * G + g]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            const float wm = sm_m[w * G + g];
            const float wgt = (wm == -INFINITY) ? 0.f : exp2f(wm - mx);
            num = fmaf(wgt, sm_acc[(w * G + g) * D + d], num);
            den = fmaf(wgt, sm_l[w * G + g], den);
        }
        if (partial == nullptr) {
            out[idx] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
        } else {
            partial[g * (D + 2) + d] = num;
            if (d == 0) {
                partial[g * (D + 2) + D] = mx;
                partial[g * (D + 2) + D + 1] = den;
            }
        }
    }
}


}  // namespace vtxdec
