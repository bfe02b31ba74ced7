// Paged grouped-query decode attention over each segment's page list.
//
// One CTA (4 warps) per (request, head) segment; warps take the listed pages round-robin.
// A (page, head) block of K or V is one contiguous run of page_size * D elements.  Every warp
// runs its own asynchronous pipeline: K and V tiles of up to 16 token rows are copied
// global -> shared with 16-byte cp.async (no register staging), three ring slots per warp, two
// tiles in flight while one is consumed; only warp-level synchronisation in the main loop.
// At the Qwen3 shapes a slot is 4 KB, a CTA holds 48 KB, four CTAs share an SM, so a batch of
// 64 requests x 8 KV heads is resident in one wave with ~128 KB in flight per SM.
// LPT lanes cover one token row (each lane owns 8 head dims); softmax is the online
// (running max / running sum) form in fp32; warps are merged through shared memory at the end.
// The last listed page contributes kv_last_page_len tokens; rows beyond it are zero-filled in
// shared memory and masked.
//
// Data contract as produced by the block-table builder (reference: csrc/utils_sglang.cu:123-184,
// indexer/context.py:117-121); in the reference the attention itself is a third-party
// paged-decode call made with effective batch bs*H_kv, one KV head and group_size q heads.
#include <mutex>

#include "decode_mma_body.cuh"
#include "vtx_common.cuh"

namespace {

using vtxdec::DecodeArgs;
using vtx::cp_async16;
using vtx::cp_async_commit;
using vtx::cp_async_wait;

constexpr int kWarps = 4;
constexpr int kSlots = 3;        // ring slots per warp
constexpr int kTileTokens = 16;  // token rows per tile
constexpr float kLog2e = 1.4426950408889634f;

template <typename T>
__device__ __forceinline__ void store_out(T* p, float v);
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }


// Eight elements of a shared-memory row widened to fp32.
template <typename T>
__device__ __forceinline__ void lds8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void lds8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    f[0] = vtx::bf16lo(r.x); f[1] = vtx::bf16hi(r.x);
    f[2] = vtx::bf16lo(r.y); f[3] = vtx::bf16hi(r.y);
    f[4] = vtx::bf16lo(r.z); f[5] = vtx::bf16hi(r.z);
    f[6] = vtx::bf16lo(r.w); f[7] = vtx::bf16hi(r.w);
}
template <>
__device__ __forceinline__ void lds8<float>(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// LPT lanes per token row (D = 8 * LPT).
template <typename T, int G, int LPT>
__global__ void __launch_bounds__(kWarps * 32, (G >= 8 ? 2 : 4)) decode_gqa_simt_kernel(DecodeArgs a) {
    constexpr int D = LPT * 8;
    constexpr int TPW = 32 / LPT;                 // token rows covered by one warp-wide access
    constexpr int UT = kTileTokens / TPW;         // row steps per tile
    constexpr int TILE_ELEMS = kTileTokens * D;
    constexpr int CHUNKS = TILE_ELEMS * (int)sizeof(T) / 16;  // 16-byte chunks per tile
    constexpr int CH_PER_ROW = D * (int)sizeof(T) / 16;
    constexpr int CPL = CHUNKS / 32;              // chunks copied per lane per tile
    static_assert(CHUNKS % 32 == 0, "tile must split evenly over a warp");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    T* ring = reinterpret_cast<T*>(smem_raw);

    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int s = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPT, tg = lane / LPT;
    const int beg = a.indptr[s];
    const int npages = a.indptr[s + 1] - beg;
    const int last_len = a.last_len[s];
    const int P = a.P;
    const int tiles_per_page = (P + kTileTokens - 1) / kTileTokens;
    const bool tpp_pow2 = (tiles_per_page & (tiles_per_page - 1)) == 0;  // then the page of a pair is a shift
    const int tpp_shift = 31 - __clz(tiles_per_page);
    auto page_of = [&](int pair) { return tpp_pow2 ? (pair >> tpp_shift) : pair / tiles_per_page; };

    T* my_ring = ring + (size_t)warp * kSlots * TILE_ELEMS;
    const uint32_t my_ring_addr = (uint32_t)__cvta_generic_to_shared(my_ring);

    float qf[G][8];
    {
        const T* qs = reinterpret_cast<const T*>(a.q) + (int64_t)s * G * D + sub * 8;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            vtx::Vec8<T> v;
            v.load_cached(qs + g * D);
            v.unpack(qf[g]);
#pragma unroll
            for (int j = 0; j < 8; ++j) qf[g][j] *= a.scale_log2;
        }
    }
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
    }

    // This warp's pages: warp, warp + kWarps, ...; items alternate K tile, V tile.
    const int my_pages = npages > warp ? (npages - warp + kWarps - 1) / kWarps : 0;
    const int n_items = my_pages * tiles_per_page * 2;
    const T* kc = reinterpret_cast<const T*>(a.k);
    const T* vc = reinterpret_cast<const T*>(a.v);

    // Row ids of up to 32 of this warp's pages live in one register per lane.
    int id_base = 0;
    int id_reg = (lane < my_pages) ? VTX_CHECK_KV_ROW(a.indices[beg + warp + kWarps * lane]) : 0;

    auto issue = [&](int item) {
        // item -> (page ordinal, tile, K or V)
        const int pair = item >> 1;
        const int po = page_of(pair), tile = pair - po * tiles_per_page;
        const int row = __shfl_sync(0xffffffffu, id_reg, (po - id_base) & 31);
        const int pg = warp + kWarps * po;
        const int nvalid_page = (pg == npages - 1) ? last_len : P;
        const int tok0 = tile * kTileTokens;
        const T* src = ((item & 1) ? vc : kc) + ((int64_t)row * P + tok0) * D;
        const uint32_t dst = my_ring_addr + (uint32_t)((item % kSlots) * TILE_ELEMS * sizeof(T));
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
            const int ch = c * 32 + lane;
            const int t = ch / CH_PER_ROW;
            cp_async16(dst + ch * 16, reinterpret_cast<const unsigned char*>(src) + (size_t)ch * 16,
                       tok0 + t < nvalid_page);
        }
    };

    // prologue: two items in flight
#pragma unroll
    for (int i = 0; i < kSlots - 1; ++i) {
        if (i < n_items) issue(i);
        cp_async_commit();
    }

    float sc[UT][G];
    for (int item = 0; item < n_items; ++item) {
        cp_async_wait<kSlots - 2>();  // item `item` has landed (this lane's part)
        __syncwarp();                 // ... and every lane's part; also: all lanes are done with the slot refilled next
        {
            const int nxt = item + kSlots - 1;
            if (nxt < n_items) {
                const int po = page_of(nxt >> 1);
                if (po - id_base >= 32) {  // refill the per-lane page ids (warp-uniform branch)
                    id_base += 32;
                    id_reg = (id_base + lane < my_pages) ? VTX_CHECK_KV_ROW(a.indices[beg + warp + kWarps * (id_base + lane)]) : 0;
                }
                issue(nxt);
            }
            cp_async_commit();
        }
        const T* tile_ptr = my_ring + (size_t)(item % kSlots) * TILE_ELEMS + sub * 8;
        const int pair = item >> 1;
        const int po = page_of(pair), tile = pair - po * tiles_per_page;
        const int pg = warp + kWarps * po;
        const int nvalid = ((pg == npages - 1) ? last_len : P) - tile * kTileTokens;  // valid rows in this tile
        if ((item & 1) == 0) {
            // ---- K tile: scores, running max, probabilities
#pragma unroll
            for (int u = 0; u < UT; ++u) {
                float f[8];
                lds8<T>(tile_ptr + (u * TPW + tg) * D, f);
                const bool valid = (u * TPW + tg) < nvalid;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float d = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) d = fmaf(qf[g][j], f[j], d);
#pragma unroll
                    for (int w = LPT / 2; w > 0; w >>= 1) d += __shfl_xor_sync(0xffffffffu, d, w);
                    sc[u][g] = valid ? d : -INFINITY;
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float cmax = sc[0][g];
#pragma unroll
                for (int u = 1; u < UT; ++u) cmax = fmaxf(cmax, sc[u][g]);
#pragma unroll
                for (int w = LPT; w < 32; w <<= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, w));
                const float mn = fmaxf(m[g], cmax);
                // a tile always holds at least one valid row, so mn is finite
                const float alpha = exp2f(m[g] - mn);
                m[g] = mn;
                l[g] *= alpha;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[g][j] *= alpha;
#pragma unroll
                for (int u = 0; u < UT; ++u) {
                    const float p = exp2f(sc[u][g] - mn);
                    l[g] += p;
                    sc[u][g] = p;
                }
            }
        } else {
            // ---- V tile: weighted accumulation (rows past the valid range are zero-filled, p = 0)
#pragma unroll
            for (int u = 0; u < UT; ++u) {
                float f[8];
                lds8<T>(tile_ptr + (u * TPW + tg) * D, f);
#pragma unroll
                for (int g = 0; g < G; ++g) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(sc[u][g], f[j], acc[g][j]);
                }
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its ring: reuse the space for the merge

    float* sm_acc = reinterpret_cast<float*>(smem_raw);           // [kWarps][G][D]
    float* sm_m = sm_acc + kWarps * G * D;                        // [kWarps][G]
    float* sm_l = sm_m + kWarps * G;                              // [kWarps][G]
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int w = LPT; w < 32; w <<= 1) {
            l[g] += __shfl_xor_sync(0xffffffffu, l[g], w);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[g][j] += __shfl_xor_sync(0xffffffffu, acc[g][j], w);
        }
        if (tg == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) sm_acc[(warp * G + g) * D + sub * 8 + j] = acc[g][j];
            if (sub == 0) {
                sm_m[warp * G + g] = m[g];
                sm_l[warp * G + g] = l[g];
            }
        }
    }
    __syncthreads();
    T* out = reinterpret_cast<T*>(a.out) + (int64_t)s * G * D;
    for (int idx = threadIdx.x; idx < G * D; idx += kWarps * 32) {
        const int g = idx / D, d = idx % D;
        float mx = sm_m[g];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) mx = fmaxf(mx, sm_m[w * G + g]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float wm = sm_m[w * G + g];
            const float wgt = (wm == -INFINITY) ? 0.f : exp2f(wm - mx);
            num = fmaf(wgt, sm_acc[(w * G + g) * D + d], num);
            den = fmaf(wgt, sm_l[w * G + g], den);
        }
        store_out<T>(out + idx, den > 0.f ? num / den : 0.f);
    }
}


// ---------------------------------------------------------------------------------------------
// bf16 path on the tensor cores (mma.sync m16n8k16, fp32 accumulate).
//
// The CUDA-core form above needs ~700 issue slots per 8 KB of K+V, which at one SM's share of HBM
// bandwidth keeps the schedulers ~70 % busy at 25 % occupancy; the MMA form needs ~150.
// Per 16-token tile and warp:
//   S^T[head, token] = q . K^T     A = q (16 rows, rows >= G are zero, held in registers),
//                                  B = K tile straight from shared memory via ldmatrix
//   O^T[dim, head]  += V^T . P^T   A = V tile via ldmatrix.trans, B = P^T, which is exactly the
//                                  accumulator layout of S^T (no data movement between the two)
// Rows of a tile are 16-byte-chunk swizzled (chunk ^ (row & 7)) so ldmatrix is conflict-free.

// D = head dim (64 or 128); G <= 8 query heads per KV head.
template <int G, int D>
__global__ void __launch_bounds__(kWarps * 32, 4) decode_gqa_mma_kernel(DecodeArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    vtxdec::decode_mma_body<G, D>(a, smem_raw, blockIdx.x);
}

// ---- split-KV: the page list of a segment is cut into num_splits parts, one CTA each; the parts'
// states go to a caller-provided workspace and a second kernel merges them.  For batches that do not
// fill the GPU with one CTA per segment (few requests, long dense lists).
template <int G, int D>
__global__ void __launch_bounds__(kWarps * 32, 4) decode_gqa_split_kernel(DecodeArgs a, float* workspace,
                                                                         int num_splits) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int s = blockIdx.x, sp = blockIdx.y;
    const int npages = a.indptr[s + 1] - a.indptr[s];
    const int chunk = (npages + num_splits - 1) / num_splits;
    const int lo = min(sp * chunk, npages);
    const int cnt = min(chunk, npages - lo);
    vtxdec::decode_mma_body<G, D>(a, smem_raw, s, lo, cnt,
                                  workspace + ((size_t)s * num_splits + sp) * G * (D + 2));
}

template <int G, int D>
__global__ void __launch_bounds__(128) decode_gqa_merge_kernel(const float* __restrict__ workspace,
                                                              __nv_bfloat16* __restrict__ out, int num_splits) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int s = blockIdx.x;
    const float* ws = workspace + (size_t)s * num_splits * G * (D + 2);
    for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
        const int g = idx / D, d = idx % D;
        float mx = -INFINITY;
        for (int sp = 0; sp < num_splits; ++sp) mx = fmaxf(mx, ws[(sp * G + g) * (D + 2) + D]);
        float num = 0.f, den = 0.f;
        for (int sp = 0; sp < num_splits; ++sp) {
            const float* p = ws + (sp * G + g) * (D + 2);
            const float w = p[D] == -INFINITY ? 0.f : exp2f(p[D] - mx);
            num = fmaf(w, p[d], num);
            den = fmaf(w, p[D + 1], den);
        }
        out[(size_t)s * G * D + idx] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    }
}

template <int G, int D>
int launch_split_cfg(const DecodeArgs& a, int eff_bs, int num_splits, float* workspace, cudaStream_t st) {
    const size_t bytes = vtxdec::decode_mma_smem_bytes<G, D>();
    auto kern = decode_gqa_split_kernel<G, D>;
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) {
            vtx::note_cuda_error(e);
            return VTX_ERR_CUDA;
        }
    }
    int rc = vtx::launch(kern, dim3(eff_bs, num_splits), dim3(kWarps * 32), bytes, st, a, workspace, num_splits);
    if (rc != VTX_OK) return rc;
    return vtx::launch(decode_gqa_merge_kernel<G, D>, dim3(eff_bs), dim3(128), 0, st, (const float*)workspace,
                       (__nv_bfloat16*)a.out, num_splits);
}

int launch_split(const DecodeArgs& a, int eff_bs, int group, int head_dim, int num_splits, float* workspace,
                 cudaStream_t st) {
#define VTX_SPLIT_CASE(G_, D_) \
    if (group == G_ && head_dim == D_) return launch_split_cfg<G_, D_>(a, eff_bs, num_splits, workspace, st);
    VTX_SPLIT_CASE(1, 64) VTX_SPLIT_CASE(2, 64) VTX_SPLIT_CASE(4, 64) VTX_SPLIT_CASE(8, 64)
    VTX_SPLIT_CASE(1, 128) VTX_SPLIT_CASE(2, 128) VTX_SPLIT_CASE(4, 128) VTX_SPLIT_CASE(8, 128)
#undef VTX_SPLIT_CASE
    return VTX_ERR_UNSUPPORTED;
}

template <int G, int D>
int launch_mma_cfg(const DecodeArgs& a, int eff_bs, cudaStream_t st) {
    const size_t bytes = vtxdec::decode_mma_smem_bytes<G, D>();
    auto kern = decode_gqa_mma_kernel<G, D>;
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) {
            vtx::note_cuda_error(e);
            return VTX_ERR_CUDA;
        }
    }
    return vtx::launch(kern, dim3(eff_bs), dim3(kWarps * 32), bytes, st, a);
}

template <int G>
int launch_mma_g(const DecodeArgs& a, int eff_bs, int head_dim, cudaStream_t st) {
    switch (head_dim) {
        case 64: return launch_mma_cfg<G, 64>(a, eff_bs, st);
        case 128: return launch_mma_cfg<G, 128>(a, eff_bs, st);
        default: return VTX_ERR_UNSUPPORTED;
    }
}

int launch_mma(const DecodeArgs& a, int eff_bs, int group, int head_dim, cudaStream_t st) {
    switch (group) {
        case 1: return launch_mma_g<1>(a, eff_bs, head_dim, st);
        case 2: return launch_mma_g<2>(a, eff_bs, head_dim, st);
        case 4: return launch_mma_g<4>(a, eff_bs, head_dim, st);
        case 8: return launch_mma_g<8>(a, eff_bs, head_dim, st);
        default: return VTX_ERR_UNSUPPORTED;
    }
}

template <typename T, int G, int LPT>
int launch_cfg(const DecodeArgs& a, int eff_bs, cudaStream_t st) {
    constexpr int D = LPT * 8;
    const size_t ring = (size_t)kWarps * kSlots * kTileTokens * D * sizeof(T);
    const size_t merge = (size_t)(kWarps * G * D + 2 * kWarps * G) * sizeof(float);
    const size_t bytes = ring > merge ? ring : merge;
    auto kern = decode_gqa_simt_kernel<T, G, LPT>;
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) {
            vtx::note_cuda_error(e);
            return VTX_ERR_CUDA;
        }
    }
    return vtx::launch(kern, dim3(eff_bs), dim3(kWarps * 32), bytes, st, a);
}

template <typename T, int G>
int launch_decode_g(const DecodeArgs& a, int eff_bs, int head_dim, cudaStream_t st) {
    switch (head_dim) {
        case 64: return launch_cfg<T, G, 8>(a, eff_bs, st);
        case 128: return launch_cfg<T, G, 16>(a, eff_bs, st);
        default: return VTX_ERR_UNSUPPORTED;
    }
}

template <typename T>
int launch_decode(const DecodeArgs& a, int eff_bs, int group, int head_dim, cudaStream_t st) {
    switch (group) {
        case 1: return launch_decode_g<T, 1>(a, eff_bs, head_dim, st);
        case 2: return launch_decode_g<T, 2>(a, eff_bs, head_dim, st);
        case 4: return launch_decode_g<T, 4>(a, eff_bs, head_dim, st);
        case 8: return launch_decode_g<T, 8>(a, eff_bs, head_dim, st);
        default: return VTX_ERR_UNSUPPORTED;
    }
}

}  // namespace

extern "C" int vtx_decode_gqa(const void* q, const void* k_cache, const void* v_cache, void* out,
                              const int32_t* kv_indptr, const int32_t* kv_indices,
                              const int32_t* kv_last_page_len, int eff_batch_size, int group_size, int head_dim,
                              int page_size, float sm_scale, int dtype, void* stream) {
    if (!q || !k_cache || !v_cache || !out || !kv_indptr || !kv_indices || !kv_last_page_len)
        return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size < 0 || group_size < 1 || head_dim < 1 || page_size < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    DecodeArgs a;
    a.q = q;
    a.k = k_cache;
    a.v = v_cache;
    a.out = out;
    a.indptr = kv_indptr;
    a.indices = kv_indices;
    a.last_len = kv_last_page_len;
    a.P = page_size;
    a.scale_log2 = sm_scale * kLog2e;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == VTX_BF16) return launch_mma(a, eff_batch_size, group_size, head_dim, st);
    if (dtype == VTX_F32) return launch_decode<float>(a, eff_batch_size, group_size, head_dim, st);
    return VTX_ERR_INVALID_ARGUMENT;
}

// ---- split-KV decode for callers that cannot allocate device memory ----
// The parts' states live in this array, which is part of the library image: every GPU that loads the
// library carries these 8 MB until the process exits.  All calls on a device share it.
static __device__ __align__(256) float g_splitkv_static_scratch[VTX_NOALLOC_SCRATCH_BYTES / sizeof(float)];

namespace {
// In host code the array's name is only a handle for the runtime; the device address has to be asked for,
// once per device, with that device current.
std::mutex g_static_scratch_mu;
float* g_static_scratch_addr[64] = {};

int static_scratch_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        vtx::note_cuda_error(e);
        return VTX_ERR_CUDA;
    }
    if (dev < 0 || dev >= 64) return VTX_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    if (g_static_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_splitkv_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            vtx::note_cuda_error(e);
            return VTX_ERR_CUDA;
        }
        g_static_scratch_addr[dev] = static_cast<float*>(p);
    }
    *out = g_static_scratch_addr[dev];
    return VTX_OK;
}
}  // namespace

extern "C" int vtx_decode_gqa_splitkv_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                              const int32_t* kv_indptr, const int32_t* kv_indices,
                                              const int32_t* kv_last_page_len, int eff_batch_size, int group_size,
                                              int head_dim, int page_size, float sm_scale, int num_splits,
                                              int dtype, void* stream) {
    if (!q || !k_cache || !v_cache || !out || !kv_indptr || !kv_indices || !kv_last_page_len)
        return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size < 0 || group_size < 1 || head_dim < 1 || page_size < 1 || num_splits < 1 || num_splits > 65535)
        return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16) return VTX_ERR_UNSUPPORTED;
    const int64_t need = (int64_t)eff_batch_size * num_splits * group_size * (head_dim + 2) * (int64_t)sizeof(float);
    if (need > (int64_t)VTX_NOALLOC_SCRATCH_BYTES) return VTX_ERR_SCRATCH_LIMIT;
    if (eff_batch_size == 0) return VTX_OK;
    float* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != VTX_OK) return rc;
    DecodeArgs a;
    a.q = q;
    a.k = k_cache;
    a.v = v_cache;
    a.out = out;
    a.indptr = kv_indptr;
    a.indices = kv_indices;
    a.last_len = kv_last_page_len;
    a.P = page_size;
    a.scale_log2 = sm_scale * kLog2e;
    // every part writes its whole state (parts without pages write the neutral one), so nothing in the
    // shared array has to be cleared between calls
    return launch_split(a, eff_batch_size, group_size, head_dim, num_splits, scratch, (cudaStream_t)stream);
}

extern "C" int64_t vtx_decode_gqa_splitkv_workspace_bytes(int eff_batch_size, int group_size, int head_dim,
                                                          int num_splits) {
    if (eff_batch_size < 0 || group_size < 1 || head_dim < 1 || num_splits < 1) return -1;
    return (int64_t)eff_batch_size * num_splits * group_size * (head_dim + 2) * (int64_t)sizeof(float);
}

extern "C" int vtx_decode_gqa_splitkv(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      const int32_t* kv_indptr, const int32_t* kv_indices,
                                      const int32_t* kv_last_page_len, int eff_batch_size, int group_size,
                                      int head_dim, int page_size, float sm_scale, int num_splits, void* workspace,
                                      int64_t workspace_bytes, int dtype, void* stream) {
    if (!q || !k_cache || !v_cache || !out || !kv_indptr || !kv_indices || !kv_last_page_len || !workspace)
        return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size < 0 || group_size < 1 || head_dim < 1 || page_size < 1 || num_splits < 1 || num_splits > 65535)
        return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16) return VTX_ERR_UNSUPPORTED;
    if (workspace_bytes < vtx_decode_gqa_splitkv_workspace_bytes(eff_batch_size, group_size, head_dim, num_splits))
        return VTX_ERR_INVALID_ARGUMENT;
    if (eff_batch_size == 0) return VTX_OK;
    DecodeArgs a;
    a.q = q;
    a.k = k_cache;
    a.v = v_cache;
    a.out = out;
    a.indptr = kv_indptr;
    a.indices = kv_indices;
    a.last_len = kv_last_page_len;
    a.P = page_size;
    a.scale_log2 = sm_scale * kLog2e;
    return launch_split(a, eff_batch_size, group_size, head_dim, num_splits, (float*)workspace,
                        (cudaStream_t)stream);
}
