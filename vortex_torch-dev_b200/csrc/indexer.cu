// Indexer kernels: grouped-query mean, centroid GeMV and top-k page selection.
//
// One CTA (4 warps) per (request, head) segment.  The fused kernel keeps the segment's scores in
// shared memory as sortable keys, so they never travel to HBM; the stand-alone GeMV and top-k
// kernels exist for flows that call the operators one by one and produce the same bits.
// Behaviour follows flow/algorithms.py:168-170, indexer/triton_kernels/mv_impl.py:53-62 and
// csrc/topk.cu:56-113 of the reference.
//
// Canonical score arithmetic (shared with the CPU checker, so selections are bit-exact):
//   q_mean[d] = round_T( (q[0][d] + q[1][d] + ... in fp32, from +0.0) / G )
//   product   = round_T( centroid[d] * q_mean[d] )          (one rounding of the exact product)
//   the D dims are cut in chunks of 8; L = min(32, pow2ceil(D/8)) partial sums; partial l adds the
//   products of chunks l, l+L, ... one by one in ascending order into an fp32 accumulator
//   starting at +0.0 (no FMA); partials are folded v[i] += v[i+w], w = L/2 .. 1;
//   score = round_T(sum).
// Selection order: score descending, ties by ascending candidate position (a stable
// descending sort), -0.0 equal to +0.0.
//
// Data movement: centroid rows are gathered global -> shared with 16-byte cp.async into a ring
// per warp (16 rows per slot, two slots in flight while one is scored), so no registers stage
// the loads and the only block-wide barriers are before and after the gather.  Two threads
// score one row: the thread of parity p owns the partial sums of parity p, which keeps every
// fold level but the last inside a thread (one shuffle per row).  Rows are stored with their
// 16-byte pieces swizzled (piece ^ 2*(row & 3)) so the 128-bit shared loads are conflict-free.
// The sort is a bitonic network over registers (4..16 keys per thread): strides below the
// per-thread block are register swaps, strides inside a warp are shuffles, and only the three
// widest strides cross warps through shared memory.
#include "decode_mma_body.cuh"
#include "vtx_common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxCandidates = 16384;
constexpr int kRowsPerSlot = 16;

// ---- sortable keys: high bits order the score, low bits make lower positions win ties ----
template <typename T>
struct KeyOf;

template <>
struct KeyOf<__nv_bfloat16> {
    using type = uint32_t;
    static __device__ __forceinline__ type make(float v, int i) {
        uint32_t b = __float_as_uint(v) >> 16;  // v is bf16-representable
        if (b == 0x8000u) b = 0u;               // -0.0 sorts as +0.0
        const uint32_t ord = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
        return (ord << 16) | (0xffffu - (uint32_t)i);
    }
    static __device__ __forceinline__ int index(type k) { return (int)(0xffffu - (k & 0xffffu)); }
};

template <>
struct KeyOf<float> {
    using type = unsigned long long;
    static __device__ __forceinline__ type make(float v, int i) {
        uint32_t b = __float_as_uint(v);
        if (b == 0x80000000u) b = 0u;
        const uint32_t ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
        return ((type)ord << 32) | (type)(0xffffffffu - (uint32_t)i);
    }
    static __device__ __forceinline__ int index(type k) { return (int)(0xffffffffu - (uint32_t)(k & 0xffffffffull)); }
};

// Descending bitonic sort of n (power of two) keys in shared memory by the whole CTA
// (general fallback for segments with more than 2048 candidates).
template <typename Key>
__device__ void block_bitonic_desc(Key* keys, int n) {
    for (int k = 2; k <= n; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < (n >> 1); i += kThreads) {
                const int a = 2 * i - (i & (j - 1));
                const int b = a + j;
                const Key ka = keys[a], kb = keys[b];
                const bool desc = (a & k) == 0;
                if ((ka < kb) == desc) {
                    keys[a] = kb;
                    keys[b] = ka;
                }
            }
            __syncthreads();
        }
    }
}

// Descending bitonic sort of kThreads * EPT keys held EPT per thread, element e = thread * EPT + r.
// xbuf: shared scratch of 2 * kThreads * EPT keys for the strides that cross warps.
template <typename Key, int EPT>
__device__ __forceinline__ void block_sort_desc_regs(Key (&v)[EPT], Key* xbuf) {
    constexpr int N = kThreads * EPT;
    const int t = threadIdx.x;
    int buf = 0;
#pragma unroll
    for (int k = 2; k <= N; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            if (j < EPT) {
#pragma unroll
                for (int r = 0; r < EPT; ++r) {
                    if ((r & j) == 0) {
                        const bool desc = (((t * EPT + r) & k) == 0);
                        const Key x = v[r], y = v[r + j];
                        const bool sw = (x < y) == desc;
                        v[r] = sw ? y : x;
                        v[r + j] = sw ? x : y;
                    }
                }
            } else {
                const int pt = j / EPT;                    // partner thread = t ^ pt
                const bool lower = (t & pt) == 0;
                const bool desc = (((t * EPT) & k) == 0);  // k > j >= EPT: bit k of e comes from t
                const bool keep_max = lower == desc;
                if (pt < 32) {
#pragma unroll
                    for (int r = 0; r < EPT; ++r) {
                        const Key o = __shfl_xor_sync(0xffffffffu, v[r], pt);
                        v[r] = keep_max ? (v[r] > o ? v[r] : o) : (v[r] < o ? v[r] : o);
                    }
                } else {
                    Key* mine = xbuf + buf * N + t * EPT;
                    const Key* theirs = xbuf + buf * N + (t ^ pt) * EPT;
#pragma unroll
                    for (int r = 0; r < EPT; ++r) mine[r] = v[r];
                    __syncthreads();
#pragma unroll
                    for (int r = 0; r < EPT; ++r) {
                        const Key o = theirs[r];
                        v[r] = keep_max ? (v[r] > o ? v[r] : o) : (v[r] < o ? v[r] : o);
                    }
                    buf ^= 1;
                }
            }
        }
    }
}

template <typename T, int EPT>
__device__ __forceinline__ void select_regs(const typename KeyOf<T>::type* keys, const int32_t* ids, int c, int K,
                                            int32_t* out, int32_t* out_pt, typename KeyOf<T>::type* xbuf) {
    using Key = typename KeyOf<T>::type;
    Key v[EPT];
#pragma unroll
    for (int r = 0; r < EPT; ++r) {
        const int e = threadIdx.x * EPT + r;
        v[r] = e < c ? keys[e] : (Key)0;  // real keys are never 0 for finite scores
    }
    block_sort_desc_regs<Key, EPT>(v, xbuf);
#pragma unroll
    for (int r = 0; r < EPT; ++r) {
        const int e = threadIdx.x * EPT + r;
        if (e < K) {
            const int32_t row = ids[KeyOf<T>::index(v[r])];
            out[e] = row;
            if (out_pt) out_pt[e] = row;
        }
    }
}

// Sort the c keys of a segment (already in shared memory, visible to all threads) and emit the
// first K row ids.  xbuf: shared scratch for the register sort (2 * max(512, min(pow2ceil(c), 2048))
// keys), or null to force the shared-memory network.
template <typename T>
__device__ void select_and_store(typename KeyOf<T>::type* keys, const int32_t* ids, int c, int K, int32_t* out,
                                 int32_t* out_pt, typename KeyOf<T>::type* xbuf) {
    using Key = typename KeyOf<T>::type;
    if (xbuf != nullptr && c <= kThreads * 4) return select_regs<T, 4>(keys, ids, c, K, out, out_pt, xbuf);
    if (xbuf != nullptr && c <= kThreads * 8) return select_regs<T, 8>(keys, ids, c, K, out, out_pt, xbuf);
    if (xbuf != nullptr && c <= kThreads * 16) return select_regs<T, 16>(keys, ids, c, K, out, out_pt, xbuf);
    const int n = vtx::pow2_ceil(c);
    for (int i = c + threadIdx.x; i < n; i += kThreads) keys[i] = (Key)0;
    __syncthreads();
    block_bitonic_desc<Key>(keys, n);
    for (int j = threadIdx.x; j < K; j += kThreads) {
        const int32_t row = ids[KeyOf<T>::index(keys[j])];
        out[j] = row;
        if (out_pt) out_pt[j] = row;
    }
}

template <typename T>
__device__ __forceinline__ float load_score(const T* p);
template <>
__device__ __forceinline__ float load_score<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float load_score<float>(const float* p) { return *p; }

template <typename T>
__device__ __forceinline__ void store_score(T* p, float v);
template <>
__device__ __forceinline__ void store_score<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ void store_score<float>(float* p, float v) { *p = v; }

struct IndexerArgs {
    const void* q;          // [eff_bs, G, D]
    const void* centroids;  // [rows, D]
    const void* centroids2; // MODE 3: second summary cache (per-page minimum); centroids is the maximum
    void* scores;           // packed, GEMV mode only
    const int32_t* dense_indptr;
    const int32_t* sparse_indptr;
    const int32_t* dense_indices;
    int32_t* sparse_indices;
    int32_t* sparse_pt;
    int64_t pt_stride;
    int G, D, K, bos, eos, key_cap;
    float scale;  // MODE 2: softmax scale
};

// ---- asynchronous row gather ----
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr, bool valid) {
    const int src_bytes = valid ? 16 : 0;  // 0 => zero-fill, the source is not read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- one chunk (8 dims) of products added one by one into acc ----
// bf16: the packed multiply rounds each exact product once to bf16, as the canonical order asks.
__device__ __forceinline__ void add_products(float& acc, const __nv_bfloat16* row_chunk, const __nv_bfloat16* q_chunk) {
    const uint4 r = *reinterpret_cast<const uint4*>(row_chunk);
    const uint4 q = *reinterpret_cast<const uint4*>(q_chunk);
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w}, qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 p = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&rr[i]),
                                         *reinterpret_cast<const __nv_bfloat162*>(&qq[i]));
        const uint32_t pw = *reinterpret_cast<const uint32_t*>(&p);
        acc = __fadd_rn(acc, vtx::bf16lo(pw));
        acc = __fadd_rn(acc, vtx::bf16hi(pw));
    }
}
__device__ __forceinline__ void add_products(float& acc, const float* row_chunk, const float* q_chunk) {
    const float4 r0 = *reinterpret_cast<const float4*>(row_chunk), r1 = *reinterpret_cast<const float4*>(row_chunk + 4);
    const float4 q0 = *reinterpret_cast<const float4*>(q_chunk), q1 = *reinterpret_cast<const float4*>(q_chunk + 4);
    acc = __fadd_rn(acc, __fmul_rn(r0.x, q0.x));
    acc = __fadd_rn(acc, __fmul_rn(r0.y, q0.y));
    acc = __fadd_rn(acc, __fmul_rn(r0.z, q0.z));
    acc = __fadd_rn(acc, __fmul_rn(r0.w, q0.w));
    acc = __fadd_rn(acc, __fmul_rn(r1.x, q1.x));
    acc = __fadd_rn(acc, __fmul_rn(r1.y, q1.y));
    acc = __fadd_rn(acc, __fmul_rn(r1.z, q1.z));
    acc = __fadd_rn(acc, __fmul_rn(r1.w, q1.w));
}

// bf16 row chunk times fp32 query chunk, products kept in fp32 (the GeMM operator's arithmetic).
__device__ __forceinline__ void add_products_f32(float& acc, const __nv_bfloat16* row_chunk, const float* q_chunk) {
    const uint4 r = *reinterpret_cast<const uint4*>(row_chunk);
    const float4 q0 = *reinterpret_cast<const float4*>(q_chunk), q1 = *reinterpret_cast<const float4*>(q_chunk + 4);
    acc = __fadd_rn(acc, __fmul_rn(vtx::bf16lo(r.x), q0.x));
    acc = __fadd_rn(acc, __fmul_rn(vtx::bf16hi(r.x), q0.y));
    acc = __fadd_rn(acc, __fmul_rn(vtx::bf16lo(r.y), q0.z));
    acc = __fadd_rn(acc, __fmul_rn(vtx::bf16hi(r.y), q0.w));
    acc = __fadd_rn(acc, __fmul_rn(vtx::bf16lo(r.z), q1.x));
    acc = __fadd_rn(acc, __fmul_rn(vtx::bf16hi(r.z), q1.y));
    acc = __fadd_rn(acc, __fmul_rn(vtx::bf16lo(r.w), q1.z));
    acc = __fadd_rn(acc, __fmul_rn(vtx::bf16hi(r.w), q1.w));
}

// Quest upper bound for one chunk: max(round_bf16(q*hi), round_bf16(q*lo)) per dim, added one by one.
__device__ __forceinline__ void add_quest_bounds(float& acc, const __nv_bfloat16* hi_chunk, const __nv_bfloat16* lo_chunk,
                                                 const __nv_bfloat16* q_chunk) {
    const uint4 h = *reinterpret_cast<const uint4*>(hi_chunk);
    const uint4 l = *reinterpret_cast<const uint4*>(lo_chunk);
    const uint4 q = *reinterpret_cast<const uint4*>(q_chunk);
    const uint32_t hh[4] = {h.x, h.y, h.z, h.w}, ll[4] = {l.x, l.y, l.z, l.w}, qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 qv = *reinterpret_cast<const __nv_bfloat162*>(&qq[i]);
        const __nv_bfloat162 u = __hmax2(__hmul2(*reinterpret_cast<const __nv_bfloat162*>(&hh[i]), qv),
                                         __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&ll[i]), qv));
        const uint32_t uw = *reinterpret_cast<const uint32_t*>(&u);
        acc = __fadd_rn(acc, vtx::bf16lo(uw));
        acc = __fadd_rn(acc, vtx::bf16hi(uw));
    }
}

// exp(x) for x <= 0 as a fixed sequence of fp32 operations, identical on CPU and GPU:
// k = rint(x * log2 e); r = x - k*ln2_hi - k*ln2_lo; degree-6 Taylor polynomial (Horner, separate
// multiply and add); result = p * 2^k; inputs below -87 give 0.
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

template <typename T, int D>
struct Geom {
    static constexpr int nchunk = D / 8;  // canonical chunks of 8 dims
    static constexpr int L = nchunk > 16 ? 32 : (nchunk > 8 ? 16 : (nchunk > 4 ? 8 : 4));
    static constexpr int row_bytes = D * (int)sizeof(T);
    static constexpr int pieces = row_bytes / 16;        // 16-byte pieces per row
    static constexpr int ppc = 8 * (int)sizeof(T) / 16;  // pieces per canonical chunk (1 bf16, 2 fp32)
    static constexpr int slot_bytes = kRowsPerSlot * row_bytes;
    static constexpr int slots = slot_bytes * 3 * kWarps <= 96 * 1024 ? 3 : 2;
    static constexpr size_t ring_bytes = (size_t)kWarps * slots * slot_bytes;
    static_assert(pieces % 8 == 0, "row must be a multiple of 128 bytes");
    static_assert(nchunk % 2 == 0, "two threads share a row by parity of the partial sums");
    // the idle ring doubles as the sort's exchange buffer (2 x 2048 keys at most)
    static_assert(ring_bytes >= 2 * 2048 * sizeof(typename KeyOf<T>::type), "ring too small for the sort scratch");
};

// New-token write for one segment, optional part of the fused sparse-layer kernel (all pointers null
// when unused).  Same arithmetic as set_kv_cmean_kernel in cache_ops.cu.
struct AppendArgs {
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    __nv_bfloat16* centroids;    // page mean of K; with QUEST: per-dim page maximum
    __nv_bfloat16* centroids2;   // QUEST only: per-dim page minimum
    const __nv_bfloat16* new_k;  // [bs, H, D]
    const __nv_bfloat16* new_v;
    const int64_t* loc;          // [bs]
    int H, P;
};

// Executed by one warp: lanes 0 .. D/8-1 each own 8 head dims of segment s = request * H + head.
// Writes the new token's K and V rows and, if the token closes its page, the page's mean of K
// (rows 0 .. P-2 from the cache in ascending order, the new row last, one division, one rounding).
// QUEST: the page's per-dim maximum and minimum instead (both exact in bf16), as vtx_creduce computes them.
template <int D, bool QUEST = false>
__device__ __forceinline__ void append_token(const AppendArgs& ap, const int s, const int lane) {
    constexpr int NCH = D / 8;
    if (lane >= NCH) return;
    const int r = s / ap.H, h = s - r * ap.H;
    const int64_t t = ap.loc[r];
    const int64_t pid = (t / ap.P) * ap.H + h;
    const int tok = (int)(t % ap.P);
    __nv_bfloat16* kpage = ap.k_cache + pid * (int64_t)ap.P * D;
    __nv_bfloat16* vpage = ap.v_cache + pid * (int64_t)ap.P * D;
    vtx::Vec8<__nv_bfloat16> nk, nv;
    nk.load_cached(ap.new_k + (int64_t)s * D + lane * 8);
    nv.load_cached(ap.new_v + (int64_t)s * D + lane * 8);
    *reinterpret_cast<uint4*>(kpage + (int64_t)tok * D + lane * 8) = nk.raw;
    *reinterpret_cast<uint4*>(vpage + (int64_t)tok * D + lane * 8) = nv.raw;
    if (tok != ap.P - 1) return;
    float acc[8], kf[8];
    nk.unpack(kf);
    if (QUEST) {
        float hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) hi[j] = lo[j] = kf[j];
        for (int r0 = 0; r0 < ap.P - 1; r0 += 8) {
            vtx::Vec8<__nv_bfloat16> v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (r0 + u < ap.P - 1) v[u].load(kpage + (int64_t)(r0 + u) * D + lane * 8);
                else v[u].raw = nk.raw;  // repeats the new row: neutral for max and min
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                float f[8];
                v[u].unpack(f);
#pragma unroll
                for (int j = 0; j < 8; ++j) { hi[j] = fmaxf(hi[j], f[j]); lo[j] = fminf(lo[j], f[j]); }
            }
        }
        vtx::store8(ap.centroids + pid * (int64_t)D + lane * 8, hi);
        vtx::store8(ap.centroids2 + pid * (int64_t)D + lane * 8, lo);
        return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r0 = 0; r0 < ap.P - 1; r0 += 8) {
        vtx::Vec8<__nv_bfloat16> v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (r0 + u < ap.P - 1) v[u].load(kpage + (int64_t)(r0 + u) * D + lane * 8);
            else v[u].zero();
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (r0 + u < ap.P - 1) {
                float f[8];
                v[u].unpack(f);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], f[j]);
            }
        }
    }
    const float denom = (float)ap.P;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = __fdiv_rn(__fadd_rn(acc[j], kf[j]), denom);
    vtx::store8(ap.centroids + pid * (int64_t)D + lane * 8, acc);
}

// MODE 0: fused mean + GeMV + top-k.  MODE 1: GeMV only (scores to global memory).
// `side_work(warp, lane)` is called once by every thread, at a point where this CTA's first gather
// batches are already in flight (or right away for segments that need no selection); the fused layer
// kernel uses it for the new-token write of one warp.
struct NoSideWork {
    __device__ __forceinline__ void operator()(int, int) const {}
};

// MODE 2 (bf16 only, GQ = query heads per KV head): the gqa_block_sparse_attention scores, i.e.
// per query head the fp32-product dot with the page's row rounded to bf16, a softmax of scale * score over
// the segment's candidates (canonical exp and sum) rounded to bf16, and the maximum over the heads.
template <typename T, int D, int MODE, typename SideWork = NoSideWork, int GQ = 1>
__device__ __forceinline__ void indexer_body(const IndexerArgs& a, unsigned char* smem_raw, const int s,
                                             SideWork side_work = SideWork()) {
    // MODE 3 (bf16 only): the gqa_quest_sparse_attention scores from two summary caches (per-page max and min):
    // per head sum_d max(round(q_d*max_d), round(q_d*min_d)) in the canonical order, rounded, maximum over heads.
    constexpr int NQ = MODE >= 2 ? GQ : 1;                          // score accumulators per row
    constexpr int NSRC = MODE == 3 ? 2 : 1;                         // summary rows gathered per page
    constexpr int QBYTES = MODE == 2 ? GQ * D * 4 : (MODE == 3 ? GQ * D * 2 : D * (int)sizeof(T));
    using Key = typename KeyOf<T>::type;
    using Gm = Geom<T, D>;
    constexpr int L = Gm::L, HALF = L / 2;
    constexpr int SLOT_B = NSRC * Gm::slot_bytes;
    constexpr int SLOTS = SLOT_B * 3 * kWarps <= 96 * 1024 ? 3 : 2;
    constexpr size_t RING_B = (size_t)kWarps * SLOTS * SLOT_B;
    // layout: [ring][q_mean][keys][ids]
    unsigned char* ring = smem_raw;
    T* qbar = reinterpret_cast<T*>(smem_raw + RING_B);
    Key* keys = reinterpret_cast<Key*>(reinterpret_cast<unsigned char*>(qbar) + QBYTES);
    int32_t* ids = reinterpret_cast<int32_t*>(keys + a.key_cap);
    __nv_bfloat16* sbuf = reinterpret_cast<__nv_bfloat16*>(ids + a.key_cap);  // MODE 2: [candidate][head] scores
    float* qf32 = reinterpret_cast<float*>(qbar);                               // MODE 2: [head][D]

    const int beg = a.dense_indptr[s] + a.bos;
    const int c = a.dense_indptr[s + 1] - a.eos - beg;
    if (c <= a.K || (MODE != 1 && c > a.key_cap)) {  // nothing to select / more candidates than shared memory holds
        side_work(threadIdx.x >> 5, threadIdx.x & 31);
        return;
    }
    const int32_t* row_ids = a.dense_indices + beg;
    if (MODE != 1) {
        for (int i = threadIdx.x; i < c; i += kThreads) ids[i] = row_ids[i];
        row_ids = ids;
    }
    __syncthreads();  // row ids are staged

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r_in = lane >> 1, par = lane & 1;  // row of the slot; parity of the partial sums this thread owns
    unsigned char* my_ring = ring + (size_t)warp * SLOTS * SLOT_B;
    const uint32_t my_ring_addr = (uint32_t)__cvta_generic_to_shared(my_ring);
    const unsigned char* cent = reinterpret_cast<const unsigned char*>(a.centroids);
    const unsigned char* cent2 = reinterpret_cast<const unsigned char*>(a.centroids2);
    const int n_batches = (c + kRowsPerSlot - 1) / kRowsPerSlot;
    const int my_batches = n_batches > warp ? (n_batches - warp + kWarps - 1) / kWarps : 0;
    constexpr int pieces_per_slot = kRowsPerSlot * Gm::pieces;

    auto issue = [&](int ord) {
        const int row0 = (warp + ord * kWarps) * kRowsPerSlot;
        const uint32_t dst = my_ring_addr + (uint32_t)((ord % SLOTS) * SLOT_B);
#pragma unroll
        for (int pc = lane; pc < pieces_per_slot; pc += 32) {
            const int r = pc / Gm::pieces, pr = pc - r * Gm::pieces;
            const int i = row0 + r;
            const bool valid = i < c;
            const int64_t row = valid ? row_ids[i] : 0;
            const uint32_t off = r * Gm::row_bytes + ((pr ^ ((r & 3) << 1)) << 4);
            cp_async16(dst + off, cent + row * Gm::row_bytes + pr * 16, valid);
            if (NSRC == 2) cp_async16(dst + Gm::slot_bytes + off, cent2 + row * Gm::row_bytes + pr * 16, valid);
        }
    };

#pragma unroll
    for (int i = 0; i < SLOTS - 1; ++i) {
        if (i < my_batches) issue(i);
        cp_async_commit();
    }
    side_work(warp, lane);
    if (MODE == 3) {  // the group's query heads as they are
        const uint4* qs = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.q) + (int64_t)s * GQ * D);
        for (int ch = threadIdx.x; ch < GQ * Gm::nchunk; ch += kThreads) reinterpret_cast<uint4*>(qbar)[ch] = qs[ch];
    }
    if (MODE == 2) {  // the group's query heads, widened to fp32
        const T* qs = reinterpret_cast<const T*>(a.q) + (int64_t)s * GQ * D;
        for (int ch = threadIdx.x; ch < GQ * Gm::nchunk; ch += kThreads) {
            vtx::Vec8<T> v;
            v.load_cached(qs + ch * 8);
            float f[8];
            v.unpack(f);
#pragma unroll
            for (int j = 0; j < 8; ++j) qf32[ch * 8 + j] = f[j];
        }
    }
    // grouped-query mean, one canonical chunk per thread
    for (int ch = threadIdx.x; MODE < 2 && ch < Gm::nchunk; ch += kThreads) {
        const T* qs = reinterpret_cast<const T*>(a.q) + (int64_t)s * a.G * D + ch * 8;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int g = 0; g < a.G; ++g) {
            vtx::Vec8<T> v;
            v.load_cached(qs + (int64_t)g * D);
            float f[8];
            v.unpack(f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], f[j]);
        }
        const float g_f = (float)a.G;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __fdiv_rn(acc[j], g_f);
        vtx::store8(qbar + ch * 8, acc);  // rounds once to T
    }
    __syncthreads();  // q_mean is staged
    for (int ord = 0; ord < my_batches; ++ord) {
        cp_async_wait<SLOTS - 2>();
        __syncwarp();
        if (ord + SLOTS - 1 < my_batches) issue(ord + SLOTS - 1);
        cp_async_commit();
        const unsigned char* row_ptr = my_ring + (size_t)(ord % SLOTS) * SLOT_B + r_in * Gm::row_bytes;
        const int sw = (r_in & 3) << 1;
        const int i = (warp + ord * kWarps) * kRowsPerSlot + r_in;
        float best = -INFINITY;  // MODE 3: running maximum over the heads
#pragma unroll
        for (int g = 0; g < NQ; ++g) {
            float acc[HALF];
#pragma unroll
            for (int ii = 0; ii < HALF; ++ii) acc[ii] = 0.f;
            // this thread owns partial sums 2*ii + par; partial l takes chunks l, l + L, ...
#pragma unroll
            for (int k = 0; k * L < Gm::nchunk; ++k) {
#pragma unroll
                for (int ii = 0; ii < HALF; ++ii) {
                    if (k * L + 2 * ii < Gm::nchunk) {  // nchunk is even, so the test holds for both parities
                        const int ch = k * L + 2 * ii + par;
                        // a chunk is ppc adjacent 16-byte pieces; the swizzle flips piece bits 1-2 only
                        const T* src = reinterpret_cast<const T*>(row_ptr + (((ch * Gm::ppc) ^ sw) << 4));
                        if constexpr (MODE == 3)
                            add_quest_bounds(acc[ii], reinterpret_cast<const __nv_bfloat16*>(src),
                                             reinterpret_cast<const __nv_bfloat16*>(
                                                 reinterpret_cast<const unsigned char*>(src) + Gm::slot_bytes),
                                             reinterpret_cast<const __nv_bfloat16*>(qbar) + g * D + ch * 8);
                        else if constexpr (MODE == 2)
                            add_products_f32(acc[ii], reinterpret_cast<const __nv_bfloat16*>(src),
                                             qf32 + g * D + ch * 8);
                        else
                            add_products(acc[ii], src, qbar + ch * 8);
                    }
                }
            }
#pragma unroll
            for (int w = HALF / 2; w > 0; w >>= 1)
#pragma unroll
                for (int ii = 0; ii < w; ++ii) acc[ii] = __fadd_rn(acc[ii], acc[ii + w]);
            const float total = __fadd_rn(acc[0], __shfl_xor_sync(0xffffffffu, acc[0], 1));
            if (par == 0 && i < c) {
                const float sc = vtx::round_to<T>(total);
                if (MODE == 0) keys[i] = KeyOf<T>::make(sc, i);
                else if (MODE == 2) sbuf[i * NQ + g] = __float2bfloat16_rn(sc);
                else if (MODE == 3) best = fmaxf(best, sc);
                else store_score<T>(reinterpret_cast<T*>(a.scores) + beg + i, sc);
            }
        }
        if (MODE == 3 && par == 0 && i < c) keys[i] = KeyOf<T>::make(best, i);
    }
    cp_async_wait<0>();
    if constexpr (MODE == 2) {
        __syncthreads();  // all head scores written; the rings are idle and lend their space to the reductions
        float* red = reinterpret_cast<float*>(ring);  // [NQ][kThreads]
        float mx[NQ], l[NQ];
#pragma unroll
        for (int g = 0; g < NQ; ++g) mx[g] = -INFINITY;
        for (int i = threadIdx.x; i < c; i += kThreads)
#pragma unroll
            for (int g = 0; g < NQ; ++g)
                mx[g] = fmaxf(mx[g], __fmul_rn(__bfloat162float(sbuf[i * NQ + g]), a.scale));
#pragma unroll
        for (int g = 0; g < NQ; ++g) red[g * kThreads + threadIdx.x] = mx[g];
        __syncthreads();
#pragma unroll
        for (int g = 0; g < NQ; ++g) {
            float m = red[g * kThreads];
            for (int t = 1; t < kThreads; ++t) m = fmaxf(m, red[g * kThreads + t]);
            mx[g] = m;
        }
        __syncthreads();
        // sum of exp: partial t takes candidates t, t + 128, ... in ascending order, then halves are folded
#pragma unroll
        for (int g = 0; g < NQ; ++g) l[g] = 0.f;
        for (int i = threadIdx.x; i < c; i += kThreads)
#pragma unroll
            for (int g = 0; g < NQ; ++g) {
                const float t = __fmul_rn(__bfloat162float(sbuf[i * NQ + g]), a.scale);
                l[g] = __fadd_rn(l[g], exp_canonical(__fsub_rn(t, mx[g])));
            }
#pragma unroll
        for (int g = 0; g < NQ; ++g) red[g * kThreads + threadIdx.x] = l[g];
        __syncthreads();
        for (int w = kThreads / 2; w > 0; w >>= 1) {
            if (threadIdx.x < w)
#pragma unroll
                for (int g = 0; g < NQ; ++g)
                    red[g * kThreads + threadIdx.x] =
                        __fadd_rn(red[g * kThreads + threadIdx.x], red[g * kThreads + threadIdx.x + w]);
            __syncthreads();
        }
#pragma unroll
        for (int g = 0; g < NQ; ++g) l[g] = red[g * kThreads];
        for (int i = threadIdx.x; i < c; i += kThreads) {
            float best = -INFINITY;
#pragma unroll
            for (int g = 0; g < NQ; ++g) {
                const float t = __fmul_rn(__bfloat162float(sbuf[i * NQ + g]), a.scale);
                const float pr = __fdiv_rn(exp_canonical(__fsub_rn(t, mx[g])), l[g]);
                best = fmaxf(best, vtx::round_to<T>(pr));
            }
            keys[i] = KeyOf<T>::make(best, i);
        }
    }
    if (MODE != 1) {
        __syncthreads();  // all keys written, every ring is idle: its space becomes the sort's scratch
        const int o0 = a.sparse_indptr[s] + a.bos;
        select_and_store<T>(keys, ids, c, a.K, a.sparse_indices + o0,
                            a.sparse_pt ? a.sparse_pt + (int64_t)s * a.pt_stride + a.bos : nullptr,
                            reinterpret_cast<Key*>(ring));
    }
}

template <typename T, int D, int MODE>
__global__ void __launch_bounds__(kThreads, 4) indexer_kernel(IndexerArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    indexer_body<T, D, MODE>(a, smem_raw, blockIdx.x);
}

// gqa_block_sparse_attention indexer: GeMM -> Softmax over pages -> Max over heads -> top-k, one launch.
template <int D, int GQ>
__global__ void __launch_bounds__(kThreads, 4) indexer_gqa_kernel(IndexerArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    indexer_body<__nv_bfloat16, D, 2, NoSideWork, GQ>(a, smem_raw, blockIdx.x);
}

// gqa_quest_sparse_attention indexer: envelope bound per head -> Max over heads -> top-k, one launch.
template <int D, int GQ>
__global__ void __launch_bounds__(kThreads, 2) indexer_quest_kernel(IndexerArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    vtx::pdl_wait();
    vtx::pdl_trigger();
    indexer_body<__nv_bfloat16, D, 3, NoSideWork, GQ>(a, smem_raw, blockIdx.x);
}

// One launch per sparse layer: page selection, then attention over the selected pages, by the same CTA.
// The decode phase of one segment overlaps the scan phase of its neighbours on the SM, so neither phase
// pays its own launch and ramp-up; the selected rows still go to the sparse page list (the decode reads
// them back after the block barrier).  bf16 only (the decode phase is the tensor-core body).
// With APPEND the CTA first writes its segment's new token (and the centroid of the page it closes):
// the page is the segment's last one, which is never a candidate (eos >= 1), and the decode phase reads
// it only after two block barriers, so the write needs no kernel of its own.
// With EARLY (programmatic launch mode 2) the CTA stages its row ids and starts its first centroid
// gathers before it waits for the preceding launch: those reads touch only the planner's outputs and
// this layer's centroid rows of non-reserved pages, which no launch between the planner and this one
// writes.  Everything else (q, the token write, the sparse list, the output) comes after the wait.
// MODE 0: scores of the block_sparse_attention flow (group mean . centroid); MODE 2: scores of the
// gqa_block_sparse_attention flow (per-head product, softmax over pages, maximum over heads) on the same
// centroid cache, so the token write is the same too; MODE 3: scores of the gqa_quest_sparse_attention flow
// from the per-page maximum and minimum caches, which the token write then maintains instead of the mean
// (twice the summary bytes per page: two CTAs per SM instead of four).
template <int D, int G, bool APPEND, bool EARLY, int MODE = 0>
__global__ void __launch_bounds__(kThreads, MODE == 3 ? 2 : 4) sparse_layer_kernel(IndexerArgs ia, vtxdec::DecodeArgs da,
                                                                  AppendArgs ap) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    if (!EARLY) vtx::pdl_wait();
    vtx::pdl_trigger();
    const int seg = blockIdx.x;
    auto side = [&](int warp, int lane) {
        if (EARLY) vtx::pdl_wait();
        if (APPEND && warp == kWarps - 1) append_token<D, MODE == 3>(ap, seg, lane);
    };
    indexer_body<__nv_bfloat16, D, MODE, decltype(side), (MODE >= 2 ? G : 1)>(ia, smem_raw, seg, side);
    __syncthreads();  // the list is complete and visible to the CTA; rings and sort scratch are idle
    vtxdec::decode_mma_body<G, D>(da, smem_raw, blockIdx.x);
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
    if (c <= a.K || c > a.key_cap) return;
    for (int i = threadIdx.x; i < c; i += kThreads) {
        ids[i] = a.dense_indices[beg + i];
        keys[i] = KeyOf<T>::make(load_score<T>(scores + beg + i), i);
    }
    __syncthreads();
    const int o0 = a.sparse_indptr[s] + a.bos;
    select_and_store<T>(keys, ids, c, a.K, a.sparse_indices + o0, nullptr, xbuf);
}

template <typename Kern>
int set_smem(Kern kern, size_t bytes) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) {
            vtx::note_cuda_error(e);
            return VTX_ERR_CUDA;
        }
    }
    return VTX_OK;
}

template <typename T, int D, int MODE>
int launch_indexer_cfg(const IndexerArgs& a, int eff_bs, cudaStream_t st) {
    using Gm = Geom<T, D>;
    using Key = typename KeyOf<T>::type;
    size_t bytes = Gm::ring_bytes + Gm::row_bytes;
    if (MODE == 0) bytes += (size_t)a.key_cap * (sizeof(Key) + sizeof(int32_t));
    if (bytes > 227 * 1024) return VTX_ERR_UNSUPPORTED;
    auto kern = indexer_kernel<T, D, MODE>;
    int rc = set_smem(kern, bytes);
    if (rc != VTX_OK) return rc;
    return vtx::launch(kern, dim3(eff_bs), dim3(kThreads), bytes, st, a);
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
    return vtx::launch(kern, dim3(eff_bs), dim3(kThreads), bytes, st, a);
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
    constexpr int slots = slot_b * 3 * kWarps <= 96 * 1024 ? 3 : 2;
    const size_t bytes = (size_t)kWarps * slots * slot_b + (size_t)GQ * D * 2 +
                         (size_t)a.key_cap * (sizeof(uint32_t) + sizeof(int32_t));
    if (bytes > 227 * 1024) return VTX_ERR_UNSUPPORTED;
    auto kern = indexer_quest_kernel<D, GQ>;
    int rc = set_smem(kern, bytes);
    if (rc != VTX_OK) return rc;
    return vtx::launch(kern, dim3(eff_bs), dim3(kThreads), bytes, st, a);
}

int launch_indexer_quest(const IndexerArgs& a, int eff_bs, cudaStream_t st) {
#define VTX_QUEST_CASE(D_, G_) \
    if (a.D == D_ && a.G == G_) return launch_indexer_quest_cfg<D_, G_>(a, eff_bs, st);
    VTX_QUEST_CASE(64, 1) VTX_QUEST_CASE(64, 2) VTX_QUEST_CASE(64, 4) VTX_QUEST_CASE(64, 8)
    VTX_QUEST_CASE(128, 1) VTX_QUEST_CASE(128, 2) VTX_QUEST_CASE(128, 4) VTX_QUEST_CASE(128, 8)
#undef VTX_QUEST_CASE
    return VTX_ERR_UNSUPPORTED;
}

template <int D, int G, int MODE>
int launch_sparse_layer_cfg(const IndexerArgs& ia, const vtxdec::DecodeArgs& da, const AppendArgs& ap, int eff_bs,
                            cudaStream_t st) {
    using Gm = Geom<__nv_bfloat16, D>;
    static_assert(vtxdec::kDecWarps * 32 == kThreads, "both phases use the same CTA shape");
    constexpr int quest_slot_b = 2 * Gm::slot_bytes;
    constexpr int quest_slots = quest_slot_b * 3 * kWarps <= 96 * 1024 ? 3 : 2;
    size_t bytes = MODE == 2 ? Gm::ring_bytes + (size_t)G * D * 4 +
                                   (size_t)ia.key_cap * (sizeof(uint32_t) + sizeof(int32_t) + G * sizeof(__nv_bfloat16))
                   : MODE == 3 ? (size_t)kWarps * quest_slots * quest_slot_b + (size_t)G * D * 2 +
                                     (size_t)ia.key_cap * (sizeof(uint32_t) + sizeof(int32_t))
                               : Gm::ring_bytes + Gm::row_bytes + (size_t)ia.key_cap * (sizeof(uint32_t) + sizeof(int32_t));
    const size_t dec = vtxdec::decode_mma_smem_bytes<G, D>();
    if (dec > bytes) bytes = dec;
    if (bytes > 227 * 1024) return VTX_ERR_UNSUPPORTED;
    const bool early = vtx::programmatic_launch_mode() == 2;
    auto kern = ap.loc ? (early ? sparse_layer_kernel<D, G, true, true, MODE> : sparse_layer_kernel<D, G, true, false, MODE>)
                       : (early ? sparse_layer_kernel<D, G, false, true, MODE> : sparse_layer_kernel<D, G, false, false, MODE>);
    int rc = set_smem(kern, bytes);
    if (rc != VTX_OK) return rc;
    return vtx::launch(kern, dim3(eff_bs), dim3(kThreads), bytes, st, ia, da, ap);
}

template <int D, int MODE>
int launch_sparse_layer_d(const IndexerArgs& ia, const vtxdec::DecodeArgs& da, const AppendArgs& ap, int eff_bs,
                          int group, cudaStream_t st) {
    switch (group) {
        case 1: return launch_sparse_layer_cfg<D, 1, MODE>(ia, da, ap, eff_bs, st);
        case 2: return launch_sparse_layer_cfg<D, 2, MODE>(ia, da, ap, eff_bs, st);
        case 4: return launch_sparse_layer_cfg<D, 4, MODE>(ia, da, ap, eff_bs, st);
        case 8: return launch_sparse_layer_cfg<D, 8, MODE>(ia, da, ap, eff_bs, st);
        default: return VTX_ERR_UNSUPPORTED;
    }
}

int check_common(const int32_t* dip, const int32_t* din, int eff_bs, int K, int bos, int eos, int maxp,
                 int dtype) {
    if (!dip || !din) return VTX_ERR_INVALID_ARGUMENT;
    if (eff_bs < 0 || K < 1 || bos < 0 || eos < 0 || maxp < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    if (maxp > kMaxCandidates) return VTX_ERR_UNSUPPORTED;
    return VTX_OK;
}

// Candidate capacity of one segment (sizes the key and row-id arrays in shared memory).
int key_capacity(int max_pages) { return vtx::pow2_ceil(max_pages); }

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
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == VTX_BF16 ? launch_indexer<__nv_bfloat16, 0>(a, eff_batch_size, st)
                             : launch_indexer<float, 0>(a, eff_batch_size, st);
}

namespace {
int sparse_layer_fused_impl(const void* q, const void* centroids, const void* centroids2, const void* k_cache,
                            const void* v_cache,
                            void* out, const void* new_k, const void* new_v, const int64_t* loc,
                            int num_kv_heads, const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                            const int32_t* dense_kv_indices, int32_t* sparse_kv_indices,
                            const int32_t* kv_last_page_len, int eff_batch_size, int group_size,
                            int head_dim, int page_size, int topk_val, int page_reserved_bos,
                            int page_reserved_eos, int max_num_pages_per_request, float sm_scale,
                            int dtype, void* stream, int score_mode, float softmax_scale) {
    int rc = check_common(dense_kv_indptr, dense_kv_indices, eff_batch_size, topk_val, page_reserved_bos,
                          page_reserved_eos, max_num_pages_per_request, dtype);
    if (rc != VTX_OK) return rc;
    if (!q || !centroids || !k_cache || !v_cache || !out || !sparse_kv_indptr || !sparse_kv_indices ||
        !kv_last_page_len)
        return VTX_ERR_INVALID_ARGUMENT;
    if (group_size < 1 || page_size < 1) return VTX_ERR_INVALID_ARGUMENT;
    const int appends = (new_k != nullptr) + (new_v != nullptr) + (loc != nullptr);
    if (appends != 0 && appends != 3) return VTX_ERR_INVALID_ARGUMENT;
    if (appends == 3 && (num_kv_heads < 1 || eff_batch_size % num_kv_heads != 0 || page_reserved_eos < 1))
        return VTX_ERR_INVALID_ARGUMENT;  // the written page must be a reserved (never scanned) one
    if (dtype != VTX_BF16) return VTX_ERR_UNSUPPORTED;
    if (eff_batch_size == 0) return VTX_OK;
    AppendArgs ap{};
    if (appends == 3) {
        ap.k_cache = (__nv_bfloat16*)const_cast<void*>(k_cache);
        ap.v_cache = (__nv_bfloat16*)const_cast<void*>(v_cache);
        ap.centroids = (__nv_bfloat16*)const_cast<void*>(centroids);
        ap.centroids2 = (__nv_bfloat16*)const_cast<void*>(centroids2);
        ap.new_k = (const __nv_bfloat16*)new_k;
        ap.new_v = (const __nv_bfloat16*)new_v;
        ap.loc = loc;
        ap.H = num_kv_heads;
        ap.P = page_size;
    }
    IndexerArgs ia{};
    ia.q = q;
    ia.centroids = centroids;
    ia.centroids2 = centroids2;
    ia.dense_indptr = dense_kv_indptr;
    ia.sparse_indptr = sparse_kv_indptr;
    ia.dense_indices = dense_kv_indices;
    ia.sparse_indices = sparse_kv_indices;
    ia.G = group_size;
    ia.D = head_dim;
    ia.K = topk_val;
    ia.bos = page_reserved_bos;
    ia.eos = page_reserved_eos;
    ia.key_cap = key_capacity(max_num_pages_per_request);
    ia.scale = softmax_scale;
    if (score_mode == 3 && !centroids2) return VTX_ERR_INVALID_ARGUMENT;
    vtxdec::DecodeArgs da;
    da.q = q;
    da.k = k_cache;
    da.v = v_cache;
    da.out = out;
    da.indptr = sparse_kv_indptr;
    da.indices = sparse_kv_indices;
    da.last_len = kv_last_page_len;
    da.P = page_size;
    da.scale_log2 = sm_scale * 1.4426950408889634f;
    cudaStream_t st = (cudaStream_t)stream;
    if (score_mode == 3) {
        switch (head_dim) {
            case 64: return launch_sparse_layer_d<64, 3>(ia, da, ap, eff_batch_size, group_size, st);
            case 128: return launch_sparse_layer_d<128, 3>(ia, da, ap, eff_batch_size, group_size, st);
            default: return VTX_ERR_UNSUPPORTED;
        }
    }
    if (score_mode == 2) {
        switch (head_dim) {
            case 64: return launch_sparse_layer_d<64, 2>(ia, da, ap, eff_batch_size, group_size, st);
            case 128: return launch_sparse_layer_d<128, 2>(ia, da, ap, eff_batch_size, group_size, st);
            default: return VTX_ERR_UNSUPPORTED;
        }
    }
    switch (head_dim) {
        case 64: return launch_sparse_layer_d<64, 0>(ia, da, ap, eff_batch_size, group_size, st);
        case 128: return launch_sparse_layer_d<128, 0>(ia, da, ap, eff_batch_size, group_size, st);
        default: return VTX_ERR_UNSUPPORTED;
    }
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
    return sparse_layer_fused_impl(q, centroids, nullptr, k_cache, v_cache, out, new_k, new_v, loc, num_kv_heads,
                                   dense_kv_indptr, sparse_kv_indptr, dense_kv_indices, sparse_kv_indices,
                                   kv_last_page_len, eff_batch_size, group_size, head_dim, page_size, topk_val,
                                   page_reserved_bos, page_reserved_eos, max_num_pages_per_request, sm_scale, dtype,
                                   stream, 0, 0.f);
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
    return sparse_layer_fused_impl(q, cache_max, cache_min, k_cache, v_cache, out, new_k, new_v, loc, num_kv_heads,
                                   dense_kv_indptr, sparse_kv_indptr, dense_kv_indices, sparse_kv_indices,
                                   kv_last_page_len, eff_batch_size, group_size, head_dim, page_size, topk_val,
                                   page_reserved_bos, page_reserved_eos, max_num_pages_per_request, sm_scale, dtype,
                                   stream, 3, 0.f);
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
    return sparse_layer_fused_impl(q, centroids, nullptr, k_cache, v_cache, out, new_k, new_v, loc, num_kv_heads,
                                   dense_kv_indptr, sparse_kv_indptr, dense_kv_indices, sparse_kv_indices,
                                   kv_last_page_len, eff_batch_size, group_size, head_dim, page_size, topk_val,
                                   page_reserved_bos, page_reserved_eos, max_num_pages_per_request, sm_scale, dtype,
                                   stream, 2, softmax_scale);
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
    return launch_indexer_quest(a, eff_batch_size, (cudaStream_t)stream);
}
