// Device code shared by the indexer kernels and the one-launch sparse layer kernels.
//
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
#pragma once
#include <type_traits>

#include "decode_mma_body.cuh"
#include "vtx_common.cuh"

namespace vtxidx {

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
    // A segment with more than `chunk` candidates is scanned by several CTAs (blockIdx.y = chunk number; the grid is
    // (segments, chunks), so the chunk numbers that only long segments have are placed last and the CTAs that
    // find nothing to do do not hold up the ones that do):
    // each keeps the K best keys of its chunk in part_keys, counts itself in tickets[segment], and the CTA
    // that arrives last sorts the union (its first K are the segment's first K: keys are unique and the
    // order is total).  chunk == 0: one CTA per segment.
    int chunk = 0, nch_max = 1;
    void* part_keys = nullptr;     // [eff_bs][nch_max][K] keys
    int32_t* tickets = nullptr;    // [eff_bs], zero between launches
    uint32_t* status = nullptr;    // sticky device status word (VTX_STATUS_* bits)
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

}  // namespace vtxidx

namespace {

using vtxidx::AppendArgs;
using vtxidx::IndexerArgs;

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxCandidates = 16384;
constexpr int kRowsPerSlot = 16;

// Barrier of the kThreads threads that run an indexer body.  BAR == 0: they are the whole CTA.  BAR > 0: they
// are one group of kThreads consecutive threads of a larger CTA (the body runs as a phase of another kernel, one
// instance per group, all from the same call site) and group g meets at named barrier BAR + g, which nothing
// else of that kernel may use during the phase.
template <int BAR>
__device__ __forceinline__ void body_sync() {
    if constexpr (BAR == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(BAR + (int)(threadIdx.x / kThreads)), "n"(kThreads) : "memory");
}

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

// Sort the c keys at `keys` (shared memory, visible to all threads) in descending order and hand the
// first K of them to emit(position, key); each position is emitted by exactly one thread.
// xbuf: shared scratch for the register sort, sort_scratch_bytes(c) bytes, or null to force the
// shared-memory network (which sorts `keys` in place; c may then be any size up to the key capacity).
template <typename Key, int EPT, typename Emit>
__device__ __forceinline__ void sort_regs_emit(const Key* keys, int c, int K, Key* xbuf, Emit& emit) {
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
        if (e < K) emit(e, v[r]);
    }
}

// Keys the register sort handles for c candidates (0: the shared-memory network takes over).
__host__ __device__ inline int sort_width(int c) {
    return c <= kThreads * 4 ? kThreads * 4 : (c <= kThreads * 8 ? kThreads * 8 : (c <= kThreads * 16 ? kThreads * 16 : 0));
}

template <typename Key, typename Emit>
__device__ __forceinline__ void sort_emit(Key* keys, int c, int K, Key* xbuf, Emit& emit) {
    if (xbuf != nullptr && c <= kThreads * 4) return sort_regs_emit<Key, 4>(keys, c, K, xbuf, emit);
    if (xbuf != nullptr && c <= kThreads * 8) return sort_regs_emit<Key, 8>(keys, c, K, xbuf, emit);
    if (xbuf != nullptr && c <= kThreads * 16) return sort_regs_emit<Key, 16>(keys, c, K, xbuf, emit);
    const int n = vtx::pow2_ceil(c);
    for (int i = c + threadIdx.x; i < n; i += kThreads) keys[i] = (Key)0;
    __syncthreads();
    block_bitonic_desc<Key>(keys, n);
    for (int j = threadIdx.x; j < K; j += kThreads) emit(j, keys[j]);
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
using vtx::add_bf16;
__device__ __forceinline__ void add_pair(float& acc, uint32_t packed) {  // low half first, then the high half
    uint16_t lo, hi;
    asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(packed));
    acc = add_bf16(acc, lo);
    acc = add_bf16(acc, hi);
}
__device__ __forceinline__ void add_products(float& acc, const __nv_bfloat16* row_chunk, const __nv_bfloat16* q_chunk) {
    const uint4 r = *reinterpret_cast<const uint4*>(row_chunk);
    const uint4 q = *reinterpret_cast<const uint4*>(q_chunk);
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w}, qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 p = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&rr[i]),
                                         *reinterpret_cast<const __nv_bfloat162*>(&qq[i]));
        add_pair(acc, *reinterpret_cast<const uint32_t*>(&p));
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

// bf16 row chunk times bf16 query chunk, products kept in fp32 (the GeMM operator's arithmetic): the product of
// two bf16 values has 16 significant bits, so it is exact in fp32 and the mixed-precision fused multiply-add of
// sm_100 (bf16 x bf16 + fp32, one rounding) returns what a separate exact multiply and a rounded add return -
// for every product inside fp32's normal range; below 2^-126 a separate multiply would round first.
__device__ __forceinline__ float fma_bf16(uint16_t x, uint16_t y, float acc) {
    float d;
    asm("fma.rn.f32.bf16 %0, %1, %2, %3;" : "=f"(d) : "h"(x), "h"(y), "f"(acc));
    return d;
}
__device__ __forceinline__ void add_products_f32(float& acc, const __nv_bfloat16* row_chunk, const __nv_bfloat16* q_chunk) {
    const uint4 r = *reinterpret_cast<const uint4*>(row_chunk);
    const uint4 q = *reinterpret_cast<const uint4*>(q_chunk);
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w}, qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint16_t r0, r1, q0, q1;
        asm("mov.b32 {%0, %1}, %2;" : "=h"(r0), "=h"(r1) : "r"(rr[i]));
        asm("mov.b32 {%0, %1}, %2;" : "=h"(q0), "=h"(q1) : "r"(qq[i]));
        acc = fma_bf16(r0, q0, acc);
        acc = fma_bf16(r1, q1, acc);
    }
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
        add_pair(acc, *reinterpret_cast<const uint32_t*>(&u));
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

// Slots of a warp's gather ring: three where four CTAs per SM still fit (ring <= 96 KB), else two.  (Three slots
// for the wide rows of the MLA latent, where one CTA per SM is all that fits anyway, were measured: the scan is
// no faster and the decode that follows is slower.)
constexpr int ring_slots(int slot_b) { return slot_b * 3 * kWarps <= 96 * 1024 ? 3 : 2; }

template <typename T, int D, int LPR = 2>
struct Geom {
    static constexpr int nchunk = D / 8;  // canonical chunks of 8 dims
    static constexpr int L = nchunk > 16 ? 32 : (nchunk > 8 ? 16 : (nchunk > 4 ? 8 : 4));
    static constexpr int row_bytes = D * (int)sizeof(T);
    static constexpr int pieces = row_bytes / 16;        // 16-byte pieces per row
    static constexpr int ppc = 8 * (int)sizeof(T) / 16;  // pieces per canonical chunk (1 bf16, 2 fp32)
    // lanes that share a row while it is scored: two; four (half the rows per batch, half the slot) where two
    // bodies have to fit side by side in one CTA's shared memory.  More, smaller batches cost a stand-alone scan
    // of wide rows 2 us, so four is the choice of that one caller, not the rule.
    static constexpr int lpr = LPR;
    static constexpr int rows_per_slot = 32 / lpr;
    // A 16-byte read of a warp is served a quarter warp (8 lanes = 8 / lpr rows) at a time, and the rows of a slot
    // start at the same bank; the piece index of row r is XORed with swizzle(r) so that the lpr consecutive
    // pieces read by the lanes of one row never meet those of the other rows of its quarter warp.
    __host__ __device__ static constexpr int swizzle(int r) { return (r % (8 / lpr)) * lpr; }
    static constexpr int slot_bytes = rows_per_slot * row_bytes;
    static constexpr int slots = ring_slots(slot_bytes);
    static constexpr size_t ring_bytes = (size_t)kWarps * slots * slot_bytes;
    static_assert(pieces % 8 == 0, "row must be a multiple of 128 bytes");
    static_assert(nchunk % lpr == 0 && L % lpr == 0, "the lanes of a row split its partial sums evenly");
    // the idle ring doubles as the sort's exchange buffer (2 x 2048 keys at most)
    static_assert(LPR != 2 || ring_bytes >= 2 * 2048 * sizeof(typename KeyOf<T>::type), "ring too small for the sort scratch");
};


// ---- new-token write of one segment s = request * H + head, executed by one warp ----
// Lanes 0 .. D/8-1 each own 8 head dims.  The write is cut in two so that its loads can be in flight together
// with the other loads a warp issues after the launch's inputs become readable:
//   append_load   reads the token's K and V rows and its cache slot;
//   append_finish writes the two rows and, if the token closes its page, the page's summary: the mean of K
//                 (rows 0 .. P-2 in ascending order, the new row last, one division, one rounding - the
//                 arithmetic of set_kv_cmean_kernel in cache_ops.cu) or, with QUEST, the per-dim maximum and
//                 minimum (exact in bf16, as vtx_creduce computes them).  The page's older rows come from
//                 `rows_smem` when the caller copied them there (row r at rows_smem + r * D * 2), else from
//                 the cache.
struct AppendRegs {
    uint4 k, v;
    int64_t slot;
};

template <int D>
__device__ __forceinline__ AppendRegs append_load(const AppendArgs& ap, const int s, const int lane) {
    AppendRegs r{};
    if (lane >= D / 8) return r;
    r.k = *reinterpret_cast<const uint4*>(ap.new_k + (int64_t)s * D + lane * 8);
    r.v = *reinterpret_cast<const uint4*>(ap.new_v + (int64_t)s * D + lane * 8);
    r.slot = VTX_CHECK_LOC(ap.loc[s / ap.H]);
    return r;
}

template <int D, bool QUEST = false>
__device__ __forceinline__ void append_finish(const AppendArgs& ap, const int s, const int lane, const AppendRegs& in,
                                              const unsigned char* rows_smem) {
    constexpr int NCH = D / 8;
    if (lane >= NCH) return;
    const int h = s % ap.H;
    const vtx::PageSlot ps = vtx::page_slot(in.slot, ap.P);
    const int64_t pid = ps.page * ap.H + h;
    const int tok = ps.row;
    __nv_bfloat16* kpage = ap.k_cache + pid * (int64_t)ap.P * D;
    __nv_bfloat16* vpage = ap.v_cache + pid * (int64_t)ap.P * D;
    *reinterpret_cast<uint4*>(kpage + (int64_t)tok * D + lane * 8) = in.k;
    *reinterpret_cast<uint4*>(vpage + (int64_t)tok * D + lane * 8) = in.v;
    if (tok != ap.P - 1) return;
    vtx::Vec8<__nv_bfloat16> nk;
    nk.raw = in.k;
    float kf[8];
    nk.unpack(kf);
    float a0[8], a1[8];  // mean: running sum (a1 unused); QUEST: running maximum and minimum
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        a0[j] = QUEST ? kf[j] : 0.f;
        a1[j] = kf[j];
    }
    for (int r0 = 0; r0 < ap.P - 1; r0 += 8) {
        vtx::Vec8<__nv_bfloat16> v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (r0 + u < ap.P - 1) {
                if (rows_smem != nullptr)
                    v[u].raw = *reinterpret_cast<const uint4*>(rows_smem + (size_t)(r0 + u) * (D * 2) + lane * 16);
                else
                    v[u].load(kpage + (int64_t)(r0 + u) * D + lane * 8);
            } else {
                v[u].raw = in.k;  // placeholder, skipped (mean) or neutral (max / min) below
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            float f[8];
            v[u].unpack(f);
            if (QUEST) {
#pragma unroll
                for (int j = 0; j < 8; ++j) { a0[j] = fmaxf(a0[j], f[j]); a1[j] = fminf(a1[j], f[j]); }
            } else if (r0 + u < ap.P - 1) {
#pragma unroll
                for (int j = 0; j < 8; ++j) a0[j] = __fadd_rn(a0[j], f[j]);
            }
        }
    }
    if (QUEST) {
        vtx::store8(ap.centroids + pid * (int64_t)D + lane * 8, a0);
        vtx::store8(ap.centroids2 + pid * (int64_t)D + lane * 8, a1);
        return;
    }
    const float denom = (float)ap.P;
#pragma unroll
    for (int j = 0; j < 8; ++j) a0[j] = __fdiv_rn(__fadd_rn(a0[j], kf[j]), denom);
    vtx::store8(ap.centroids + pid * (int64_t)D + lane * 8, a0);
}

// ---- the best keys of a warp, kept sorted in registers while the warp scores its rows ----
// 32 * KPL keys per warp, element e = lane * KPL + r, descending in e.  Keys are unique and never 0 for
// finite scores; 0 marks an empty place.
template <typename Key, int KPL>
__device__ __forceinline__ void warp_bitonic_desc(Key (&v)[KPL], const int lane, const int k_first) {
    // bitonic network over the warp's 32 * KPL elements; stages k = k_first .. N (k_first = 2: full sort of
    // any input; k_first = N: the last merge only, which sorts a bitonic sequence)
    constexpr int N = 32 * KPL;
#pragma unroll
    for (int k = 2; k <= N; k <<= 1) {
        if (k < k_first) continue;
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            if (j < KPL) {
#pragma unroll
                for (int r = 0; r < KPL; ++r) {
                    if ((r & j) == 0) {
                        const bool desc = (((lane * KPL + r) & k) == 0);
                        const Key x = v[r], y = v[r + j];
                        const bool sw = (x < y) == desc;
                        v[r] = sw ? y : x;
                        v[r + j] = sw ? x : y;
                    }
                }
            } else {
                const int pt = j / KPL;
                const bool keep_max = ((lane & pt) == 0) == (((lane * KPL) & k) == 0);
#pragma unroll
                for (int r = 0; r < KPL; ++r) {
                    const Key o = __shfl_xor_sync(0xffffffffu, v[r], pt);
                    v[r] = keep_max ? (v[r] > o ? v[r] : o) : (v[r] < o ? v[r] : o);
                }
            }
        }
    }
}

// run <- the best 32 * KPL keys of run (sorted) and add (any order)
template <typename Key, int KPL>
__device__ __forceinline__ void warp_topk_merge(Key (&run)[KPL], Key (&add)[KPL], const int lane) {
    warp_bitonic_desc<Key, KPL>(add, lane, 2);
    // element e of run against element N-1-e of add: a descending and an ascending sequence, whose
    // elementwise maximum is a bitonic sequence holding the best N of the union
#pragma unroll
    for (int r = 0; r < KPL; ++r) {
        const Key o = __shfl_sync(0xffffffffu, add[KPL - 1 - r], 31 - lane);
        run[r] = run[r] > o ? run[r] : o;
    }
    warp_bitonic_desc<Key, KPL>(run, lane, 32 * KPL);
}

// Hooks of the fused layer kernel into the indexer body (the stand-alone indexer kernels use the no-op form).
//   issue_extra(warp, lane, spare)  between the issue and the commit of a warp's last prologue gather batch:
//                                   may start asynchronous copies into the warp's still unused ring slot
//                                   (shared address `spare`), which then belong to that copy group;
//   wait()                          first point at which the launch's own inputs (q, new token) are read;
//   load(warp, lane) / finish(warp, lane, spare_ptr)  per-warp extra work around the query staging: `load`
//                                   issues global loads only, `finish` runs once the warp's prologue copies
//                                   have landed (it may read the spare slot) and before the gather loop;
//   pre_sort(n)                     by every thread right before the step after which this CTA owns the
//                                   segment's complete page list (every ring is idle, n keys are left to
//                                   order); returns the byte offset in the CTA's shared memory at which
//                                   that step may put its scratch.
struct NoHooks {
    struct Regs {};
    __device__ __forceinline__ void issue_extra(int, int, uint32_t) const {}
    __device__ __forceinline__ void wait() const {}
    __device__ __forceinline__ Regs load(int, int) const { return Regs{}; }
    __device__ __forceinline__ bool needs_spare(int) const { return false; }
    __device__ __forceinline__ void finish(int, int, const Regs&, const unsigned char*) const {}
    __device__ __forceinline__ int pre_sort(int) const { return 0; }
};

// Emits position e of a sorted key sequence: into the chunk's slot of part_keys, or - for the last sort
// of a segment - the row id of the candidate the key names into the sparse page list (and block table).
template <typename T>
struct EmitSelection {
    using Key = typename KeyOf<T>::type;
    bool to_scratch;
    Key* part;
    const int32_t* ids;  // candidate position -> row id
    int32_t* out;
    int32_t* out_pt;
    __device__ __forceinline__ void operator()(int e, Key k) const {
        if (to_scratch) {
            part[e] = k;
            return;
        }
        const int32_t row = ids[KeyOf<T>::index(k)];
        out[e] = row;
        if (out_pt) out_pt[e] = row;
    }
};

// Keys a warp keeps per lane for top-k values up to 32 * kpl (0: the keys go to shared memory and are
// sorted by the whole CTA afterwards).
__host__ __device__ inline int stream_kpl(int K) { return K <= 32 ? 1 : (K <= 64 ? 2 : 0); }

// Shared-memory bytes of the query staging area.
template <typename T, int D, int MODE, int GQ>
constexpr int q_stage_bytes() {
    // MODE 0 / 1: one copy of the query mean per warp; rows of 1 KB and more (one CTA per SM, every byte of
    // shared memory wanted by the ring) share a single copy
    return MODE == 2 ? GQ * D * 4 : (MODE == 3 ? GQ * D * 2 : (D * (int)sizeof(T) >= 1024 ? 1 : kWarps) * D * (int)sizeof(T));
}

// The gather-and-score loop of one warp.  KPL > 0: the warp's best 32 * KPL keys stay in `run` (registers);
// KPL == 0: every key goes to keys[] in shared memory (MODE 0, 3) or every score to sbuf / global (MODE 2, 1).
template <typename T, int D, int MODE, int GQ, int KPL, int SLOTS, int SLOT_B, int LPRX, typename Issue>
__device__ __forceinline__ void score_rows(const IndexerArgs& a, Issue& issue, const int my_batches, const int warp,
                                           const int lane, const unsigned char* my_ring, const T* qv, const float* qf32,
                                           typename KeyOf<T>::type* keys, __nv_bfloat16* sbuf, const int beg,
                                           const int lo, const int cnt,
                                           typename KeyOf<T>::type (&run)[KPL > 0 ? KPL : 1]) {
    using Key = typename KeyOf<T>::type;
    using Gm = Geom<T, D, LPRX>;
    constexpr int NQ = MODE >= 2 ? GQ : 1;
    constexpr int LPR = Gm::lpr;               // lanes per row
    constexpr int L = Gm::L, HALF = L / LPR;   // partial sums of a row; those this thread owns
    constexpr int KP = KPL > 0 ? KPL : 1;
    const int r_in = lane / LPR, par = lane % LPR;  // row of the slot; residue of the partial sums this thread owns
    Key pend[KP];
#pragma unroll
    for (int r = 0; r < KP; ++r) pend[r] = (Key)0;
    int filled = 0;  // batches whose keys sit in pend
    for (int ord = 0; ord < my_batches; ++ord) {
        cp_async_wait<SLOTS - 2>();
        __syncwarp();
        if (ord + SLOTS - 1 < my_batches) issue(ord + SLOTS - 1);
        cp_async_commit();
        const unsigned char* row_ptr = my_ring + (size_t)(ord % SLOTS) * SLOT_B + r_in * Gm::row_bytes;
        const int sw = Gm::swizzle(r_in);
        const int i = (warp + ord * kWarps) * Gm::rows_per_slot + r_in;  // position inside this CTA's chunk
        float best = -INFINITY;  // MODE 3: running maximum over the heads
        float row_score = 0.f;
#pragma unroll
        for (int g = 0; g < NQ; ++g) {
            float acc[HALF];
#pragma unroll
            for (int ii = 0; ii < HALF; ++ii) acc[ii] = 0.f;
            // this thread owns partial sums LPR*ii + par; partial l takes chunks l, l + L, ...
#pragma unroll
            for (int k = 0; k * L < Gm::nchunk; ++k) {
#pragma unroll
                for (int ii = 0; ii < HALF; ++ii) {
                    if (k * L + LPR * ii < Gm::nchunk) {  // nchunk is a multiple of LPR: the test holds for every residue
                        const int ch = k * L + LPR * ii + par;
                        // a chunk is ppc adjacent 16-byte pieces; the swizzle never flips piece bit 0
                        const T* src = reinterpret_cast<const T*>(row_ptr + (((ch * Gm::ppc) ^ sw) << 4));
                        if constexpr (MODE == 3)
                            add_quest_bounds(acc[ii], reinterpret_cast<const __nv_bfloat16*>(src),
                                             reinterpret_cast<const __nv_bfloat16*>(
                                                 reinterpret_cast<const unsigned char*>(src) + Gm::slot_bytes),
                                             reinterpret_cast<const __nv_bfloat16*>(qv) + g * D + ch * 8);
                        else if constexpr (MODE == 2)
                            add_products_f32(acc[ii], reinterpret_cast<const __nv_bfloat16*>(src),
                                             reinterpret_cast<const __nv_bfloat16*>(qf32) + g * D + ch * 8);
                        else
                            add_products(acc[ii], src, qv + ch * 8);
                    }
                }
            }
#pragma unroll
            for (int w = HALF / 2; w > 0; w >>= 1)
#pragma unroll
                for (int ii = 0; ii < w; ++ii) acc[ii] = __fadd_rn(acc[ii], acc[ii + w]);
            // the last folds (widths LPR/2 .. 1) cross the lanes of the row: v[i] += v[i + w] for i < w
            float total = acc[0];
#pragma unroll
            for (int w = LPR / 2; w > 0; w >>= 1) total = __fadd_rn(total, __shfl_xor_sync(0xffffffffu, total, w));
            const float sc = vtx::round_to<T>(total);
            if (MODE == 3) best = fmaxf(best, sc);
            else row_score = sc;
            if (par == 0 && i < cnt) {
                if (MODE == 2) sbuf[i * NQ + g] = __float2bfloat16_rn(sc);
                else if (MODE == 1) store_score<T>(reinterpret_cast<T*>(a.scores) + beg + lo + i, sc);
            }
        }
        if (MODE == 0 || MODE == 3) {
            const Key key = (par == 0 && i < cnt) ? KeyOf<T>::make(MODE == 3 ? best : row_score, lo + i) : (Key)0;
            if (KPL == 0) {
                if (par == 0 && i < cnt) keys[i] = key;
            } else {
                // LPR batches fill one 32-key row of pend: batch f of the row moves its keys (held by the lanes
                // of residue 0) to the lanes of residue f
                const int f = filled % LPR;
                const Key moved = __shfl_up_sync(0xffffffffu, key, f);
                const Key mine = par == f ? moved : (Key)0;
#pragma unroll
                for (int r = 0; r < KP; ++r)
                    if (r == filled / LPR) pend[r] = pend[r] | mine;  // disjoint lanes: OR keeps all batches
                if (++filled == LPR * KP) {
                    warp_topk_merge<Key, KP>(run, pend, lane);
#pragma unroll
                    for (int r = 0; r < KP; ++r) pend[r] = (Key)0;
                    filled = 0;
                }
            }
        }
    }
    if (KPL > 0 && filled > 0) warp_topk_merge<Key, KP>(run, pend, lane);
    cp_async_wait<0>();
}

// MODE 0: fused mean + GeMV + top-k.  MODE 1: GeMV only (scores to global memory).
// MODE 2 (bf16 only, GQ = query heads per KV head): the gqa_block_sparse_attention scores, i.e.
// per query head the fp32-product dot with the page's row rounded to bf16, a softmax of scale * score over
// the segment's candidates (canonical exp and sum) rounded to bf16, and the maximum over the heads.
// MODE 3 (bf16 only): the gqa_quest_sparse_attention scores from two summary caches (per-page max and min):
// per head sum_d max(round(q_d*max_d), round(q_d*min_d)) in the canonical order, rounded, maximum over heads.
// Returns true when this CTA leaves with the segment's page list complete (it is the only CTA of the
// segment, or the last of its chunks to arrive), false when it has nothing more to do for the segment.
template <typename T, int D, int MODE, typename HooksRef = NoHooks, int GQ = 1, int BAR = 0, int SLOTS_FORCE = 0,
          int LPRX = 2>
__device__ __forceinline__ bool indexer_body(const IndexerArgs& a, unsigned char* smem_raw, const int s, const int j,
                                             HooksRef hooks = HooksRef()) {
    using Hooks = typename std::remove_reference<HooksRef>::type;
    constexpr int NQ = MODE >= 2 ? GQ : 1;                          // score accumulators per row
    constexpr int NSRC = MODE == 3 ? 2 : 1;                         // summary rows gathered per page
    constexpr int QBYTES = q_stage_bytes<T, D, MODE, GQ>();
    using Key = typename KeyOf<T>::type;
    using Gm = Geom<T, D, LPRX>;
    constexpr int SLOT_B = NSRC * Gm::slot_bytes;
    constexpr int SLOTS = SLOTS_FORCE ? SLOTS_FORCE : ring_slots(SLOT_B);
    constexpr size_t RING_B = (size_t)kWarps * SLOTS * SLOT_B;
    static_assert(BAR != 0 || RING_B >= 2 * 2048 * sizeof(Key), "the idle ring doubles as the sort's exchange buffer");
    // layout: [ring][query staging][keys][ids]
    unsigned char* ring = smem_raw;
    T* qbar = reinterpret_cast<T*>(smem_raw + RING_B);
    Key* keys = reinterpret_cast<Key*>(reinterpret_cast<unsigned char*>(qbar) + QBYTES);
    int32_t* ids = reinterpret_cast<int32_t*>(keys + a.key_cap);
    __nv_bfloat16* sbuf = reinterpret_cast<__nv_bfloat16*>(ids + a.key_cap);  // MODE 2: [candidate][head] scores
    float* qf32 = reinterpret_cast<float*>(qbar);                               // MODE 2: [head][D]
    __shared__ int s_last_arrival;
    // as a phase of a larger CTA (BAR > 0) the body's threads are numbered within their group of kThreads
    const int tix = BAR == 0 ? (int)threadIdx.x : (int)(threadIdx.x & (kThreads - 1));
    const int warp = tix >> 5, lane = tix & 31;

    const int beg = a.dense_indptr[s] + a.bos;
    const int c = a.dense_indptr[s + 1] - a.eos - beg;  // candidates of the whole segment
    // a.chunk > 0: chunks of that many candidates; a.chunk < 0: -a.chunk chunks of equal length per segment
    const int chunk_len = a.chunk >= 0 ? a.chunk : (c + (-a.chunk) - 1) / (-a.chunk);
    const bool split = MODE != 2 && chunk_len > 0 && c > chunk_len;
    const int nch = split ? (c + chunk_len - 1) / chunk_len : 1;
    if (j >= nch) return false;
    const bool overflow = split ? (nch > a.nch_max || chunk_len > a.key_cap) : (MODE != 1 && c > a.key_cap);
    if (c <= a.K || overflow) {
        // Nothing to select (the block-table builder already wrote the whole list), or more candidates than
        // the caller's max_num_pages_per_request promised (shared memory or the grid cannot hold them: flag it
        // and select the first K candidates so that the list stays well defined).
        if (j != 0) return false;
        hooks.wait();
        const typename Hooks::Regs hr = hooks.load(warp, lane);
        hooks.finish(warp, lane, hr, nullptr);
        if (c > a.K) {
            if (tix == 0 && a.status) atomicOr(a.status, (uint32_t)VTX_STATUS_CANDIDATE_OVERFLOW);
            if (MODE != 1) {
                const int o0 = a.sparse_indptr[s] + a.bos;
                for (int e = tix; e < a.K; e += kThreads) {
                    const int32_t row = a.dense_indices[beg + e];
                    a.sparse_indices[o0 + e] = row;
                    if (a.sparse_pt) a.sparse_pt[(int64_t)s * a.pt_stride + a.bos + e] = row;
                }
            }
        }
        return true;
    }
    const int lo = split ? j * chunk_len : 0;           // this CTA's candidates: [lo, lo + cnt)
    const int cnt = split ? min(chunk_len, c - lo) : c;
    // Wide rows (1 KB and more: one CTA per SM, registers to spare, many query heads): the heads' chunks this
    // thread will average are requested now, so that their round trip overlaps the dependent loads below
    // (segment bounds -> row ids -> first gathers) instead of following them.
    constexpr bool WIDE = MODE < 2 && Gm::row_bytes >= 1024 && std::is_same<Hooks, NoHooks>::value;
    constexpr int GW = 16;
    vtx::Vec8<T> qpre[WIDE ? GW : 1];
    if constexpr (WIDE) {
        if (tix < Gm::nchunk) {
            const T* qs = reinterpret_cast<const T*>(a.q) + (int64_t)s * a.G * D + tix * 8;
#pragma unroll
            for (int g = 0; g < GW; ++g)
                if (g < a.G) qpre[g].load_cached(qs + (int64_t)g * D);
        }
    }
    const int32_t* row_ids = a.dense_indices + beg + lo;
    if (MODE != 1) {
        for (int i = tix; i < cnt; i += kThreads) ids[i] = row_ids[i];
        row_ids = ids;
    }
    body_sync<BAR>();  // row ids are staged

    unsigned char* my_ring = ring + (size_t)warp * SLOTS * SLOT_B;
    const uint32_t my_ring_addr = (uint32_t)__cvta_generic_to_shared(my_ring);
    const unsigned char* cent = reinterpret_cast<const unsigned char*>(a.centroids);
    const unsigned char* cent2 = reinterpret_cast<const unsigned char*>(a.centroids2);
    const int n_batches = (cnt + Gm::rows_per_slot - 1) / Gm::rows_per_slot;
    const int my_batches = n_batches > warp ? (n_batches - warp + kWarps - 1) / kWarps : 0;
    constexpr int pieces_per_slot = Gm::rows_per_slot * Gm::pieces;

    auto issue = [&](int ord) {
        const int row0 = (warp + ord * kWarps) * Gm::rows_per_slot;
        const uint32_t dst = my_ring_addr + (uint32_t)((ord % SLOTS) * SLOT_B);
        if constexpr (Gm::pieces == 16 && MODE != 1) {
            // 256-byte rows: a lane takes one 16-byte piece of RPL consecutive rows (lanes 0-15 the first half of
            // the batch, lanes 16-31 the second), so that its row ids are 16-byte reads of the staged list and the
            // swizzle of its k-th row is a constant of the unrolled loop
            constexpr int RPL = Gm::rows_per_slot / 2;  // 8, or 4 with four lanes per row
            static_assert(RPL % 4 == 0, "row ids are read four at a time");
            const int rbase = (lane >> 4) * RPL, pr = lane & 15;
            const int i0 = row0 + rbase;
            int rid[RPL];
            if (i0 + RPL <= cnt) {
#pragma unroll
                for (int k = 0; k < RPL; k += 4) {
                    const int4 v = *reinterpret_cast<const int4*>(row_ids + i0 + k);
                    rid[k] = v.x; rid[k + 1] = v.y; rid[k + 2] = v.z; rid[k + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int k = 0; k < RPL; ++k) rid[k] = i0 + k < cnt ? row_ids[i0 + k] : -1;
            }
            const unsigned char* src = cent + pr * 16;
            const uint32_t d0 = dst + (uint32_t)(rbase * Gm::row_bytes);
#pragma unroll
            for (int k = 0; k < RPL; ++k) {
                const bool valid = i0 + k < cnt;
                const int64_t row = valid ? VTX_CHECK_SUMMARY_ROW(rid[k]) : 0;
                const uint32_t off = k * Gm::row_bytes + ((pr ^ Gm::swizzle(k)) << 4);  // swizzle(rbase + k) == swizzle(k)
                cp_async16(d0 + off, src + row * Gm::row_bytes, valid);
                if (NSRC == 2) cp_async16(d0 + Gm::slot_bytes + off, cent2 + row * Gm::row_bytes + pr * 16, valid);
            }
            return;
        }
#pragma unroll
        for (int pc = lane; pc < pieces_per_slot; pc += 32) {
            const int r = pc / Gm::pieces, pr = pc - r * Gm::pieces;
            const int i = row0 + r;
            const bool valid = i < cnt;
            const int64_t row = valid ? VTX_CHECK_SUMMARY_ROW(row_ids[i]) : 0;
            const uint32_t off = r * Gm::row_bytes + ((pr ^ Gm::swizzle(r)) << 4);
            cp_async16(dst + off, cent + row * Gm::row_bytes + pr * 16, valid);
            if (NSRC == 2) cp_async16(dst + Gm::slot_bytes + off, cent2 + row * Gm::row_bytes + pr * 16, valid);
        }
    };

    // prologue: SLOTS - 1 batches in flight; the last slot stays free until the loop's first iteration
    const uint32_t spare_addr = my_ring_addr + (uint32_t)((SLOTS - 1) * SLOT_B);
    const unsigned char* spare = my_ring + (size_t)(SLOTS - 1) * SLOT_B;
#pragma unroll
    for (int i = 0; i < SLOTS - 1; ++i) {
        if (i < my_batches) issue(i);
        if (i == SLOTS - 2) hooks.issue_extra(warp, lane, spare_addr);
        cp_async_commit();
    }
    hooks.wait();
    // Grouped-query mean.  Small groups: every warp computes it for itself (no block barrier between the wait
    // and the first score).  Large groups (many heads or a long latent): the CTA computes it once.
    const bool shared_q = MODE < 2 && (a.G * Gm::nchunk > 4 * 32 || Gm::row_bytes >= 1024);
    T* my_q = qbar + ((MODE < 2 && !shared_q) ? warp * D : 0);
    if constexpr (MODE < 2) {
        // one canonical chunk per thread and pass; all loads of a pass are issued before anything is stored
        const typename Hooks::Regs hr = hooks.load(warp, lane);
        constexpr int GMAX = 8;
        const int tid = shared_q ? tix : lane, nthr = shared_q ? kThreads : 32;
        for (int ch0 = 0; ch0 < Gm::nchunk; ch0 += nthr) {
            const int ch = ch0 + tid;
            const T* qs = reinterpret_cast<const T*>(a.q) + (int64_t)s * a.G * D + ch * 8;
            float acc[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) acc[jj] = 0.f;
            if (ch < Gm::nchunk) {
                int g_first = 0;
                if constexpr (WIDE) {
                    if (ch0 == 0) {  // this pass's first GW heads are already in registers (same order of additions)
#pragma unroll
                        for (int g = 0; g < GW; ++g) {
                            if (g < a.G) {
                                float f[8];
                                qpre[g].unpack(f);
#pragma unroll
                                for (int jj = 0; jj < 8; ++jj) acc[jj] = __fadd_rn(acc[jj], f[jj]);
                            }
                        }
                        g_first = GW;
                    }
                }
                for (int g0 = g_first; g0 < a.G; g0 += GMAX) {
                    vtx::Vec8<T> v[GMAX];
#pragma unroll
                    for (int g = 0; g < GMAX; ++g)
                        if (g0 + g < a.G) v[g].load_cached(qs + (int64_t)(g0 + g) * D);
#pragma unroll
                    for (int g = 0; g < GMAX; ++g) {
                        if (g0 + g < a.G) {
                            float f[8];
                            v[g].unpack(f);
#pragma unroll
                            for (int jj = 0; jj < 8; ++jj) acc[jj] = __fadd_rn(acc[jj], f[jj]);
                        }
                    }
                }
                const float g_f = (float)a.G;
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) acc[jj] = __fdiv_rn(acc[jj], g_f);
                vtx::store8(my_q + ch * 8, acc);  // rounds once to T
            }
        }
        if (hooks.needs_spare(warp)) cp_async_wait<0>();  // the copies of issue_extra have landed (this lane's part)
        __syncwarp();                                      // ... every lane's part; the warp's query mean is staged
        hooks.finish(warp, lane, hr, spare);
        if (shared_q) body_sync<BAR>();                    // the CTA's query mean is staged
        else __syncwarp();                                 // the spare slot may be refilled from here on
    } else {
        const typename Hooks::Regs hr = hooks.load(warp, lane);
        if (MODE == 3) {  // the group's query heads as they are
            const uint4* qs = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.q) + (int64_t)s * GQ * D);
            for (int ch = threadIdx.x; ch < GQ * Gm::nchunk; ch += kThreads) reinterpret_cast<uint4*>(qbar)[ch] = qs[ch];
        } else {          // the group's query heads as they are (the products are formed in fp32, see add_products_f32)
            const uint4* qs = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.q) + (int64_t)s * GQ * D);
            for (int ch = threadIdx.x; ch < GQ * Gm::nchunk; ch += kThreads) reinterpret_cast<uint4*>(qbar)[ch] = qs[ch];
        }
        if (hooks.needs_spare(warp)) cp_async_wait<0>();
        __syncwarp();
        hooks.finish(warp, lane, hr, spare);
        __syncthreads();  // the query heads are staged
    }

    const int kpl = (MODE == 0 || MODE == 3) ? stream_kpl(a.K) : 0;
    Key run1[1] = {(Key)0}, run2[2] = {(Key)0, (Key)0};
    if (kpl == 1)
        score_rows<T, D, MODE, GQ, 1, SLOTS, SLOT_B, LPRX>(a, issue, my_batches, warp, lane, my_ring, my_q, qf32, keys, sbuf, beg, lo,
                                                     cnt, run1);
    else if (kpl == 2)
        score_rows<T, D, MODE, GQ, 2, SLOTS, SLOT_B, LPRX>(a, issue, my_batches, warp, lane, my_ring, my_q, qf32, keys, sbuf, beg, lo,
                                                     cnt, run2);
    else
        score_rows<T, D, MODE, GQ, 0, SLOTS, SLOT_B, LPRX>(a, issue, my_batches, warp, lane, my_ring, my_q, qf32, keys, sbuf, beg, lo,
                                                     cnt, run1);
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
        // the maximum is exact in any order: warp shuffles, then the warps' results through shared memory
#pragma unroll
        for (int g = 0; g < NQ; ++g) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx[g] = fmaxf(mx[g], __shfl_xor_sync(0xffffffffu, mx[g], o));
            if (lane == 0) red[g * kWarps + warp] = mx[g];
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < NQ; ++g) {
            float m = red[g * kWarps];
#pragma unroll
            for (int w = 1; w < kWarps; ++w) m = fmaxf(m, red[g * kWarps + w]);
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
        const int o0 = a.sparse_indptr[s] + a.bos;
        // this segment's chunks (as a phase of a larger CTA, part_keys is that CTA's own scratch)
        Key* part = reinterpret_cast<Key*>(a.part_keys) + (BAR != 0 ? (size_t)0 : (size_t)s * a.nch_max * a.K);
        EmitSelection<T> emit;
        emit.part = part + (size_t)j * a.K;
        emit.ids = split ? a.dense_indices + beg : ids;  // keys name candidates by their position in the segment
        emit.out = a.sparse_indices + o0;
        emit.out_pt = a.sparse_pt ? a.sparse_pt + (int64_t)s * a.pt_stride + a.bos : nullptr;
        emit.to_scratch = split;
        bool merged = false;  // this CTA's own keys are dealt with
        if (kpl > 0) {
            // every warp holds its best 32 * kpl keys in registers: hand them over through keys[] and let warp 0
            // fold the four sorted lists into one (each fold: elementwise maximum against the reversed other
            // list, then one bitonic merge)
            const int n = 32 * kpl;
            if (kpl == 1) keys[warp * n + lane] = run1[0];
            else { keys[warp * n + lane * 2] = run2[0]; keys[warp * n + lane * 2 + 1] = run2[1]; }
            body_sync<BAR>();  // lists are visible, every ring is idle
            if (!split) hooks.pre_sort(0);
            if (warp == 0) {
                if (kpl == 1) {
#pragma unroll
                    for (int w = 1; w < kWarps; ++w) {
                        const Key o = keys[w * n + 31 - lane];
                        run1[0] = run1[0] > o ? run1[0] : o;
                        warp_bitonic_desc<Key, 1>(run1, lane, 32);
                    }
                    if (lane < a.K) emit(lane, run1[0]);
                } else {
#pragma unroll
                    for (int w = 1; w < kWarps; ++w) {
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const Key o = keys[w * n + (31 - lane) * 2 + (1 - r)];
                            run2[r] = run2[r] > o ? run2[r] : o;
                        }
                        warp_bitonic_desc<Key, 2>(run2, lane, 64);
                    }
#pragma unroll
                    for (int r = 0; r < 2; ++r)
                        if (lane * 2 + r < a.K) emit(lane * 2 + r, run2[r]);
                }
            }
            merged = true;
            if (!split) return true;  // the caller's block barrier publishes the list to the CTA
        } else {
            __syncthreads();  // all keys written, every ring is idle: its space becomes the sort's scratch
        }
        // As a phase of another kernel only the streaming form above exists (MODE 0, K <= 64, no split: the
        // host checks); the block-wide sorts below use the CTA barrier.
        if constexpr (BAR != 0) return true;
        int n_sort = cnt;
        bool partial = split;
        for (;;) {
            if (!merged) {
                const int xoff = partial ? 0 : hooks.pre_sort(n_sort);
                emit.to_scratch = partial;
                sort_emit<Key>(keys, n_sort, a.K, reinterpret_cast<Key*>(smem_raw + xoff), emit);
                if (!partial) break;
            }
            merged = false;
            // publish this chunk's keys, then find out whether every other chunk of the segment is in
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const int t = atomicAdd(a.tickets + s, 1);
                const int last = t == nch - 1;
                if (last) a.tickets[s] = 0;  // every chunk has counted itself: ready for the next launch
                __threadfence();
                s_last_arrival = last;
            }
            __syncthreads();
            if (!s_last_arrival) return false;
            n_sort = nch * a.K;
            for (int i = threadIdx.x; i < n_sort; i += kThreads) keys[i] = __ldcg(part + i);
            __syncthreads();
            partial = false;
        }
    }
    return true;
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

int check_common(const int32_t* dip, const int32_t* din, int eff_bs, int K, int bos, int eos, int maxp,
                 int dtype) {
    if (!dip || !din) return VTX_ERR_INVALID_ARGUMENT;
    if (eff_bs < 0 || K < 1 || bos < 0 || eos < 0 || maxp < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    if (maxp > kMaxCandidates) return VTX_ERR_UNSUPPORTED;
    return VTX_OK;
}

// Candidate capacity of one segment (sizes the key and row-id arrays in shared memory).
int key_capacity(int max_pages) { return vtx::pow2_ceil(max_pages < 256 ? 256 : max_pages); }  // >= 4 warps x 64 keys

// Candidates one CTA scans when a workspace allows a segment's scan to be split: 512, or 768 for small batches
// (fewer than ~1.5 segments per CTA slot of the GPU), where fewer, longer chunks keep the whole grid in one wave.
// A function of the batch size alone, so that the workspace size is known before the lengths are.
inline int chunk_rows(int eff_bs) { return eff_bs <= 384 ? 768 : 512; }

int split_chunks(int eff_bs, int max_pages, int bos, int eos) {
    const int cand = max_pages - bos - eos, chunk = chunk_rows(eff_bs);
    return cand > chunk ? (cand + chunk - 1) / chunk : 1;
}

int64_t split_workspace_bytes(int eff_bs, int max_pages, int K, int bos, int eos) {
    const int nch = split_chunks(eff_bs, max_pages, bos, eos);
    if (nch == 1) return 0;
    const int64_t tickets = ((int64_t)eff_bs * 4 + 255) / 256 * 256;
    return tickets + (int64_t)eff_bs * nch * K * 8;  // keys are at most 8 bytes
}

// Fill the split fields of `a` (and shrink its key capacity to one chunk) when the caller's workspace
// allows it; otherwise leave the one-CTA-per-segment form.
void plan_split(IndexerArgs& a, int eff_bs, int max_pages, void* workspace, int64_t workspace_bytes) {
    a.status = vtx::device_status_word();
    const int nch = split_chunks(eff_bs, max_pages, a.bos, a.eos), chunk = chunk_rows(eff_bs);
    if (workspace == nullptr || nch == 1) return;
    if (workspace_bytes < split_workspace_bytes(eff_bs, max_pages, a.K, a.bos, a.eos)) return;
    a.chunk = chunk;
    a.nch_max = nch;
    a.key_cap = vtx::pow2_ceil(nch * a.K > chunk ? nch * a.K : chunk);
    a.tickets = reinterpret_cast<int32_t*>(workspace);
    a.part_keys = reinterpret_cast<unsigned char*>(workspace) + ((int64_t)eff_bs * 4 + 255) / 256 * 256;
}

}  // namespace
