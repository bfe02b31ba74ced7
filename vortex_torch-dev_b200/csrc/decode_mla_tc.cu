// Block-table decode attention over a shared compressed latent, on the 5th-generation tensor cores.
//
// 16 query heads share one 576-dim latent row per token: keys are the whole row, values its first 512
// dims.  The reference project has no such kernel; the block-table inputs are the ones its planner
// produces (csrc/utils_sglang.cu:949-1083: page table [bs, stride] and per-request sequence lengths).
//
// One CTA per request walks the request's tokens in tiles of 64.  Both products are written with the
// tokens or the value dims as the M side of a tcgen05.mma, so the 16 heads are the N side and nothing is
// padded:
//   S^T[token, head] = K . Q^T      64 x 16 x 16: A = latent tile, K-major (dims contiguous), B = q, 36 k-steps
//   O^T[dim,  head] += V^T . P^T    128 x 16 x 16: A = the same tile read MN-major (dims are M), B = P^T, 4 x 4 k-steps
// A latent tile sits in shared memory as nine blocks of 64 tokens x 64 dims (128-byte swizzle).  It is
// fetched once, by three TMA copies through a 3-d view of the cache [64 dims][tokens][9 blocks]: two
// "quads" of four value blocks (32 KB, two 128-dim groups of the PV product each) and the rope block.
// Few large copies matter: a copy costs the issuing thread ~0.2 us, and nine 8 KB copies per tile capped
// the kernel at two thirds of the HBM rate that three copies reach.  The quad ring holds 3 tiles: with
// less, a copy could only be issued about one tile time before its data is needed, which is less than an
// HBM round trip under load.
// Accumulators live in TMEM: S^T twice, as four partial sums of 16 columns each (an M = 64 product puts
// rows 16w..16w+15 in lanes 32w..32w+15), and O^T (64 columns, lane = dim).
//
// Warp roles: warps 0 and 7 issue the TMA copies (quads, rope), warps 1 and 6 the MMAs (S^T, PV) from one
// elected lane each, warps 2-5 do
// the online softmax in fp32: S^T out of TMEM, per-head maxima over the tile, P^T as bf16 into shared
// memory, O^T rescaled in TMEM only when a maximum moved, and the final normalisation.
// All hand-offs are mbarriers; every wait is bounded and, when it gives up, raises a fault word that the
// host can read, drains the copies in flight and leaves through the common exit that frees TMEM.
#include <cuda.h>

#include "indexer_body.cuh"
#include "vtx_common.cuh"

namespace {
namespace mla {  // own scope: the indexer body included above has constants of the same names for its 128 threads

using vtxidx::IndexerArgs;

constexpr int kHeads = 16;
constexpr int kDl = 576;                  // latent row: keys
constexpr int kDv = 512;                  // leading dims: values
constexpr int kTile = 64;                 // tokens per tile
constexpr int kBlockDims = 64;            // dims per block: one 128-byte swizzle row
constexpr int kBlockB = kTile * 128;      // 8 KB: 64 tokens x 64 dims
constexpr int kQuadB = 4 * kBlockB;       // 32 KB: 256 dims of the values
constexpr int kQuadSlots = 6;             // a tile holds 2
constexpr int kRopeSlots = 1;             // read first by the S^T product, so it is free again a tile ahead of its next use
constexpr int kRopeAhead = 3;             // tiles whose rope block is pulled into L2 ahead of its copy
constexpr int kQB = kHeads * kDl * 2;     // 18 KB: 9 blocks of 16 heads x 64 dims
constexpr int kPB = kHeads * kTile * 2;   // 2 KB: 16 heads x 64 tokens
constexpr int kThreads = 256;            // warps: 0 TMA quads, 1 S^T issue, 2-5 softmax, 6 PV issue, 7 TMA rope
constexpr int kSoftmaxThreads = 128;
constexpr uint32_t kTmemCols = 512;
constexpr int kAcc = 5;  // partial S^T accumulators per buffer: k-step j of every value block adds into accumulator j,
                         // the rope block (issued by the other MMA warp) into accumulator 4
constexpr int kSBufs = 3;  // S^T buffers: the rope part of tile i + 1 is issued before the quads of tile i
constexpr uint32_t kColS = 0, kColO = kSBufs * kAcc * 16;
constexpr float kLog2e = 1.4426950408889634f;

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr int kOffQuads = 0;
constexpr int kOffRope = kOffQuads + kQuadSlots * kQuadB;
constexpr int kOffQ = kOffRope + kRopeSlots * kBlockB;
constexpr int kOffP = kOffQ + kQB;
constexpr int kOffWmax = kOffP + kPB;                   // [2][4 warps][16] floats
constexpr int kOffWsum = kOffWmax + 2 * 4 * 16 * 4;     // [4 warps][16] floats
constexpr int kOffBars = kOffWsum + 4 * 16 * 4;
enum Bar {
    kFullQuad = 0,
    kEmptyQuad = kFullQuad + kQuadSlots,
    kFullRope = kEmptyQuad + kQuadSlots,
    kEmptyRope = kFullRope + kRopeSlots,
    kSFull = kEmptyRope + kRopeSlots,  // kSBufs
    kSFree = kSFull + kSBufs,          // kSBufs
    kPFull = kSFree + kSBufs,
    kODone,
    kFixed,
    kQReady,
    kNumBars
};
constexpr int kOffMisc = kOffBars + kNumBars * 8;       // tmem base (u32), abort flag (int)
constexpr int kSmemBytes = kOffMisc + 16 + 1024;        // + slack for the manual 1024-byte alignment
static_assert(kSmemBytes <= 227 * 1024, "over the shared memory of one CTA");

__device__ unsigned int g_mla_fault = 0;  // sticky: a bounded wait gave up (bit = which barrier kind)

struct TcArgs {
    const __nv_bfloat16* q;   // [bs, 16, 576]
    __nv_bfloat16* out;       // [bs, 16, 512]
    const int32_t* page_table;
    int64_t pt_stride;
    const int32_t* seqlens;
    int P;                    // tokens per page
    int box_tok;              // tokens per TMA box: min(P, 64)
    float scale_log2;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// non-blocking test (try_wait may suspend the thread for a while before it answers)
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2 s of SM clocks or as soon as another thread of the CTA has given up.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned code) {
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > 4000000000ll) {
            *abort_flag = 1;
            atomicOr(&g_mla_fault, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned code) {
    if (mbar_test(bar, parity)) return true;  // a try_wait costs ~140 cycles even when the phase is already complete
    if (mbar_try(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, code);
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

// the same box fetched into L2 only (no shared-memory slot involved)
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// the same load without the wait: the registers are valid only after tmem_wait_ld()
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, float (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]),
          "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15])
        : "r"(taddr)
        : "memory");
}
// Wait for the loads in flight; naming the registers as in/out operands keeps every use of them below the wait.
__device__ __forceinline__ void tmem_wait_ld(float (&v)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]), "+f"(v[4]), "+f"(v[5]), "+f"(v[6]), "+f"(v[7]),
                   "+f"(v[8]), "+f"(v[9]), "+f"(v[10]), "+f"(v[11]), "+f"(v[12]), "+f"(v[13]), "+f"(v[14]), "+f"(v[15])
                 :
                 : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
          "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
          "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15]))
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] . B[smem], one M x 16 x 16 bf16 product issued by the calling thread
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle.  `lbo`: byte distance between 64-element groups
// along M/N (MN-major operands only); `sbo`: byte distance between groups of 8 rows (K-major) or of 8
// k-indices (MN-major).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulate, bf16 operands, N = 16; M in bits 24-28; bit 15 set = A is MN-major.
constexpr uint32_t kIdescBase = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17);
constexpr uint32_t kIdescQK = kIdescBase | ((64u >> 4) << 24);
constexpr uint32_t kIdescPV = kIdescBase | ((128u >> 4) << 24) | (1u << 15);

// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
        "elect.sync rx|px, 0xffffffff;\n\t"
        "@px mov.s32 %0, 1;\n\t}"
        : "+r"(pred));
    return pred != 0;
}

// 2^x on the special-function unit (2^-inf = 0)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ int float_key(float x) {  // order-preserving map to signed int
    const int i = __float_as_int(x);
    return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float key_float(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7fffffff)); }

// fault codes (bits of g_mla_fault): which kind of barrier a wait gave up on
enum : unsigned { kFaultEmpty = 1, kFaultFull = 2, kFaultS = 4, kFaultP = 8, kFaultO = 16, kFaultFixed = 32, kFaultQ = 64, kFaultDrain = 128 };

// The selection phase of the fused form: four lanes per row (8-row batches of 9 KB) and two batches per warp, so
// that two instances fit under the decode's idle tile ring.  Eight lanes per row with five 4-row batches per warp
// fit too and select the same pages, but are no faster (69.0 against 68.4 us on 128 requests of 256 candidate
// pages): while it streams, the scan already moves 5.5 TB/s; its cost is the latency before and after.
constexpr int kFusedLpr = 4, kFusedSlots = 2;
// Shared memory of one instance of the indexer body in the fused form: ring (kFusedSlots per warp), query mean,
// keys and row ids of its candidates; rounded up so that the next instance starts 128-byte aligned.
__host__ __device__ inline size_t fused_instance_bytes(int key_cap) {
    using Gm = Geom<__nv_bfloat16, kDl, kFusedLpr>;
    const size_t n = (size_t)4 * kFusedSlots * Gm::slot_bytes + (size_t)q_stage_bytes<__nv_bfloat16, kDl, 0, 1>() +
                     (size_t)key_cap * (sizeof(KeyOf<__nv_bfloat16>::type) + sizeof(int32_t));
    return (n + 127) & ~(size_t)127;
}

// FUSED: the request's page selection (query mean over the heads, scores of its candidate pages' summary rows,
// top-K; the body of the stand-alone indexer kernel) runs first, on warps 0-3 with the tile ring as its scratch,
// and writes the page-table row the decode then walks.  One launch instead of two, and none of the second
// launch's start-up between the selection and the first tile.
// FUSED = the ring slots per warp of that phase (3, or 2 when the candidates' keys need the room), 0 = decode only.
template <int FUSED>
__global__ void __launch_bounds__(kThreads, 1) decode_mla_tc_kernel(TcArgs a, const IndexerArgs ia,
                                                                         const __grid_constant__ CUtensorMap quad_map,
                                                                         const __grid_constant__ CUtensorMap block_map) {
    extern __shared__ unsigned char smem_unaligned[];
    // Under programmatic dependent launch the set-up below (barriers, TMEM) touches nothing the preceding
    // launch could still be writing, so it runs ahead of the wait; every global access comes after it.
    vtx::pdl_trigger();

    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_unaligned);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* gbase = smem_unaligned + (base - raw);
    const uint32_t bars = base + kOffBars;
    auto bar = [&](int which) { return bars + 8u * (uint32_t)which; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kOffMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + kOffMisc + 4);

    const int b = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kQuadSlots; ++i) { mbar_init(bar(kFullQuad + i), 1); mbar_init(bar(kEmptyQuad + i), 1); }
        for (int i = 0; i < kRopeSlots; ++i) { mbar_init(bar(kFullRope + i), 1); mbar_init(bar(kEmptyRope + i), 1); }
        for (int i = 0; i < kSBufs; ++i) { mbar_init(bar(kSFull + i), 2); mbar_init(bar(kSFree + i), kSoftmaxThreads); }
        mbar_init(bar(kPFull), kSoftmaxThreads);
        mbar_init(bar(kODone), 1);
        mbar_init(bar(kFixed), kSoftmaxThreads);
        mbar_init(bar(kQReady), kSoftmaxThreads);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(base + kOffMisc, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    vtx::pdl_wait();
    if constexpr (FUSED != 0) {
        // The pages the planner reserved (the request's first and last page: entries 0 and n - 1 of its page-table
        // row, written before this launch) will be read by the decode whatever the selection finds.  Their tiles
        // are pulled into L2 now: HBM is idle while every CTA of the launch walks the dependent loads that open
        // the selection (segment bounds -> row ids -> first gathers), and the decode then finds them in L2.
        if (warp == 7 && a.P == kTile && lane < 2 * 9) {
            const int nt = (a.seqlens[b] + kTile - 1) / kTile;
            const int which = lane / 9, blk = lane - which * 9;
            const int entry = which == 0 ? 0 : nt - 1;
            if ((which == 0 ? ia.bos > 0 : (ia.eos > 0 && nt > 1)) && nt > 0)
                tma_prefetch_2d(&block_map, blk * kBlockDims, a.page_table[(int64_t)b * a.pt_stride + entry] * a.P);
        }
        // The ring and the q / P areas are idle until the first copy is issued below; barriers, the TMEM slot and
        // the abort flag live behind them (kOffBars) and stay untouched: the host checked that everything used
        // here ends before kOffWmax.  Two instances of the indexer body, warps 0-3 on the first half of the
        // request's candidate pages and warps 4-7 on the second, each with its own ring, query mean and named
        // barrier; each leaves the K best keys of its half in `part`, and warp 0 orders the union.
        using Key = KeyOf<__nv_bfloat16>::type;
        const int inst = warp >> 2;
        const size_t inst_bytes = fused_instance_bytes(ia.key_cap);
        unsigned char* scratch = gbase + kOffQuads + (size_t)inst * inst_bytes;
        Key* part = reinterpret_cast<Key*>(gbase + kOffQuads + 2 * inst_bytes);
        IndexerArgs mine = ia;
        mine.part_keys = part;
        indexer_body<__nv_bfloat16, kDl, 0, NoHooks, 1, /*BAR=*/2, kFusedSlots, kFusedLpr>(mine, scratch, b, inst);  // barriers 2, 3
        __syncthreads();  // both halves' keys are in `part` (or the whole list was written: nothing to select)
        const int beg = ia.dense_indptr[b] + ia.bos;
        const int c = ia.dense_indptr[b + 1] - ia.eos - beg;
        const int half = (c + 1) / 2;
        if (warp == 0 && c > ia.K && half <= ia.key_cap) {  // else: nothing to select, or the body's overflow path ran
            // 2 K keys (K <= 64) as 2 or 4 per lane; a full sort; the first K name the selected candidates
            EmitSelection<__nv_bfloat16> emit;
            emit.to_scratch = false;
            emit.part = nullptr;
            emit.ids = ia.dense_indices + beg;  // keys name candidates by their position in the segment
            emit.out = ia.sparse_indices + ia.sparse_indptr[b] + ia.bos;
            emit.out_pt = ia.sparse_pt ? ia.sparse_pt + (int64_t)b * ia.pt_stride + ia.bos : nullptr;
            if (ia.K <= 32) {
                Key u[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int e = lane * 2 + r, h = e >> 5, k = e & 31;  // 32 places per half, K of them filled
                    u[r] = k < ia.K ? part[h * ia.K + k] : (Key)0;
                }
                warp_bitonic_desc<Key, 2>(u, lane, 2);
#pragma unroll
                for (int r = 0; r < 2; ++r)
                    if (lane * 2 + r < ia.K) emit(lane * 2 + r, u[r]);
            } else {
                Key u[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int e = lane * 4 + r, h = e >> 6, k = e & 63;
                    u[r] = k < ia.K ? part[h * ia.K + k] : (Key)0;
                }
                warp_bitonic_desc<Key, 4>(u, lane, 2);
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (lane * 4 + r < ia.K) emit(lane * 4 + r, u[r]);
            }
        }
        __syncthreads();  // the page-table row of this request is complete and visible to the CTA
    }
    const int ntok = a.seqlens[b];
    const int n_tiles = (ntok + kTile - 1) / kTile;
    const bool last_partial = (ntok % kTile) != 0;

    if (warp == 0 || warp == 7) {
        // ================================================= TMA producers.  Three units per tile: rope (block 8), quad 0
        // (blocks 0-3), quad 1 (blocks 4-7).  Warp 0 streams the quads, warp 7 the rope blocks: two queues, so
        // that a wait for the single rope slot never holds back the quads behind it.  Pages of 64 tokens or more: one copy per unit from an elected
        // lane.  Smaller pages: a unit is (blocks x boxes) copies of [64 dims x page] spread over the lanes.
        const int nb = kTile / a.box_tok;
        const bool big_pages = nb == 1;
        unsigned armed = 0, armed_parity = 0;  // per full barrier: armed at least once, parity of the last use
        bool ok = true;
        auto box_row = [&](int tile, int box) -> int {  // first cache row (token index in the whole cache) of a box
            const int tok = tile * kTile + box * a.box_tok;
            if (tok >= ntok) return -1;
            const int page = tok / a.P;
            return a.page_table[(int64_t)b * a.pt_stride + page] * a.P + (tok - page * a.P);
        };
        // this lane's box of the tile: the only box (big pages) or box lane % nb
        // The single rope slot makes "rope part of S^T(i) done -> slot free -> copy of block i + 1 -> rope part of
        // S^T(i + 1)" a chain with one memory round trip per tile.  Pulling the rope blocks of the next tiles
        // into L2 ahead of time (8 KB per tile) shortens that round trip from an HBM access to an L2 hit.
        auto prefetch_rope = [&](int tile) {
            if (warp != 7 || tile >= n_tiles) return;
            const int yp = box_row(tile, big_pages ? 0 : lane % nb);
            if (yp >= 0 && (big_pages ? lane == 0 : lane < nb)) tma_prefetch_2d(&block_map, 8 * kBlockDims, yp);
            __syncwarp();
        };
        for (int t = 1; t <= kRopeAhead; ++t) prefetch_rope(t);
        int y_next = n_tiles > 0 ? box_row(0, big_pages ? 0 : lane % nb) : -1;
        for (int i = 0; i < n_tiles && ok; ++i) {
            const int y = y_next;
            if (i + 1 < n_tiles) y_next = box_row(i + 1, big_pages ? 0 : lane % nb);
            prefetch_rope(i + 1 + kRopeAhead);
            const int left = ntok - i * kTile;
            const int nload = left >= kTile ? nb : (left + a.box_tok - 1) / a.box_tok;
            const uint32_t block_bytes = (uint32_t)nload * a.box_tok * 128u;
            for (int u = (warp == 7 ? 0 : 1); u < (warp == 7 ? 1 : 3) && ok; ++u) {
                const bool rope = u == 0;
                const int idx = rope ? i : 2 * i + u - 1, nslots = rope ? kRopeSlots : kQuadSlots;
                const int slot = idx % nslots, use = idx / nslots;
                const int full = (rope ? kFullRope : kFullQuad) + slot, empty = (rope ? kEmptyRope : kEmptyQuad) + slot;
                if (use > 0) ok = mbar_wait(bar(empty), (use - 1) & 1, abort_flag, kFaultEmpty);
                ok = __all_sync(0xffffffffu, ok) != 0;
                if (!ok) break;
                armed |= 1u << full;
                armed_parity = (armed_parity & ~(1u << full)) | ((unsigned)(use & 1) << full);
                const uint32_t dst = base + (rope ? kOffRope + slot * kBlockB : kOffQuads + slot * kQuadB);
                const int nblk = rope ? 1 : 4, blk0 = rope ? 8 : 4 * (u - 1);
                if (big_pages) {
                    if (elect_one()) {
                        mbar_arrive_expect_tx(bar(full), block_bytes * nblk);
                        if (rope) tma_load_2d(dst, &block_map, 8 * kBlockDims, y, bar(full));
                        else tma_load_3d(dst, &quad_map, 0, y, blk0, bar(full));
                    }
                } else {
                    if (lane == 0) mbar_arrive_expect_tx(bar(full), block_bytes * nblk);
                    __syncwarp();
                    // copy c of the unit: block c / nb, box c % nb; lanes with the same lane % nb share a box row
                    for (int c = lane; c < nblk * nb; c += 32) {
                        const int blk = c / nb, box = c % nb;
                        if (box < nload)
                            tma_load_2d(dst + blk * kBlockB + box * a.box_tok * 128, &block_map, (blk0 + blk) * kBlockDims,
                                        y, bar(full));
                    }
                }
                __syncwarp();
            }
        }
        if (*abort_flag && lane == 0) {
            // leaving early: wait (bounded) until the copies already issued have landed
            for (int f = 0; f < kEmptyRope; ++f) {
                if (f >= kEmptyQuad && f < kFullRope) continue;
                if (!(armed >> f & 1)) continue;
                const long long t0 = clock64();
                while (!mbar_try(bar(f), armed_parity >> f & 1))
                    if (clock64() - t0 > 200000000ll) { atomicOr(&g_mla_fault, kFaultDrain); break; }
            }
        }
    } else if (warp == 1 || warp == 6) {
        // ================================================= MMA issuers: warp 1 the S^T products, warp 6 the PV
        // products.  Two warps, so that PV(i) never queues behind a wait for the next tile's data and S^T(i + 1)
        // never behind the softmax of tile i.  The whole warp walks the loop and waits; one elected lane issues
        // (the elect.sync form lets the descriptors live in uniform registers, which more than halves the cost
        // of an issue compared with a lane-0 branch).
        if (n_tiles > 0) {
            bool ok = true;
            auto wait_all = [&](int which, uint32_t parity, unsigned code) {
                ok = ok && mbar_wait(bar(which), parity, abort_flag, code);
                ok = __all_sync(0xffffffffu, ok) != 0;
                return ok;
            };
            wait_all(kQReady, 0, kFaultQ);  // both issuers read q
            // descriptors: constant high part + (byte address >> 4)
            const uint64_t dk = smem_desc(0, 0, 1024), dmn = smem_desc(0, kBlockB, 1024);
            const uint64_t qd = dk + ((base + kOffQ) >> 4), pd = dk + ((base + kOffP) >> 4);
            auto is_partial = [&](int i) { return last_partial && i == n_tiles - 1; };
            // S^T of tile i goes into buffer i % 3 in two parts, each by its own warp: the two quads (32 k-steps;
            // k-step j of every block into accumulator j) from warp 1, the rope block (4 k-steps into accumulator
            // 4, then the commit that releases the rope slot) from warp 6 between its PV products.  Each part
            // ends with a commit on the buffer's "full" barrier, which expects both.  A last tile that is not
            // full is ready, as a whole, once the softmax warps have zeroed its tail.
            auto part_wait = [&](int i, int part) {
                if (is_partial(i)) return wait_all(kFixed, 0, kFaultFixed);
                if (part == 0) return wait_all(kFullRope + i % kRopeSlots, (i / kRopeSlots) & 1, kFaultFull);
                return wait_all(kFullQuad + (2 * i + part - 1) % kQuadSlots, ((2 * i + part - 1) / kQuadSlots) & 1, kFaultFull);
            };
            // S^T buffer i % 3 was last read by the softmax of tile i - 3
            auto sbuf_free = [&](int i) {
                return i < kSBufs || wait_all(kSFree + i % kSBufs, ((i - kSBufs) / kSBufs) & 1, kFaultS);
            };
            auto part_issue = [&](int i, int part) {  // part 0: the rope block; part 1: both quads
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t sd = tmem + kColS + (i % kSBufs) * kAcc * 16;
                    if (part > 0) {
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const uint64_t ad = dk + ((base + kOffQuads + ((2 * i + u) % kQuadSlots) * kQuadB) >> 4);
#pragma unroll
                            for (int blk = 0; blk < 4; ++blk)
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    umma(sd + j * 16, ad + ((blk * kBlockB + j * 32) >> 4),
                                         qd + (((4 * u + blk) * 2048 + j * 32) >> 4), kIdescQK, (u | blk) != 0 ? 1u : 0u);
                        }
                    } else {
                        const int rslot = i % kRopeSlots;
                        const uint64_t ad = dk + ((base + kOffRope + rslot * kBlockB) >> 4);
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            umma(sd + 4 * 16, ad + ((j * 32) >> 4), qd + ((8 * 2048 + j * 32) >> 4), kIdescQK, j != 0 ? 1u : 0u);
                        umma_commit(bar(kEmptyRope + rslot));
                    }
                    umma_commit(bar(kSFull + i % kSBufs));  // one of the two arrivals that publish S^T
                }
                __syncwarp();
            };
            if (warp == 1) {
                // one issue block for both quads of a tile: every wait / fence / elect / commit round costs the
                // issuing warp some hundreds of cycles, about as much as the 32 products themselves
                for (int i = 0; i < n_tiles && ok; ++i)
                    if (sbuf_free(i) && part_wait(i, 1) && part_wait(i, 2)) part_issue(i, 1);
            }
            auto rope_part = [&](int i) {
                if (sbuf_free(i) && part_wait(i, 0)) part_issue(i, 0);
            };
            if (warp == 6) rope_part(0);
            for (int i = 0; i < n_tiles && ok && warp == 6; ++i) {
                // the next tile's rope part first: its block has been in flight for a tile time, and the sooner
                // it is consumed the sooner the single rope slot takes the block after it
                if (i + 1 < n_tiles) rope_part(i + 1);
                if (!ok || !wait_all(kPFull, i & 1, kFaultP)) break;
                tc_fence_after();
                const int slot0 = (2 * i) % kQuadSlots, slot1 = (2 * i + 1) % kQuadSlots;
                if (elect_one()) {
                    // 128-dim group g: blocks 2g, 2g+1 = the lower or upper half of quad g / 2
                    const uint32_t ga[4] = {base + kOffQuads + slot0 * kQuadB, base + kOffQuads + slot0 * kQuadB + 2 * kBlockB,
                                            base + kOffQuads + slot1 * kQuadB, base + kOffQuads + slot1 * kQuadB + 2 * kBlockB};
                    // quad by quad, so that the first one is released half a product earlier
#pragma unroll
                    for (int qd2 = 0; qd2 < 2; ++qd2) {
#pragma unroll
                        for (int t = 0; t < kTile / 16; ++t)
#pragma unroll
                            for (int g = 2 * qd2; g < 2 * qd2 + 2; ++g)
                                umma(tmem + kColO + g * 16, dmn + ((ga[g] + t * 2048) >> 4),
                                     pd + ((t * 32) >> 4), kIdescPV, (i | t) != 0 ? 1u : 0u);
                        umma_commit(bar(kEmptyQuad + (qd2 == 0 ? slot0 : slot1)));
                    }
                    umma_commit(bar(kODone));
                }
                __syncwarp();
            }
        }
    } else {
        // ================================================= softmax warps: thread <-> TMEM lane `row`
        // A thread whose wait gave up keeps going through the motions (later waits fail at once) so that
        // the named barrier below always gets its 128 arrivals.
        // S^T: lanes 0-15 of warp quarter q4 hold tokens 16*q4 .. 16*q4+15 of the tile (lanes 16-31 idle there);
        // O^T: thread <-> dim row 32*q4 + lane of each 128-dim group.
        const int q4 = warp & 3, row = q4 * 32 + lane, st = threadIdx.x - 64;
        const int trow = q4 * 16 + (lane & 15);
        const bool tlive = lane < 16;
        const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
        __nv_bfloat16* ob = a.out + (int64_t)b * kHeads * kDv;
        if (n_tiles == 0) {
            for (int i = st; i < kHeads * kDv; i += kSoftmaxThreads) ob[i] = __float2bfloat16_rn(0.f);
        } else {
            // ---- q as the B operand of S^T: 9 blocks of [16 heads][64 dims], 16-byte chunks swizzled by head
            {
                const uint4* qsrc = reinterpret_cast<const uint4*>(a.q + (int64_t)b * kHeads * kDl);
#pragma unroll
                for (int it = 0; it < kQB / 16 / kSoftmaxThreads; ++it) {
                    const int c = it * kSoftmaxThreads + st;
                    const int h = c / 72, cr = c - h * 72, kb = cr >> 3, ck = cr & 7;
                    *reinterpret_cast<uint4*>(gbase + kOffQ + kb * 2048 + h * 128 + ((ck ^ (h & 7)) << 4)) = qsrc[c];
                }
                fence_proxy_async();
                mbar_arrive(bar(kQReady));
            }
            // ---- a last tile that is not full: once it has landed, zero the rows past the end of the
            // request (unwritten cache rows may hold anything, and 0 x NaN would poison the PV product)
            auto zero_tail = [&](int i) {
                bool ok = true;
                for (int u = 0; u < 2 && ok; ++u) {
                    const int idx = 2 * i + u;
                    ok = mbar_wait(bar(kFullQuad + idx % kQuadSlots), (idx / kQuadSlots) & 1, abort_flag, kFaultFull);
                }
                ok = ok && mbar_wait(bar(kFullRope + i % kRopeSlots), (i / kRopeSlots) & 1, abort_flag, kFaultFull);
                if (ok && tlive && i * kTile + trow >= ntok) {
                    const uint4 z = make_uint4(0, 0, 0, 0);
                    for (int blk = 0; blk < 8; ++blk) {
                        unsigned char* p = gbase + kOffQuads + ((2 * i + (blk >> 2)) % kQuadSlots) * kQuadB +
                                           (blk & 3) * kBlockB + trow * 128;
#pragma unroll
                        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(p + c * 16) = z;
                    }
                    unsigned char* p = gbase + kOffRope + (i % kRopeSlots) * kBlockB + trow * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(p + c * 16) = z;
                }
                fence_proxy_async();
                mbar_arrive(bar(kFixed));
            };
            if (last_partial && n_tiles == 1) zero_tail(0);

            float m[kHeads], l[kHeads];
#pragma unroll
            for (int h = 0; h < kHeads; ++h) { m[h] = -INFINITY; l[h] = 0.f; }
            float* wmax = reinterpret_cast<float*>(gbase + kOffWmax);

            for (int i = 0; i < n_tiles; ++i) {
                const int buf = i % kSBufs;
                if (last_partial && i + 1 == n_tiles - 1) zero_tail(i + 1);
                mbar_wait(bar(kSFull + buf), (i / kSBufs) & 1, abort_flag, kFaultS);
                tc_fence_after();
                float s[kHeads];
                {
                    float part[kAcc][kHeads];  // the five partial sums, one round trip to TMEM
#pragma unroll
                    for (int acc = 0; acc < kAcc; ++acc) tmem_ld16_nowait(tlane + kColS + (buf * kAcc + acc) * 16, part[acc]);
#pragma unroll
                    for (int acc = 0; acc < kAcc; ++acc) tmem_wait_ld(part[acc]);
#pragma unroll
                    for (int h = 0; h < kHeads; ++h) s[h] = ((part[0][h] + part[1][h]) + (part[2][h] + part[3][h])) + part[4][h];
                }
                tc_fence_before();
                mbar_arrive(bar(kSFree + buf));
                const bool valid = tlive && i * kTile + trow < ntok;
                int key[kHeads];
#pragma unroll
                for (int h = 0; h < kHeads; ++h) {
                    s[h] = valid ? s[h] * a.scale_log2 : -INFINITY;
                    key[h] = __reduce_max_sync(0xffffffffu, float_key(s[h]));
                }
                if (lane == 0) {
                    float4* w = reinterpret_cast<float4*>(wmax + ((i & 1) * 4 + q4) * 16);
#pragma unroll
                    for (int h4 = 0; h4 < 4; ++h4)
                        w[h4] = make_float4(key_float(key[4 * h4]), key_float(key[4 * h4 + 1]),
                                            key_float(key[4 * h4 + 2]), key_float(key[4 * h4 + 3]));
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                // every tile holds at least one token of the request, so the new maxima are finite
                float alpha[kHeads];
                bool moved = false;
#pragma unroll
                for (int h4 = 0; h4 < 4; ++h4) {
                    float4 t = *reinterpret_cast<const float4*>(wmax + ((i & 1) * 4 + 0) * 16 + 4 * h4);
#pragma unroll
                    for (int w = 1; w < 4; ++w) {
                        const float4 u = *reinterpret_cast<const float4*>(wmax + ((i & 1) * 4 + w) * 16 + 4 * h4);
                        t.x = fmaxf(t.x, u.x); t.y = fmaxf(t.y, u.y); t.z = fmaxf(t.z, u.z); t.w = fmaxf(t.w, u.w);
                    }
                    const float tm[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int h = 4 * h4 + k;
                        alpha[h] = fmaxf(m[h], tm[k]);  // the new maximum for now
                        moved |= alpha[h] != m[h];
                    }
                }
                if (moved) {  // same decision in every thread: they all hold the same maxima
#pragma unroll
                    for (int h = 0; h < kHeads; ++h) {
                        const float mn = alpha[h];
                        alpha[h] = ex2(m[h] - mn);
                        l[h] *= alpha[h];
                        m[h] = mn;
                    }
                }
#pragma unroll
                for (int h = 0; h < kHeads; ++h) {
                    s[h] = ex2(s[h] - m[h]);
                    l[h] += s[h];
                }
                if (i > 0) {
                    // the previous PV product must be complete before P^T is overwritten or O^T rescaled
                    mbar_wait(bar(kODone), (i - 1) & 1, abort_flag, kFaultO);
                    tc_fence_after();
                    if (moved) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            float o[kHeads];
                            tmem_ld16(tlane + kColO + g * 16, o);
#pragma unroll
                            for (int h = 0; h < kHeads; ++h) o[h] *= alpha[h];
                            tmem_st16(tlane + kColO + g * 16, o);
                        }
                        tmem_wait_st();
                    }
                }
                // P^T as the B operand of O^T: [16 heads][64 tokens], 16-byte chunks swizzled by head
                if (tlive) {
                    unsigned char* p = gbase + kOffP + (trow & 7) * 2;
                    const int chunk = trow >> 3;
#pragma unroll
                    for (int h = 0; h < kHeads; ++h)
                        *reinterpret_cast<__nv_bfloat16*>(p + h * 128 + ((chunk ^ (h & 7)) << 4)) = __float2bfloat16_rn(s[h]);
                }
                fence_proxy_async();
                tc_fence_before();
                mbar_arrive(bar(kPFull));
            }

            // ---- epilogue: row sums over the 128 token threads, then O^T / l out of TMEM
#pragma unroll
            for (int h = 0; h < kHeads; ++h)
#pragma unroll
                for (int w = 16; w >= 1; w >>= 1) l[h] += __shfl_xor_sync(0xffffffffu, l[h], w);
            float* wsum = reinterpret_cast<float*>(gbase + kOffWsum);
            if (lane == 0) {
#pragma unroll
                for (int h4 = 0; h4 < 4; ++h4)
                    *reinterpret_cast<float4*>(wsum + q4 * 16 + 4 * h4) = make_float4(l[4 * h4], l[4 * h4 + 1], l[4 * h4 + 2], l[4 * h4 + 3]);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            float inv[kHeads];
#pragma unroll
            for (int h = 0; h < kHeads; ++h) {
                const float t = (wsum[h] + wsum[16 + h]) + (wsum[32 + h] + wsum[48 + h]);
                inv[h] = t > 0.f ? 1.f / t : 0.f;
            }
            const bool done = mbar_wait(bar(kODone), (n_tiles - 1) & 1, abort_flag, kFaultO);
            tc_fence_after();
            if (done) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float o[kHeads];
                    tmem_ld16(tlane + kColO + g * 16, o);
#pragma unroll
                    for (int h = 0; h < kHeads; ++h)
                        ob[h * kDv + g * 128 + row] = __float2bfloat16_rn(o[h] * inv[h]);
                }
            }
        }
    }
    // ================================================= common exit: every tcgen05 access is done, free TMEM
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

}  // namespace mla
}  // namespace

namespace vtx {

bool mla_tc_supported(int page_size) {
    return page_size >= 16 && (page_size & (page_size - 1)) == 0 && mla::encode_tiled_fn() != nullptr;
}

// Launches the tcgen05 form.  `num_cache_pages` bounds the token rows the tensor map may address.
static int launch_tc(const void* q, const void* latent_cache, int64_t num_cache_pages, void* out,
                     const int32_t* page_table, int64_t page_table_stride, const int32_t* cache_seqlens,
                     int batch_size, int page_size, float sm_scale, const vtxidx::IndexerArgs* ia, int ring_slots_fused,
                     cudaStream_t stream) {
    const int box_tok = page_size < mla::kTile ? page_size : mla::kTile;
    const cuuint64_t tokens = (cuuint64_t)num_cache_pages * (cuuint64_t)page_size;
    if (tokens == 0 || tokens > 0x7fffffffull) return VTX_ERR_INVALID_ARGUMENT;
    void* gaddr = const_cast<void*>(latent_cache);
    // 2-d view [576 dims][tokens], box = one block of one page-box; 3-d view [64 dims][tokens][9 blocks], box = 4 blocks
    CUtensorMap block_map, quad_map;
    {
        const cuuint64_t gdim[2] = {(cuuint64_t)mla::kDl, tokens};
        const cuuint64_t gstride[1] = {(cuuint64_t)mla::kDl * 2};
        const cuuint32_t box[2] = {(cuuint32_t)mla::kBlockDims, (cuuint32_t)box_tok};
        const cuuint32_t estr[2] = {1, 1};
        if (mla::encode_tiled_fn()(&block_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, gaddr, gdim, gstride, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return VTX_ERR_INVALID_ARGUMENT;
    }
    {
        const cuuint64_t gdim[3] = {(cuuint64_t)mla::kBlockDims, tokens, (cuuint64_t)(mla::kDl / mla::kBlockDims)};
        const cuuint64_t gstride[2] = {(cuuint64_t)mla::kDl * 2, (cuuint64_t)mla::kBlockDims * 2};
        const cuuint32_t box[3] = {(cuuint32_t)mla::kBlockDims, (cuuint32_t)box_tok, 4};
        const cuuint32_t estr[3] = {1, 1, 1};
        if (mla::encode_tiled_fn()(&quad_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, gaddr, gdim, gstride, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return VTX_ERR_INVALID_ARGUMENT;
    }
    mla::TcArgs a;
    a.q = (const __nv_bfloat16*)q;
    a.out = (__nv_bfloat16*)out;
    a.page_table = page_table;
    a.pt_stride = page_table_stride;
    a.seqlens = cache_seqlens;
    a.P = page_size;
    a.box_tok = box_tok;
    a.scale_log2 = sm_scale * mla::kLog2e;
    (void)ring_slots_fused;
    auto kern = !ia ? mla::decode_mla_tc_kernel<0> : mla::decode_mla_tc_kernel<2>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, mla::kSmemBytes);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        return VTX_ERR_CUDA;
    }
    return launch(kern, dim3(batch_size), dim3(mla::kThreads), (size_t)mla::kSmemBytes, stream, a,
                  ia ? *ia : vtxidx::IndexerArgs{}, quad_map, block_map);
}

int launch_decode_mla_tc(const void* q, const void* latent_cache, int64_t num_cache_pages, void* out,
                         const int32_t* page_table, int64_t page_table_stride, const int32_t* cache_seqlens,
                         int batch_size, int page_size, float sm_scale, cudaStream_t stream) {
    return launch_tc(q, latent_cache, num_cache_pages, out, page_table, page_table_stride, cache_seqlens, batch_size,
                     page_size, sm_scale, nullptr, 0, stream);
}

// Page selection + decode in one launch.  VTX_ERR_UNSUPPORTED when the selection cannot run as a phase of the
// decode kernel (more than 64 pages to select, or more candidates than its scratch holds): the caller then
// issues the two launches.
int launch_mla_sparse_layer_tc(const void* q, const void* summary, const void* latent_cache, int64_t num_cache_pages,
                               void* out, const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                               const int32_t* dense_kv_indices, int32_t* sparse_kv_indices, int32_t* sparse_page_table,
                               int64_t page_table_stride, const int32_t* sparse_cache_seqlens, int batch_size,
                               int page_size, int topk_val, int bos, int eos, int max_pages, float sm_scale,
                               cudaStream_t stream) {
    vtxidx::IndexerArgs ia{};
    ia.q = q;
    ia.centroids = summary;
    ia.dense_indptr = dense_kv_indptr;
    ia.sparse_indptr = sparse_kv_indptr;
    ia.dense_indices = dense_kv_indices;
    ia.sparse_indices = sparse_kv_indices;
    ia.sparse_pt = sparse_page_table;
    ia.pt_stride = page_table_stride;
    ia.G = mla::kHeads;
    ia.D = mla::kDl;
    ia.K = topk_val;
    ia.bos = bos;
    ia.eos = eos;
    ia.key_cap = key_capacity(max_pages);
    ia.status = device_status_word();
    // every request's candidates are scanned in two halves by two instances of the body
    ia.chunk = -2;
    ia.nch_max = 2;
    ia.key_cap = key_capacity((max_pages + 1) / 2);  // keys and row ids of one half
    const int slots = 2;
    const size_t need = 2 * mla::fused_instance_bytes(ia.key_cap) + 2 * (size_t)topk_val * sizeof(KeyOf<__nv_bfloat16>::type);
    if (stream_kpl(topk_val) == 0 || need > (size_t)mla::kOffWmax) return VTX_ERR_UNSUPPORTED;
    return launch_tc(q, latent_cache, num_cache_pages, out, sparse_page_table, page_table_stride, sparse_cache_seqlens,
                     batch_size, page_size, sm_scale, &ia, slots, stream);
}

void* mla_fault_word() {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, mla::g_mla_fault) != cudaSuccess) return nullptr;
    return p;
}

}  // namespace vtx
