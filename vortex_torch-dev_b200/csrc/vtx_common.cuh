// Shared device/host helpers for the vortex_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "vortex_b200.h"

namespace vtx {

// Records the text of a failing CUDA runtime call for vtx_last_cuda_error().
void note_cuda_error(cudaError_t e);

inline int finish_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error(e);
        return VTX_ERR_CUDA;
    }
    return VTX_OK;
}

// Programmatic dependent launch.  Every kernel of this library starts with pdl_wait() (all work of the
// preceding launch on the stream is complete and visible once it returns) followed by pdl_trigger()
// (the next launch may start placing its CTAs), so a launch never reads or writes anything before its
// predecessor has finished; what overlaps is only the launch latency and CTA start-up of the next kernel
// with the drain of the current one.  Both instructions are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- checked build (-DVTX_CHECKED, relocatable device code) ----
// Every index that a kernel reads from a caller's array and then uses as an address (a row of the K/V cache, a
// row of a page-summary cache, a token slot of ``loc`` or of the request-to-token table, a row of that table) goes
// through one of the VTX_CHECK_* macros.  In the checked build the macro compares the index with the limit set by
// vtx_checked_set_limits (a negative limit = not set = not compared); an index outside [0, limit) raises
// VTX_STATUS_BAD_ROW in the sticky status word and is replaced by 0, so the bad address is never touched and the
// kernel finishes.  In the normal build the macros are the identity and cost nothing.
#ifdef VTX_CHECKED
enum { kLimKvRows = 0, kLimSummaryRows = 1, kLimLocTokens = 2, kLimReqRows = 3, kNumLimits = 4 };
extern __device__ long long g_checked_limit[kNumLimits];
extern __device__ uint32_t g_checked_status;
__device__ __forceinline__ long long checked_index(long long idx, int which) {
    const long long lim = g_checked_limit[which];
    if (lim >= 0 && (idx < 0 || idx >= lim)) {
        atomicOr(&g_checked_status, (uint32_t)VTX_STATUS_BAD_ROW);
        return 0;
    }
    return idx;
}
#define VTX_CHECK_KV_ROW(i) ((int)vtx::checked_index((i), vtx::kLimKvRows))
#define VTX_CHECK_SUMMARY_ROW(i) ((int)vtx::checked_index((i), vtx::kLimSummaryRows))
#define VTX_CHECK_LOC(i) (vtx::checked_index((i), vtx::kLimLocTokens))
#define VTX_CHECK_REQ_ROW(i) (vtx::checked_index((i), vtx::kLimReqRows))
#else
#define VTX_CHECK_KV_ROW(i) (i)
#define VTX_CHECK_SUMMARY_ROW(i) (i)
#define VTX_CHECK_LOC(i) (i)
#define VTX_CHECK_REQ_ROW(i) (i)
#endif

bool programmatic_launch_enabled();
uint32_t* device_status_word();  // device address of the sticky status word on the current device, or null

template <typename... KArgs, typename... Args>
inline int launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = programmatic_launch_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        return VTX_ERR_CUDA;
    }
    return finish_launch();
}

// ---- asynchronous 16-byte global -> shared copies and warp-level tensor-core primitives ----
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr, bool valid) {
    const int src_bytes = valid ? 16 : 0;  // 0 => the 16 bytes are zero-filled, the source is not read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Page and in-page row of cache slot t (>= 0) for pages of P tokens.  A 64-bit division by a run-time P costs a
// thread on the order of a hundred instructions, and the cache kernels do one per (token, head) item: pages of
// a power of two take a shift and a mask, other sizes a 32-bit division while the slot fits 32 bits.
struct PageSlot {
    int64_t page;
    int row;
};
__device__ __forceinline__ PageSlot page_slot(int64_t t, int P) {
    PageSlot r;
    if ((P & (P - 1)) == 0) {
        r.page = t >> (31 - __clz(P));
        r.row = (int)(t & (int64_t)(P - 1));
    } else if ((uint64_t)t <= 0xffffffffull) {
        const uint32_t u = (uint32_t)t, q = u / (uint32_t)P;
        r.page = q;
        r.row = (int)(u - q * (uint32_t)P);
    } else {
        r.page = t / P;
        r.row = (int)(t % P);
    }
    return r;
}

// a / b and a % b for a >= 0, b > 0, with a 32-bit division whenever a fits 32 bits.
struct DivMod {
    int64_t q;
    int r;
};
__device__ __forceinline__ DivMod divmod(int64_t a, int b) {
    DivMod d;
    if ((uint64_t)a <= 0xffffffffull) {
        const uint32_t u = (uint32_t)a, q = u / (uint32_t)b;
        d.q = q;
        d.r = (int)(u - q * (uint32_t)b);
    } else {
        d.q = a / b;
        d.r = (int)(a % b);
    }
    return d;
}

__host__ __device__ inline int pow2_ceil(int n) {
    int p = 1;
    while (p < n) p <<= 1;
    return p;
}

// ---- streaming 16-byte loads (read-only path, no L1 allocation) ----
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// acc + (the bf16 value x widened to fp32), rounded to nearest even: the mixed-precision add of sm_100 does the
// (exact) widening and the addition in one instruction.
__device__ __forceinline__ float add_bf16(float acc, uint16_t x) {
    float d;
    asm("add.rn.f32.bf16 %0, %1, %2;" : "=f"(d) : "h"(x), "f"(acc));
    return d;
}
// acc0 += low half, acc1 += high half of a packed pair of bf16 values
__device__ __forceinline__ void add_bf16x2(float& acc0, float& acc1, uint32_t packed) {
    uint16_t lo, hi;
    asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(packed));
    acc0 = add_bf16(acc0, lo);
    acc1 = add_bf16(acc1, hi);
}

// Eight consecutive elements widened to fp32.
template <typename T>
struct Vec8;

template <>
struct Vec8<__nv_bfloat16> {
    uint4 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = ld_stream16(p); }
    __device__ __forceinline__ void load_cached(const __nv_bfloat16* p) {
        raw = *reinterpret_cast<const uint4*>(p);
    }
    __device__ __forceinline__ void zero() { raw = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
    __device__ __forceinline__ void unpack(float (&f)[8]) const {
        f[0] = bf16lo(raw.x); f[1] = bf16hi(raw.x);
        f[2] = bf16lo(raw.y); f[3] = bf16hi(raw.y);
        f[4] = bf16lo(raw.z); f[5] = bf16hi(raw.z);
        f[6] = bf16lo(raw.w); f[7] = bf16hi(raw.w);
    }
};

template <>
struct Vec8<float> {
    uint4 raw0, raw1;
    __device__ __forceinline__ void load(const float* p) {
        raw0 = ld_stream16(p);
        raw1 = ld_stream16(p + 4);
    }
    __device__ __forceinline__ void load_cached(const float* p) {
        raw0 = *reinterpret_cast<const uint4*>(p);
        raw1 = *reinterpret_cast<const uint4*>(p + 4);
    }
    __device__ __forceinline__ void zero() {
        raw0 = make_uint4(0, 0, 0, 0);
        raw1 = raw0;
    }
    __device__ __forceinline__ void store(float* p) const {
        *reinterpret_cast<uint4*>(p) = raw0;
        *reinterpret_cast<uint4*>(p + 4) = raw1;
    }
    __device__ __forceinline__ void unpack(float (&f)[8]) const {
        f[0] = __uint_as_float(raw0.x); f[1] = __uint_as_float(raw0.y);
        f[2] = __uint_as_float(raw0.z); f[3] = __uint_as_float(raw0.w);
        f[4] = __uint_as_float(raw1.x); f[5] = __uint_as_float(raw1.y);
        f[6] = __uint_as_float(raw1.z); f[7] = __uint_as_float(raw1.w);
    }
};

// Round fp32 to T (RNE) and store eight consecutive elements.
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 o;
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(f[2], f[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(f[4], f[5]);
    __nv_bfloat162 d = __floats2bfloat162_rn(f[6], f[7]);
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    o.z = *reinterpret_cast<uint32_t*>(&c);
    o.w = *reinterpret_cast<uint32_t*>(&d);
    *reinterpret_cast<uint4*>(p) = o;
}
__device__ __forceinline__ void store8(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

// Value of x after one rounding to T, widened back to fp32.
template <typename T>
__device__ __forceinline__ float round_to(float x);
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}
template <>
__device__ __forceinline__ float round_to<float>(float x) { return x; }

}  // namespace vtx
