// Paged grouped-query decode attention over each segment's page list.
//
// One CTA (4 warps) per (request, head) segment; warps take the listed pages round-robin.
// A (page, head) block of K or V is one contiguous run of page_size * D elements, so a warp
// reads it with 16-byte loads, LPT lanes per token row (each lane owns 8 head dims).  Softmax
// is the online (running max / running sum) form in fp32; partial results of the warps are
// merged through shared memory.  The last listed page contributes kv_last_page_len tokens.
//
// Data contract as produced by the block-table builder (reference: csrc/utils_sglang.cu:123-184,
// indexer/context.py:117-121); in the reference the attention itself is a third-party
// paged-decode call made with effective batch bs*H_kv, one KV head and group_size q heads.
#include "vtx_common.cuh"

namespace {

constexpr int kWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;

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

template <typename T>
__device__ __forceinline__ void store_out(T* p, float v);
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }

// LPT lanes per token row (D = 8 * LPT); UT token rows in flight per lane.
template <typename T, int G, int LPT, int UT>
__global__ void __launch_bounds__(kWarps * 32) decode_gqa_kernel(DecodeArgs a) {
    constexpr int D = LPT * 8;
    constexpr int TPW = 32 / LPT;  // token rows covered by one warp-wide load
    __shared__ float sm_acc[kWarps][G][D];
    __shared__ float sm_m[kWarps][G];
    __shared__ float sm_l[kWarps][G];

    const int s = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPT, tg = lane / LPT;
    const int beg = a.indptr[s];
    const int npages = a.indptr[s + 1] - beg;
    const int last_len = a.last_len[s];

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

    const T* kc = reinterpret_cast<const T*>(a.k);
    const T* vc = reinterpret_cast<const T*>(a.v);
    for (int pg = warp; pg < npages; pg += kWarps) {
        const int64_t row = a.indices[beg + pg];
        const int nvalid = (pg == npages - 1) ? last_len : a.P;
        const T* kp = kc + row * a.P * D + sub * 8;
        const T* vp = vc + row * a.P * D + sub * 8;
        for (int t0 = 0; t0 < nvalid; t0 += UT * TPW) {
            vtx::Vec8<T> kr[UT], vr[UT];
#pragma unroll
            for (int u = 0; u < UT; ++u) {
                const int t = t0 + u * TPW + tg;
                if (t < nvalid) kr[u].load(kp + (int64_t)t * D);
                else kr[u].zero();
            }
#pragma unroll
            for (int u = 0; u < UT; ++u) {
                const int t = t0 + u * TPW + tg;
                if (t < nvalid) vr[u].load(vp + (int64_t)t * D);
                else vr[u].zero();
            }
            float sc[UT][G];
#pragma unroll
            for (int u = 0; u < UT; ++u) {
                float f[8];
                kr[u].unpack(f);
                const bool valid = (t0 + u * TPW + tg) < nvalid;
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
                const float mn = fmaxf(m[g], cmax);  // finite: token t0 of this chunk is valid
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
#pragma unroll
            for (int u = 0; u < UT; ++u) {
                float f[8];
                vr[u].unpack(f);
#pragma unroll
                for (int g = 0; g < G; ++g) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(sc[u][g], f[j], acc[g][j]);
                }
            }
        }
    }

    // fold the token groups of the warp (they share m), then merge warps through shared memory
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
            for (int j = 0; j < 8; ++j) sm_acc[warp][g][sub * 8 + j] = acc[g][j];
            if (sub == 0) {
                sm_m[warp][g] = m[g];
                sm_l[warp][g] = l[g];
            }
        }
    }
    __syncthreads();
    T* out = reinterpret_cast<T*>(a.out) + (int64_t)s * G * D;
    for (int idx = threadIdx.x; idx < G * D; idx += kWarps * 32) {
        const int g = idx / D, d = idx % D;
        float mx = sm_m[0][g];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) mx = fmaxf(mx, sm_m[w][g]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float wm = sm_m[w][g];
            const float wgt = (wm == -INFINITY) ? 0.f : exp2f(wm - mx);
            num = fmaf(wgt, sm_acc[w][g][d], num);
            den = fmaf(wgt, sm_l[w][g], den);
        }
        store_out<T>(out + idx, den > 0.f ? num / den : 0.f);
    }
}

template <typename T, int G, int UT>
int launch_decode_g(const DecodeArgs& a, int eff_bs, int head_dim, cudaStream_t st) {
    switch (head_dim) {
        case 64: decode_gqa_kernel<T, G, 8, UT><<<eff_bs, kWarps * 32, 0, st>>>(a); break;
        case 128: decode_gqa_kernel<T, G, 16, UT><<<eff_bs, kWarps * 32, 0, st>>>(a); break;
        default: return VTX_ERR_UNSUPPORTED;
    }
    return vtx::finish_launch();
}

template <typename T, int UT>
int launch_decode(const DecodeArgs& a, int eff_bs, int group, int head_dim, cudaStream_t st) {
    switch (group) {
        case 1: return launch_decode_g<T, 1, UT>(a, eff_bs, head_dim, st);
        case 2: return launch_decode_g<T, 2, UT>(a, eff_bs, head_dim, st);
        case 4: return launch_decode_g<T, 4, UT>(a, eff_bs, head_dim, st);
        case 8: return launch_decode_g<T, 8, UT>(a, eff_bs, head_dim, st);
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
    if (dtype == VTX_BF16) return launch_decode<__nv_bfloat16, 8>(a, eff_batch_size, group_size, head_dim, st);
    if (dtype == VTX_F32) return launch_decode<float, 4>(a, eff_batch_size, group_size, head_dim, st);
    return VTX_ERR_INVALID_ARGUMENT;
}
