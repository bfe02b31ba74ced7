// Cache-side kernels: KV scatter (defines the paged layout) and the page-completion mean.
//
// Layout (cache/triton_kernels/set_kv.py:28-33 of the reference): K and V are separate
// buffers [num_pages, H, page_size, D]; token slot t of head h sits in flattened row
// (t / P) * H + h at token offset t % P, so one (page, head) block is contiguous.
#include <algorithm>

#include "vtx_common.cuh"

namespace {

// One thread moves 16 bytes of K and 16 bytes of V.
__global__ void __launch_bounds__(256) set_kv_kernel(uint4* __restrict__ k_cache, uint4* __restrict__ v_cache,
                                                    const uint4* __restrict__ new_k,
                                                    const uint4* __restrict__ new_v,
                                                    const int64_t* __restrict__ loc, int64_t nnz, int H,
                                                    int vec_per_row, int P) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int64_t total = nnz * H * vec_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % vec_per_row);
        const int64_t th = i / vec_per_row;
        const int h = (int)(th % H);
        const int64_t tok = th / H;
        const int64_t t = VTX_CHECK_LOC(loc[tok]);
        const int64_t dst = (((t / P) * H + h) * P + (t % P)) * vec_per_row + c;
        k_cache[dst] = new_k[i];
        v_cache[dst] = new_v[i];
    }
}

// A group of LANES threads owns one (new token, head) item; each lane owns chunks of eight
// columns and reduces the page's rows in ascending order.  OP 0: mean (fp32 accumulators that start at
// +0.0, one division by the row count, one rounding to T); OP 1 / 2: maximum / minimum (exact).
template <typename T, int LANES, int OP>
__global__ void __launch_bounds__(256) creduce_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                     const int64_t* __restrict__ loc, int64_t nnz, int H,
                                                     int rows, int cols, int P) {
    constexpr int GROUPS = 256 / LANES;
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int lane = threadIdx.x % LANES;
    const int64_t items = nnz * H;
    const int nchunk = cols / 8;
    const float denom = (float)rows;
    for (int64_t it = (int64_t)blockIdx.x * GROUPS + threadIdx.x / LANES; it < items;
         it += (int64_t)gridDim.x * GROUPS) {
        const int64_t t = VTX_CHECK_LOC(loc[it / H]);
        if ((t + 1) % P != 0) continue;
        const int h = (int)(it % H);
        const int64_t pid = (t / P) * H + h;
        const T* src = x + pid * (int64_t)rows * cols;
        for (int c = lane; c < nchunk; c += LANES) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = OP == 0 ? 0.f : (OP == 1 ? -INFINITY : INFINITY);
            for (int r = 0; r < rows; r += 8) {
                vtx::Vec8<T> v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (r + u < rows) v[u].load(src + (int64_t)(r + u) * cols + c * 8);
                    else v[u].zero();
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (r + u < rows) {
                        float f[8];
                        v[u].unpack(f);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            acc[j] = OP == 0 ? __fadd_rn(acc[j], f[j]) : (OP == 1 ? fmaxf(acc[j], f[j]) : fminf(acc[j], f[j]));
                    }
                }
            }
            if (OP == 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = __fdiv_rn(acc[j], denom);
            }
            vtx::store8(out + pid * (int64_t)cols + c * 8, acc);
        }
    }
}

// KV write fused with the centroid update of the pages the new tokens complete.
// One group of LANES threads per (new token, head); each lane owns chunks of eight columns.
// The mean adds the page's rows in ascending order, the new row (still in registers) last, so the result
// has the same bits as set_kv_kernel followed by the mean kernel.  An older row of the page is taken from
// the cache unless this same launch writes it: a launch may write several rows of one page (a prefill) as
// long as they are consecutive entries of loc in ascending slot order, in which case the row written by
// entry i - d sits d slots below entry i's slot and is read from new_k instead (the cache copy of that row
// may not have landed yet).
template <typename T, int LANES>
__global__ void __launch_bounds__(256) set_kv_cmean_kernel(T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                          const T* __restrict__ new_k, const T* __restrict__ new_v,
                                                          T* __restrict__ centroids, const int64_t* __restrict__ loc,
                                                          int64_t nnz, int H, int D, int P) {
    constexpr int GROUPS = 256 / LANES;
    vtx::pdl_wait();
    vtx::pdl_trigger();
    const int lane = threadIdx.x % LANES;
    const int64_t items = nnz * H;
    const int nchunk = D / 8;
    const float denom = (float)P;
    for (int64_t it = (int64_t)blockIdx.x * GROUPS + threadIdx.x / LANES; it < items;
         it += (int64_t)gridDim.x * GROUPS) {
        const int64_t idx = it / H;  // entry of loc
        const int64_t t = VTX_CHECK_LOC(loc[idx]);
        const int h = (int)(it % H);
        const int64_t pid = (t / P) * H + h;
        const int tok = (int)(t % P);
        T* kpage = k_cache + pid * (int64_t)P * D;
        T* vpage = v_cache + pid * (int64_t)P * D;
        const bool closes = tok == P - 1;
        // how many of the page's older rows this launch writes itself: entries idx-1, idx-2, ... while their
        // slots count down from t-1
        int own = 0;
        if (closes)
            while (own < P - 1 && idx - (own + 1) >= 0 && loc[idx - (own + 1)] == t - (own + 1)) ++own;
        for (int c = lane; c < nchunk; c += LANES) {
            vtx::Vec8<T> nk, nv;
            nk.load_cached(new_k + it * D + c * 8);
            nv.load_cached(new_v + it * D + c * 8);
            float kf[8], vf[8];
            nk.unpack(kf);
            nv.unpack(vf);
            vtx::store8(kpage + (int64_t)tok * D + c * 8, kf);  // values are already T-representable: exact copy
            vtx::store8(vpage + (int64_t)tok * D + c * 8, vf);
            if (!closes) continue;
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            // rows 0 .. P-2, eight loads in flight at a time (predicated tail): row r is P-1-r slots below
            for (int r = 0; r < P - 1; r += 8) {
                vtx::Vec8<T> v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int back = P - 1 - (r + u);
                    if (r + u >= P - 1) v[u].zero();
                    else if (back <= own) v[u].load_cached(new_k + ((idx - back) * H + h) * (int64_t)D + c * 8);
                    else v[u].load(kpage + (int64_t)(r + u) * D + c * 8);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (r + u < P - 1) {
                        float f[8];
                        v[u].unpack(f);
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], f[j]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = __fdiv_rn(__fadd_rn(acc[j], kf[j]), denom);
            vtx::store8(centroids + pid * (int64_t)D + c * 8, acc);
        }
    }
}

template <typename T>
int launch_set_kv_cmean(void* k, void* v, const void* nk, const void* nv, void* cent, const int64_t* loc,
                        int64_t nnz, int H, int D, int P, cudaStream_t st) {
    const int64_t items = nnz * H;
    if (D <= 128) {
        const int64_t blocks = (items + 15) / 16;
        return vtx::launch(set_kv_cmean_kernel<T, 16>, dim3((unsigned)std::min<int64_t>(blocks, 1 << 20)), dim3(256), 0, st,
                           (T*)k, (T*)v, (const T*)nk, (const T*)nv, (T*)cent, loc, nnz, H, D, P);
    } else {
        const int64_t blocks = (items + 7) / 8;
        return vtx::launch(set_kv_cmean_kernel<T, 32>, dim3((unsigned)std::min<int64_t>(blocks, 1 << 20)), dim3(256), 0, st,
                           (T*)k, (T*)v, (const T*)nk, (const T*)nv, (T*)cent, loc, nnz, H, D, P);
    }
    return vtx::finish_launch();
}

template <typename T, int OP>
int launch_creduce_op(const void* x, void* out, const int64_t* loc, int64_t nnz, int H, int rows, int cols, int P,
                      cudaStream_t st) {
    const int64_t items = nnz * H;
    if (cols <= 128) {
        const int64_t blocks = (items + 15) / 16;
        return vtx::launch(creduce_kernel<T, 16, OP>, dim3((unsigned)std::min<int64_t>(blocks, 1 << 20)), dim3(256), 0,
                           st, (const T*)x, (T*)out, loc, nnz, H, rows, cols, P);
    }
    const int64_t blocks = (items + 7) / 8;
    return vtx::launch(creduce_kernel<T, 32, OP>, dim3((unsigned)std::min<int64_t>(blocks, 1 << 20)), dim3(256), 0, st,
                       (const T*)x, (T*)out, loc, nnz, H, rows, cols, P);
}

template <typename T>
int launch_creduce(const void* x, void* out, const int64_t* loc, int64_t nnz, int H, int rows, int cols, int P,
                   int op, cudaStream_t st) {
    switch (op) {
        case 0: return launch_creduce_op<T, 0>(x, out, loc, nnz, H, rows, cols, P, st);
        case 1: return launch_creduce_op<T, 1>(x, out, loc, nnz, H, rows, cols, P, st);
        case 2: return launch_creduce_op<T, 2>(x, out, loc, nnz, H, rows, cols, P, st);
        default: return VTX_ERR_INVALID_ARGUMENT;
    }
}

}  // namespace

extern "C" int vtx_set_kv(void* k_cache, void* v_cache, const void* new_k, const void* new_v,
                          const int64_t* loc, int64_t nnz, int num_kv_heads, int head_dim, int page_size,
                          int dtype, void* stream) {
    if (!k_cache || !v_cache || !new_k || !new_v || !loc) return VTX_ERR_INVALID_ARGUMENT;
    if (nnz < 0 || num_kv_heads < 1 || head_dim < 1 || page_size < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    const int esize = dtype == VTX_BF16 ? 2 : 4;
    if ((head_dim * esize) % 16 != 0) return VTX_ERR_UNSUPPORTED;
    if (nnz == 0) return VTX_OK;
    const int vec_per_row = head_dim * esize / 16;
    const int64_t total = nnz * num_kv_heads * vec_per_row;
    const unsigned blocks = (unsigned)std::min<int64_t>((total + 255) / 256, 1 << 20);
    return vtx::launch(set_kv_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (uint4*)k_cache,
                       (uint4*)v_cache, (const uint4*)new_k, (const uint4*)new_v, loc, nnz, num_kv_heads,
                       vec_per_row, page_size);
}

extern "C" int vtx_creduce(const void* x, void* out, const int64_t* loc, int64_t nnz, int num_kv_heads, int rows,
                           int cols, int page_size, int op, int dtype, void* stream) {
    if (!x || !out || !loc) return VTX_ERR_INVALID_ARGUMENT;
    if (nnz < 0 || num_kv_heads < 1 || rows < 1 || cols < 1 || page_size < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (op < 0 || op > 2) return VTX_ERR_INVALID_ARGUMENT;
    if (cols % 8 != 0) return VTX_ERR_UNSUPPORTED;
    if (nnz == 0) return VTX_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == VTX_BF16)
        return launch_creduce<__nv_bfloat16>(x, out, loc, nnz, num_kv_heads, rows, cols, page_size, op, st);
    if (dtype == VTX_F32) return launch_creduce<float>(x, out, loc, nnz, num_kv_heads, rows, cols, page_size, op, st);
    return VTX_ERR_INVALID_ARGUMENT;
}

extern "C" int vtx_cmean(const void* x, void* out, const int64_t* loc, int64_t nnz, int num_kv_heads, int rows,
                         int cols, int page_size, int dtype, void* stream) {
    return vtx_creduce(x, out, loc, nnz, num_kv_heads, rows, cols, page_size, 0, dtype, stream);
}

extern "C" int vtx_set_kv_cmean(void* k_cache, void* v_cache, const void* new_k, const void* new_v,
                                void* centroids, const int64_t* loc, int64_t nnz, int num_kv_heads,
                                int head_dim, int page_size, int dtype, void* stream) {
    if (!k_cache || !v_cache || !new_k || !new_v || !centroids || !loc) return VTX_ERR_INVALID_ARGUMENT;
    if (nnz < 0 || num_kv_heads < 1 || head_dim < 1 || page_size < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (head_dim % 8 != 0) return VTX_ERR_UNSUPPORTED;
    if (nnz == 0) return VTX_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == VTX_BF16)
        return launch_set_kv_cmean<__nv_bfloat16>(k_cache, v_cache, new_k, new_v, centroids, loc, nnz, num_kv_heads,
                                                  head_dim, page_size, st);
    if (dtype == VTX_F32)
        return launch_set_kv_cmean<float>(k_cache, v_cache, new_k, new_v, centroids, loc, nnz, num_kv_heads,
                                          head_dim, page_size, st);
    return VTX_ERR_INVALID_ARGUMENT;
}
