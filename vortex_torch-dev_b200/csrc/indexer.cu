// Indexer kernels: grouped-query mean, centroid GeMV and top-k page selection.
//
// One CTA per (request, head) segment.  The fused kernel keeps the segment's scores in
// shared memory as sortable keys, so they never travel to HBM; the stand-alone GeMV and
// top-k kernels exist for flows that call the operators one by one and produce the same
// bits.  Behaviour follows flow/algorithms.py:168-170, indexer/triton_kernels/mv_impl.py:53-62
// and csrc/topk.cu:56-113 of the reference.
//
// Canonical score arithmetic (shared with the CPU checker, so selections are bit-exact):
//   q_mean[d] = round_T( (q[0][d] + q[1][d] + ... in fp32, from +0.0) / G )
//   product   = round_T( centroid[d] * q_mean[d] )          (fp32 multiply, then rounding to T)
//   the D dims are cut in chunks of 8; LANES = min(32, pow2ceil(D/8)) partial sums; lane l adds
//   the products of chunks l, l+LANES, ... one by one in ascending order into an fp32
//   accumulator starting at +0.0 (no FMA); lanes are folded v[i] += v[i+w], w = LANES/2 .. 1;
//   score = round_T(sum).
// Selection order: score descending, ties by ascending candidate position (a stable
// descending sort), -0.0 equal to +0.0.
#include "vtx_common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxCandidates = 16384;

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

// Descending bitonic sort of n (power of two) keys in shared memory by the whole CTA.
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

// Sort the c keys of a segment and emit the first K row ids.
template <typename T>
__device__ void select_and_store(typename KeyOf<T>::type* keys, const int32_t* ids, int c, int K,
                                 int32_t* out, int32_t* out_pt) {
    using Key = typename KeyOf<T>::type;
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

struct IndexerArgs {
    const void* q;          // [eff_bs, G, D]
    const void* centroids;  // [rows, D]
    void* scores;           // packed, GEMV mode only
    const int32_t* dense_indptr;
    const int32_t* sparse_indptr;
    const int32_t* dense_indices;
    int32_t* sparse_indices;
    int32_t* sparse_pt;
    int64_t pt_stride;
    int G, D, K, bos, eos, key_cap;
};

// MODE 0: fused mean + GeMV + top-k.  MODE 1: GeMV only (scores to global memory).
template <typename T, int LANES, int CPL, int U, int MODE>
__global__ void __launch_bounds__(kThreads) indexer_kernel(IndexerArgs a) {
    using Key = typename KeyOf<T>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Key* keys = reinterpret_cast<Key*>(smem_raw);
    int32_t* ids = reinterpret_cast<int32_t*>(smem_raw + (size_t)a.key_cap * sizeof(Key));

    const int s = blockIdx.x;
    const int beg = a.dense_indptr[s] + a.bos;
    const int c = a.dense_indptr[s + 1] - a.eos - beg;
    if (c <= a.K) return;
    const int32_t* row_ids = a.dense_indices + beg;
    if (MODE == 0) {
        if (c > a.key_cap) return;  // more candidates than the caller sized shared memory for
        for (int i = threadIdx.x; i < c; i += kThreads) ids[i] = row_ids[i];
        row_ids = ids;
    }

    constexpr int NGRP = kThreads / LANES;
    const int lane = threadIdx.x % LANES, grp = threadIdx.x / LANES;
    const int nchunk = a.D / 8;

    // grouped-query mean for the chunks this lane owns
    float qm[CPL][8];
    {
        const T* qs = reinterpret_cast<const T*>(a.q) + (int64_t)s * a.G * a.D;
        const float g_f = (float)a.G;
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
            const int ch = lane + k * LANES;
#pragma unroll
            for (int j = 0; j < 8; ++j) qm[k][j] = 0.f;
            if (ch < nchunk) {
                for (int g = 0; g < a.G; ++g) {
                    vtx::Vec8<T> v;
                    v.load_cached(qs + (int64_t)g * a.D + ch * 8);
                    float f[8];
                    v.unpack(f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) qm[k][j] = __fadd_rn(qm[k][j], f[j]);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) qm[k][j] = vtx::round_to<T>(__fdiv_rn(qm[k][j], g_f));
            }
        }
    }
    __syncthreads();

    const T* cent = reinterpret_cast<const T*>(a.centroids);
    // Every thread runs the same number of iterations: the folds below shuffle across full warps.
    for (int base = 0; base < c; base += NGRP * U) {
        const int i0 = base + grp * U;
        vtx::Vec8<T> v[U][CPL];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u;
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
                const int ch = lane + k * LANES;
                if (i < c && ch < nchunk) v[u][k].load(cent + (int64_t)row_ids[i] * a.D + ch * 8);
                else v[u][k].zero();
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
                float f[8];
                v[u][k].unpack(f);
                if (lane + k * LANES < nchunk) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        acc = __fadd_rn(acc, vtx::round_to<T>(__fmul_rn(f[j], qm[k][j])));
                }
            }
#pragma unroll
            for (int w = LANES / 2; w > 0; w >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, w));
            const int i = i0 + u;
            if (lane == 0 && i < c) {
                const float sc = vtx::round_to<T>(acc);
                if (MODE == 0) keys[i] = KeyOf<T>::make(sc, i);
                else store_score<T>(reinterpret_cast<T*>(a.scores) + beg + i, sc);
            }
        }
    }
    if (MODE == 0) {
        __syncthreads();
        const int o0 = a.sparse_indptr[s] + a.bos;
        select_and_store<T>(keys, ids, c, a.K, a.sparse_indices + o0,
                            a.sparse_pt ? a.sparse_pt + (int64_t)s * a.pt_stride + a.bos : nullptr);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) topk_kernel(const T* __restrict__ scores, IndexerArgs a) {
    using Key = typename KeyOf<T>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Key* keys = reinterpret_cast<Key*>(smem_raw);
    int32_t* ids = reinterpret_cast<int32_t*>(smem_raw + (size_t)a.key_cap * sizeof(Key));
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
    select_and_store<T>(keys, ids, c, a.K, a.sparse_indices + o0, nullptr);
}

template <typename T>
size_t smem_bytes(int key_cap) {
    return (size_t)key_cap * (sizeof(typename KeyOf<T>::type) + sizeof(int32_t));
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

template <typename T, int LANES, int CPL, int U, int MODE>
int launch_indexer_cfg(const IndexerArgs& a, int eff_bs, cudaStream_t st) {
    const size_t bytes = MODE == 0 ? smem_bytes<T>(a.key_cap) : 0;
    auto kern = indexer_kernel<T, LANES, CPL, U, MODE>;
    int rc = set_smem(kern, bytes);
    if (rc != VTX_OK) return rc;
    kern<<<eff_bs, kThreads, bytes, st>>>(a);
    return vtx::finish_launch();
}

template <typename T, int MODE>
int launch_indexer(const IndexerArgs& a, int eff_bs, cudaStream_t st) {
    switch (a.D) {
        case 64: return launch_indexer_cfg<T, 8, 1, 8, MODE>(a, eff_bs, st);
        case 128: return launch_indexer_cfg<T, 16, 1, 8, MODE>(a, eff_bs, st);
        case 256: return launch_indexer_cfg<T, 32, 1, 8, MODE>(a, eff_bs, st);
        case 512: return launch_indexer_cfg<T, 32, 2, 4, MODE>(a, eff_bs, st);
        case 576: return launch_indexer_cfg<T, 32, 3, 4, MODE>(a, eff_bs, st);
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
    a.key_cap = 0;  // GeMV mode keeps nothing in shared memory
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
    a.key_cap = vtx::pow2_ceil(max_num_pages_per_request);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == VTX_BF16) {
        const size_t bytes = smem_bytes<__nv_bfloat16>(a.key_cap);
        rc = set_smem(topk_kernel<__nv_bfloat16>, bytes);
        if (rc != VTX_OK) return rc;
        topk_kernel<__nv_bfloat16><<<eff_batch_size, kThreads, bytes, st>>>((const __nv_bfloat16*)scores, a);
    } else {
        const size_t bytes = smem_bytes<float>(a.key_cap);
        rc = set_smem(topk_kernel<float>, bytes);
        if (rc != VTX_OK) return rc;
        topk_kernel<float><<<eff_batch_size, kThreads, bytes, st>>>((const float*)scores, a);
    }
    return vtx::finish_launch();
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
    a.key_cap = vtx::pow2_ceil(max_num_pages_per_request);
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == VTX_BF16 ? launch_indexer<__nv_bfloat16, 0>(a, eff_batch_size, st)
                             : launch_indexer<float, 0>(a, eff_batch_size, st);
}
