// Block-table decode attention over a shared compressed latent (multi-head latent attention).
//
// 16 query heads share one latent row per token: keys are the full row (kv_lora_rank + rope dims =
// 576), values its first 512 dims, so every byte read from HBM feeds both products.  The reference
// project has no such kernel; the block-table inputs are the ones its planner produces
// (csrc/utils_sglang.cu:949-1083: page table [bs, stride] and per-request sequence lengths).
//
// One CTA per request: two groups of 4 warps, each group takes every other 16-token tile (18 KB) of the
// token list and keeps its own running softmax state; the two states are merged once at the end.  Each
// group streams its tiles global -> shared through its own 4-slot ring of 16-byte cp.async copies
// (~110 KB in flight per SM) and synchronises on its own named barrier, so the groups overlap freely.
// Rows are stored chunk-swizzled (chunk ^ (row & 7)) so ldmatrix is conflict-free.  Per tile, on
// mma.sync m16n8k16 (the 16 heads are exactly one M tile):
//   S^T[head, token] = q . K^T   the 576 dims are split over the warps (9 k-steps each, q fragments in
//                                registers); partial sums meet in shared memory
//   O^T[dim, head]  += V^T . P^T each warp owns 128 output dims; P^T is the accumulator layout of S^T
// Softmax is the online form in fp32, computed redundantly by every warp from the summed S^T.
#include "vtx_common.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kHeads = 16;
constexpr int kDl = 576;                 // latent row: keys
constexpr int kDv = 512;                 // leading dims: values
constexpr int kTile = 16;                // tokens per tile
constexpr int kRowB = kDl * 2;           // 1152 bytes
constexpr int kTileB = kTile * kRowB;    // 18432 bytes
constexpr int kGroups = 2;               // warp groups per CTA, alternating tiles
constexpr int kStages = 4;               // ring slots per group
constexpr int kKsteps = kDl / 16;        // 36
constexpr int kKsPerWarp = kKsteps / kWarps;          // 9
constexpr int kMtPerWarp = kDv / 16 / kWarps;         // 8 output tiles of 16 dims per warp
constexpr int kChunksPerRow = kRowB / 16;             // 72
constexpr int kChunksPerTile = kTile * kChunksPerRow; // 1152
constexpr float kLog2e = 1.4426950408889634f;

struct MlaArgs {
    const __nv_bfloat16* q;       // [bs, 16, 576]
    const unsigned char* latent;  // [rows, P, 576] bf16
    __nv_bfloat16* out;           // [bs, 16, 512]
    const int32_t* page_table;
    int64_t pt_stride;
    const int32_t* seqlens;
    int P;
    float scale_log2;
};

__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr, bool valid) {
    const int src_bytes = valid ? 16 : 0;
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

__device__ __forceinline__ void group_sync(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(kWarps * 32) : "memory");
}

__global__ void __launch_bounds__(kGroups * kWarps * 32, 1) decode_mla_kernel(MlaArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // layout: [group 0 ring][group 1 ring][partial S^T: per group 2 buffers x kWarps x 2 n-tiles x 32 lanes x 4]
    vtx::pdl_wait();
    vtx::pdl_trigger();

    const int b = blockIdx.x;
    const int group = threadIdx.x / (kWarps * 32), gthread = threadIdx.x % (kWarps * 32);
    const int warp = gthread >> 5, lane = threadIdx.x & 31;
    float* s_part = reinterpret_cast<float*>(smem_raw + (size_t)kGroups * kStages * kTileB) +
                    (size_t)group * (2 * kWarps * 2 * 32 * 4);
    const int gid = lane >> 2, tid = lane & 3;
    const int ntok = a.seqlens[b];
    const int n_tiles = (ntok + kTile - 1) / kTile;
    const int tiles_per_page = a.P / kTile;
    const int32_t* pt = a.page_table + (int64_t)b * a.pt_stride;
    const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(smem_raw) + group * (kStages * kTileB);
    // this group's tiles: group, group + kGroups, ...; `ord` counts them
    const int my_tiles = n_tiles > group ? (n_tiles - group + kGroups - 1) / kGroups : 0;

    // q fragments (A operand, 16 heads x 16 dims per k-step) for this warp's 9 k-steps
    uint32_t qa[kKsPerWarp][4];
    {
        const uint32_t* q0 = reinterpret_cast<const uint32_t*>(a.q + ((int64_t)b * kHeads + gid) * kDl);
        const uint32_t* q1 = reinterpret_cast<const uint32_t*>(a.q + ((int64_t)b * kHeads + gid + 8) * kDl);
#pragma unroll
        for (int i = 0; i < kKsPerWarp; ++i) {
            const int ks = warp * kKsPerWarp + i;
            qa[i][0] = q0[ks * 8 + tid];
            qa[i][1] = q1[ks * 8 + tid];
            qa[i][2] = q0[ks * 8 + 4 + tid];
            qa[i][3] = q1[ks * 8 + 4 + tid];
        }
    }
    float o[kMtPerWarp][2][4];  // O^T: [16 dims of tile][8 heads of n-tile j]
#pragma unroll
    for (int mt = 0; mt < kMtPerWarp; ++mt)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[mt][j][i] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;  // heads gid and gid + 8

    auto issue = [&](int ord) {
        const int tile = group + ord * kGroups;
        const int page = tile / tiles_per_page, t_in = tile - page * tiles_per_page;
        const int64_t row = pt[page];
        const unsigned char* src = a.latent + ((row * a.P) + (int64_t)t_in * kTile) * kRowB;
        const uint32_t dst = ring_addr + (uint32_t)((ord % kStages) * kTileB);
        const int tok0 = tile * kTile;
#pragma unroll
        for (int c = 0; c < kChunksPerTile / (kWarps * 32); ++c) {
            const int ch = c * (kWarps * 32) + gthread;
            const int t = ch / kChunksPerRow, cr = ch - t * kChunksPerRow;
            cp_async16(dst + t * kRowB + ((cr ^ (t & 7)) << 4), src + (size_t)ch * 16, tok0 + t < ntok);
        }
    };

#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {
        if (i < my_tiles) issue(i);
        cp_async_commit();
    }
    const int lm_t = ((lane >> 4) << 3) + (lane & 7);
    const int lm_c = (lane >> 3) & 1;

    for (int ord = 0; ord < my_tiles; ++ord) {
        const int tile = group + ord * kGroups;
        cp_async_wait<kStages - 2>();
        group_sync(group);  // tile landed for the whole group; the group is done with the slot refilled next
        if (ord + kStages - 1 < my_tiles) issue(ord + kStages - 1);
        cp_async_commit();

        const uint32_t tile_addr = ring_addr + (uint32_t)((ord % kStages) * kTileB) + lm_t * kRowB;
        // ---- partial S^T over this warp's dims
        float st[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) st[j][i] = 0.f;
#pragma unroll
        for (int i = 0; i < kKsPerWarp; ++i) {
            const int ks = warp * kKsPerWarp + i;
            uint32_t kb[4];
            ldmatrix_x4(kb, tile_addr + ((((ks << 1) + lm_c) ^ (lm_t & 7)) << 4));
            mma_bf16(st[0], qa[i][0], qa[i][1], qa[i][2], qa[i][3], kb[0], kb[1]);  // tokens 0-7
            mma_bf16(st[1], qa[i][0], qa[i][1], qa[i][2], qa[i][3], kb[2], kb[3]);  // tokens 8-15
        }
        float* part = s_part + (size_t)(ord & 1) * (kWarps * 2 * 32 * 4);
#pragma unroll
        for (int j = 0; j < 2; ++j)
            *reinterpret_cast<float4*>(part + ((warp * 2 + j) * 32 + lane) * 4) =
                make_float4(st[j][0], st[j][1], st[j][2], st[j][3]);
        group_sync(group);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {  // fixed order: every warp gets the same bits
                const float4 v = *reinterpret_cast<const float4*>(part + ((w * 2 + j) * 32 + lane) * 4);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            st[j][0] = acc.x; st[j][1] = acc.y; st[j][2] = acc.z; st[j][3] = acc.w;
        }
        // ---- online softmax; this lane: heads gid (c0,c1) and gid+8 (c2,c3), tokens tid*2+{0,1} (+8 for j=1)
        const int tok0 = tile * kTile;
        float sv[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const bool v0 = tok0 + j * 8 + tid * 2 < ntok, v1 = tok0 + j * 8 + tid * 2 + 1 < ntok;
            sv[j][0] = v0 ? st[j][0] * a.scale_log2 : -INFINITY;
            sv[j][1] = v1 ? st[j][1] * a.scale_log2 : -INFINITY;
            sv[j][2] = v0 ? st[j][2] * a.scale_log2 : -INFINITY;
            sv[j][3] = v1 ? st[j][3] * a.scale_log2 : -INFINITY;
        }
        float mx_lo = fmaxf(fmaxf(sv[0][0], sv[0][1]), fmaxf(sv[1][0], sv[1][1]));
        float mx_hi = fmaxf(fmaxf(sv[0][2], sv[0][3]), fmaxf(sv[1][2], sv[1][3]));
#pragma unroll
        for (int w = 1; w <= 2; w <<= 1) {
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, w));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, w));
        }
        // every tile holds at least one valid token (tile < ceil(ntok/16)), so the new maxima are finite
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float al_lo = exp2f(m_lo - mn_lo), al_hi = exp2f(m_hi - mn_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        float p[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            p[j][0] = exp2f(sv[j][0] - mn_lo);
            p[j][1] = exp2f(sv[j][1] - mn_lo);
            p[j][2] = exp2f(sv[j][2] - mn_hi);
            p[j][3] = exp2f(sv[j][3] - mn_hi);
        }
        l_lo = l_lo * al_lo + (p[0][0] + p[0][1]) + (p[1][0] + p[1][1]);
        l_hi = l_hi * al_hi + (p[0][2] + p[0][3]) + (p[1][2] + p[1][3]);
        // P^T as B operand: n-tile 0 = heads 0-7 (rows gid), n-tile 1 = heads 8-15 (rows gid+8)
        const uint32_t pb[2][2] = {{pack_bf16x2(p[0][0], p[0][1]), pack_bf16x2(p[1][0], p[1][1])},
                                   {pack_bf16x2(p[0][2], p[0][3]), pack_bf16x2(p[1][2], p[1][3])}};
        // rescale factors of the O^T columns this lane holds: heads 8j + tid*2 + {0,1}
        float sc[2][2];
        sc[0][0] = __shfl_sync(0xffffffffu, al_lo, (tid * 2) << 2);
        sc[0][1] = __shfl_sync(0xffffffffu, al_lo, (tid * 2 + 1) << 2);
        sc[1][0] = __shfl_sync(0xffffffffu, al_hi, (tid * 2) << 2);
        sc[1][1] = __shfl_sync(0xffffffffu, al_hi, (tid * 2 + 1) << 2);
        // ---- O^T += V^T . P^T for this warp's 128 dims
#pragma unroll
        for (int mt = 0; mt < kMtPerWarp; ++mt) {
            const int mg = warp * kMtPerWarp + mt;
            uint32_t va[4];
            ldmatrix_x4_trans(va, tile_addr + ((((mg << 1) + lm_c) ^ (lm_t & 7)) << 4));
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                o[mt][j][0] *= sc[j][0]; o[mt][j][1] *= sc[j][1];
                o[mt][j][2] *= sc[j][0]; o[mt][j][3] *= sc[j][1];
                mma_bf16(o[mt][j], va[0], va[1], va[2], va[3], pb[j][0], pb[j][1]);
            }
        }
    }
    cp_async_wait<0>();

    // row sums over the 4 lanes of a head row
#pragma unroll
    for (int w = 1; w <= 2; w <<= 1) {
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, w);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, w);
    }
    // ---- merge the two groups: group 1 parks its state in shared memory (the rings are idle now)
    __syncthreads();
    float* park = reinterpret_cast<float*>(smem_raw);  // [128 threads][68]: 64 accumulators + m_lo, m_hi, l_lo, l_hi
    if (group == 1) {
        float* mine = park + gthread * 68;
#pragma unroll
        for (int mt = 0; mt < kMtPerWarp; ++mt)
#pragma unroll
            for (int j = 0; j < 2; ++j)
                *reinterpret_cast<float4*>(mine + (mt * 2 + j) * 4) =
                    make_float4(o[mt][j][0], o[mt][j][1], o[mt][j][2], o[mt][j][3]);
        *reinterpret_cast<float4*>(mine + 64) = make_float4(m_lo, m_hi, l_lo, l_hi);
    }
    __syncthreads();
    if (group == 1) return;
    {
        const float* other = park + gthread * 68;
        const float4 st1 = *reinterpret_cast<const float4*>(other + 64);
        const float M_lo = fmaxf(m_lo, st1.x), M_hi = fmaxf(m_hi, st1.y);
        // a group that saw no tile has m = -inf and l = 0: its weight must be 0, not NaN
        const float f0_lo = m_lo == -INFINITY ? 0.f : exp2f(m_lo - M_lo), f1_lo = st1.x == -INFINITY ? 0.f : exp2f(st1.x - M_lo);
        const float f0_hi = m_hi == -INFINITY ? 0.f : exp2f(m_hi - M_hi), f1_hi = st1.y == -INFINITY ? 0.f : exp2f(st1.y - M_hi);
        l_lo = l_lo * f0_lo + st1.z * f1_lo;
        l_hi = l_hi * f0_hi + st1.w * f1_hi;
        float w0[2][2], w1[2][2];  // weights of the columns this lane holds: heads 8j + tid*2 + {0,1}
        w0[0][0] = __shfl_sync(0xffffffffu, f0_lo, (tid * 2) << 2);
        w0[0][1] = __shfl_sync(0xffffffffu, f0_lo, (tid * 2 + 1) << 2);
        w0[1][0] = __shfl_sync(0xffffffffu, f0_hi, (tid * 2) << 2);
        w0[1][1] = __shfl_sync(0xffffffffu, f0_hi, (tid * 2 + 1) << 2);
        w1[0][0] = __shfl_sync(0xffffffffu, f1_lo, (tid * 2) << 2);
        w1[0][1] = __shfl_sync(0xffffffffu, f1_lo, (tid * 2 + 1) << 2);
        w1[1][0] = __shfl_sync(0xffffffffu, f1_hi, (tid * 2) << 2);
        w1[1][1] = __shfl_sync(0xffffffffu, f1_hi, (tid * 2 + 1) << 2);
#pragma unroll
        for (int mt = 0; mt < kMtPerWarp; ++mt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float4 v = *reinterpret_cast<const float4*>(other + (mt * 2 + j) * 4);
                o[mt][j][0] = o[mt][j][0] * w0[j][0] + v.x * w1[j][0];
                o[mt][j][1] = o[mt][j][1] * w0[j][1] + v.y * w1[j][1];
                o[mt][j][2] = o[mt][j][2] * w0[j][0] + v.z * w1[j][0];
                o[mt][j][3] = o[mt][j][3] * w0[j][1] + v.w * w1[j][1];
            }
    }
    // normalise the columns this lane holds
    float inv[2][2];
    {
        const float i_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, i_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
        inv[0][0] = __shfl_sync(0xffffffffu, i_lo, (tid * 2) << 2);
        inv[0][1] = __shfl_sync(0xffffffffu, i_lo, (tid * 2 + 1) << 2);
        inv[1][0] = __shfl_sync(0xffffffffu, i_hi, (tid * 2) << 2);
        inv[1][1] = __shfl_sync(0xffffffffu, i_hi, (tid * 2 + 1) << 2);
    }
    __nv_bfloat16* ob = a.out + (int64_t)b * kHeads * kDv;
#pragma unroll
    for (int mt = 0; mt < kMtPerWarp; ++mt) {
        const int d0 = (warp * kMtPerWarp + mt) * 16 + gid;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int h0 = j * 8 + tid * 2;
            ob[(int64_t)h0 * kDv + d0] = __float2bfloat16_rn(o[mt][j][0] * inv[j][0]);
            ob[(int64_t)(h0 + 1) * kDv + d0] = __float2bfloat16_rn(o[mt][j][1] * inv[j][1]);
            ob[(int64_t)h0 * kDv + d0 + 8] = __float2bfloat16_rn(o[mt][j][2] * inv[j][0]);
            ob[(int64_t)(h0 + 1) * kDv + d0 + 8] = __float2bfloat16_rn(o[mt][j][3] * inv[j][1]);
        }
    }
}

int g_mla_path = 0;  // 0: tcgen05 form where supported, 1: always the mma.sync form

}  // namespace

namespace vtx {
bool mla_tc_supported(int page_size);
int launch_decode_mla_tc(const void* q, const void* latent_cache, int64_t num_cache_pages, void* out,
                         const int32_t* page_table, int64_t page_table_stride, const int32_t* cache_seqlens,
                         int batch_size, int page_size, float sm_scale, cudaStream_t stream);
void* mla_fault_word();
int launch_mla_sparse_layer_tc(const void* q, const void* summary, const void* latent_cache, int64_t num_cache_pages,
                               void* out, const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                               const int32_t* dense_kv_indices, int32_t* sparse_kv_indices, int32_t* sparse_page_table,
                               int64_t page_table_stride, const int32_t* sparse_cache_seqlens, int batch_size,
                               int page_size, int topk_val, int bos, int eos, int max_pages, float sm_scale,
                               cudaStream_t stream);
}  // namespace vtx

extern "C" int vtx_set_mla_path(int path) {
    const int old = g_mla_path;
    g_mla_path = path == 1 ? 1 : 0;
    return old;
}

extern "C" void* vtx_mla_fault_word(void) { return vtx::mla_fault_word(); }

extern "C" int vtx_mla_fault_read(uint32_t* host_bits) {
    void* w = vtx::mla_fault_word();
    if (!host_bits || !w) return VTX_ERR_INVALID_ARGUMENT;
    cudaError_t e = cudaMemcpy(host_bits, w, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        vtx::note_cuda_error(e);
        return VTX_ERR_CUDA;
    }
    return VTX_OK;
}

extern "C" int vtx_decode_mla(const void* q, const void* latent_cache, int64_t num_cache_pages, void* out,
                              const int32_t* page_table, int64_t page_table_stride, const int32_t* cache_seqlens,
                              int batch_size, int num_heads, int latent_dim, int value_dim, int page_size,
                              float sm_scale, int dtype, void* stream) {
    if (!q || !latent_cache || !out || !page_table || !cache_seqlens) return VTX_ERR_INVALID_ARGUMENT;
    if (batch_size < 0 || page_table_stride < 1 || page_size < 1 || num_cache_pages < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 || num_heads != kHeads || latent_dim != kDl || value_dim != kDv || page_size % kTile != 0)
        return VTX_ERR_UNSUPPORTED;
    if (batch_size == 0) return VTX_OK;
    if (g_mla_path == 0 && vtx::mla_tc_supported(page_size))
        return vtx::launch_decode_mla_tc(q, latent_cache, num_cache_pages, out, page_table, page_table_stride,
                                         cache_seqlens, batch_size, page_size, sm_scale, (cudaStream_t)stream);
    MlaArgs a;
    a.q = (const __nv_bfloat16*)q;
    a.latent = (const unsigned char*)latent_cache;
    a.out = (__nv_bfloat16*)out;
    a.page_table = page_table;
    a.pt_stride = page_table_stride;
    a.seqlens = cache_seqlens;
    a.P = page_size;
    a.scale_log2 = sm_scale * kLog2e;
    const size_t bytes = (size_t)kGroups * kStages * kTileB + (size_t)kGroups * 2 * kWarps * 2 * 32 * 4 * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(decode_mla_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) {
        vtx::note_cuda_error(e);
        return VTX_ERR_CUDA;
    }
    return vtx::launch(decode_mla_kernel, dim3(batch_size), dim3(kGroups * kWarps * 32), bytes, (cudaStream_t)stream, a);
}

extern "C" int vtx_mla_sparse_layer(const void* q, const void* summary, const void* latent_cache, int64_t num_cache_pages,
                                    void* out, const int32_t* dense_kv_indptr, const int32_t* sparse_kv_indptr,
                                    const int32_t* dense_kv_indices, int32_t* sparse_kv_indices,
                                    int32_t* sparse_page_table, int64_t page_table_stride,
                                    const int32_t* sparse_cache_seqlens, int batch_size, int num_heads, int latent_dim,
                                    int value_dim, int page_size, int topk_val, int page_reserved_bos,
                                    int page_reserved_eos, int max_num_pages_per_request, float sm_scale, int dtype,
                                    void* stream) {
    if (!q || !summary || !latent_cache || !out || !dense_kv_indptr || !sparse_kv_indptr || !dense_kv_indices ||
        !sparse_kv_indices || !sparse_page_table || !sparse_cache_seqlens)
        return VTX_ERR_INVALID_ARGUMENT;
    if (batch_size < 0 || page_table_stride < 1 || page_size < 1 || num_cache_pages < 1 || topk_val < 1 ||
        page_reserved_bos < 0 || page_reserved_eos < 0 || max_num_pages_per_request < 1)
        return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 || num_heads != kHeads || latent_dim != kDl || value_dim != kDv || page_size % kTile != 0)
        return VTX_ERR_UNSUPPORTED;
    if (batch_size == 0) return VTX_OK;
    if (g_mla_path == 0 && vtx::mla_tc_supported(page_size)) {
        const int rc = vtx::launch_mla_sparse_layer_tc(
            q, summary, latent_cache, num_cache_pages, out, dense_kv_indptr, sparse_kv_indptr, dense_kv_indices,
            sparse_kv_indices, sparse_page_table, page_table_stride, sparse_cache_seqlens, batch_size, page_size,
            topk_val, page_reserved_bos, page_reserved_eos, max_num_pages_per_request, sm_scale, (cudaStream_t)stream);
        if (rc != VTX_ERR_UNSUPPORTED) return rc;
    }
    // the two launches
    const int rc = vtx_indexer_fused(q, summary, dense_kv_indptr, sparse_kv_indptr, dense_kv_indices, sparse_kv_indices,
                                     sparse_page_table, page_table_stride, batch_size, num_heads, latent_dim, topk_val,
                                     page_reserved_bos, page_reserved_eos, max_num_pages_per_request, dtype, stream);
    if (rc != VTX_OK) return rc;
    return vtx_decode_mla(q, latent_cache, num_cache_pages, out, sparse_page_table, page_table_stride,
                          sparse_cache_seqlens, batch_size, num_heads, latent_dim, value_dim, page_size, sm_scale, dtype,
                          stream);
}
