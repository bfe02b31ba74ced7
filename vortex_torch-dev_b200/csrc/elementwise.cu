// Unary elementwise operators on RAGGED indexer tensors ([max_num_pages, C, D] bf16, packed rows).
//
// Replaces elementwise_rr_kernel (indexer/triton_kernels/elementwise_impl.py:8-114) behind the operators
// Relu / Sigmoid / Silu / Abs / Add_Mul (indexer/elementwise.py:158-297).  The reference walks its
// workload windows, which together cover the packed rows [0, dense_kv_indptr[eff_bs]); this kernel reads
// that row count from device memory and streams the range with 16-byte accesses, so no host value is
// needed and the launch can sit in a CUDA graph.
//
// Arithmetic, fixed so that results do not depend on the compiler: alpha and beta are rounded to bf16 first
// (as the reference does); every bf16 operation rounds once to bf16 (z = bf16(bf16(beta * x) + alpha));
// the logistic forms widen z to fp32, use the library's canonical exp (indexer.cu's softmax uses the same)
// and round the quotient once.
#include "vtx_common.cuh"

namespace {

// exp for fp32 with a fixed operation sequence (no FMA contraction, no fast-math): range reduction by
// ln 2 split in two, degree-6 polynomial, scaling by 2^k.  The CPU checker of the test-suite
// restates the same sequence, so results compare bit for bit.
__device__ __forceinline__ float exp_canonical(float x) {
    if (x > 88.f) return __int_as_float(0x7f800000);
    if (x < -87.0f) return 0.f;
    const float k = rintf(__fmul_rn(x, 1.44269504f));
    float r = __fsub_rn(x, __fmul_rn(k, 0.693145751953125f));
    r = __fsub_rn(r, __fmul_rn(k, 1.42860677e-6f));
    float p = (float)(1.0 / 720.0);
    p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 120.0));
    p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 24.0));
    p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 6.0));
    p = __fadd_rn(__fmul_rn(p, r), 0.5f);
    p = __fadd_rn(__fmul_rn(p, r), 1.f);
    p = __fadd_rn(__fmul_rn(p, r), 1.f);
    return __fmul_rn(p, __int_as_float(((int)k + 127) << 23));
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <int OP>
__device__ __forceinline__ float apply(float x, float alpha, float beta) {
    if (OP == 0) return x >= alpha ? x : beta;  // relu form: x >= alpha ? x : beta
    const float z = bf16_round(__fadd_rn(bf16_round(__fmul_rn(beta, x)), alpha));
    if (OP == 1) return __fdiv_rn(1.f, __fadd_rn(1.f, exp_canonical(z)));  // 1 / (1 + exp(beta x + alpha))
    if (OP == 2) return __fdiv_rn(x, __fadd_rn(1.f, exp_canonical(z)));    // x / (1 + exp(beta x + alpha))
    if (OP == 3) return fabsf(z);                                          // |beta x + alpha|
    return z;                                                              // beta x + alpha
}

template <int OP>
__global__ void __launch_bounds__(256) elementwise_kernel(const __nv_bfloat16* __restrict__ x,
                                                         __nv_bfloat16* __restrict__ out,
                                                         const int32_t* __restrict__ row_count, int64_t max_rows,
                                                         int inner, float alpha, float beta) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    int64_t rows = *row_count;
    if (rows > max_rows) rows = max_rows;
    const int64_t n = rows * inner;
    const int64_t n8 = n / 8;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
        vtx::Vec8<__nv_bfloat16> v;
        v.load(x + i * 8);
        float f[8];
        v.unpack(f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = apply<OP>(f[j], alpha, beta);
        vtx::store8(out + i * 8, f);
    }
    for (int64_t i = n8 * 8 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(apply<OP>(__bfloat162float(x[i]), alpha, beta));
}

// Binary form on two RAGGED tensors with broadcasting over the two inner dims (a size of 1 repeats).
// OP 0 max, 1 min, 2 bf16(bf16(alpha x) + bf16(beta y)), 3 bf16(x y)  (elementwise_binary_rrr_kernel,
// indexer/triton_kernels/elementwise_binary_impl.py:7-100).
template <int OP>
__global__ void __launch_bounds__(256) elementwise_binary_kernel(const __nv_bfloat16* __restrict__ x,
                                                                const __nv_bfloat16* __restrict__ y,
                                                                __nv_bfloat16* __restrict__ out,
                                                                const int32_t* __restrict__ row_count, int64_t max_rows,
                                                                int xc, int xd, int yc, int yd, int oc, int od,
                                                                float alpha, float beta) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    int64_t rows = *row_count;
    if (rows > max_rows) rows = max_rows;
    const int inner = oc * od;
    const int64_t n = rows * inner;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / inner;
        const int e = (int)(i - r * inner), c = e / od, d = e - c * od;
        const float a = __bfloat162float(x[(r * xc + (xc == 1 ? 0 : c)) * xd + (xd == 1 ? 0 : d)]);
        const float b = __bfloat162float(y[(r * yc + (yc == 1 ? 0 : c)) * yd + (yd == 1 ? 0 : d)]);
        float o;
        if (OP == 0) o = fmaxf(a, b);
        else if (OP == 1) o = fminf(a, b);
        else if (OP == 2) o = __fadd_rn(bf16_round(__fmul_rn(alpha, a)), bf16_round(__fmul_rn(beta, b)));
        else o = __fmul_rn(a, b);
        out[i] = __float2bfloat16_rn(o);
    }
}

}  // namespace

extern "C" int vtx_elementwise_binary(const void* x, const void* y, void* out, const int32_t* packed_row_count,
                                      int64_t max_rows, int x_c, int x_d, int y_c, int y_d, int op, float alpha,
                                      float beta, int dtype, void* stream) {
    if (!x || !y || !out || !packed_row_count || max_rows < 0) return VTX_ERR_INVALID_ARGUMENT;
    if (x_c < 1 || x_d < 1 || y_c < 1 || y_d < 1 || op < 0 || op > 3) return VTX_ERR_INVALID_ARGUMENT;
    if ((x_c != y_c && x_c != 1 && y_c != 1) || (x_d != y_d && x_d != 1 && y_d != 1)) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16) return VTX_ERR_UNSUPPORTED;
    if (max_rows == 0) return VTX_OK;
    const int oc = x_c > y_c ? x_c : y_c, od = x_d > y_d ? x_d : y_d;
    const float a = __bfloat162float(__float2bfloat16_rn(alpha)), b = __bfloat162float(__float2bfloat16_rn(beta));
    const int64_t n = max_rows * oc * od;
    int blocks = (int)((n + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    const auto* xp = (const __nv_bfloat16*)x;
    const auto* yp = (const __nv_bfloat16*)y;
    auto* op_ = (__nv_bfloat16*)out;
    cudaStream_t st = (cudaStream_t)stream;
#define VTX_EB_CASE(N) \
    case N: return vtx::launch(elementwise_binary_kernel<N>, dim3(blocks), dim3(256), 0, st, xp, yp, op_, packed_row_count, \
                               max_rows, x_c, x_d, y_c, y_d, oc, od, a, b);
    switch (op) {
        VTX_EB_CASE(0) VTX_EB_CASE(1) VTX_EB_CASE(2)
        default: return vtx::launch(elementwise_binary_kernel<3>, dim3(blocks), dim3(256), 0, st, xp, yp, op_,
                                    packed_row_count, max_rows, x_c, x_d, y_c, y_d, oc, od, a, b);
    }
#undef VTX_EB_CASE
}

extern "C" int vtx_elementwise(const void* x, void* out, const int32_t* packed_row_count, int64_t max_rows,
                               int inner_size, int op, float alpha, float beta, int dtype, void* stream) {
    if (!x || !out || !packed_row_count || max_rows < 0 || inner_size < 1) return VTX_ERR_INVALID_ARGUMENT;
    if (op < 0 || op > 4) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16 && dtype != VTX_F32) return VTX_ERR_INVALID_ARGUMENT;
    if (dtype != VTX_BF16) return VTX_ERR_UNSUPPORTED;
    if (max_rows == 0) return VTX_OK;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) return VTX_ERR_INVALID_ARGUMENT;
    const float a = __bfloat162float(__float2bfloat16_rn(alpha)), b = __bfloat162float(__float2bfloat16_rn(beta));
    const int64_t n8 = max_rows * inner_size / 8 + 1;
    int blocks = (int)((n8 + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    const auto* xp = (const __nv_bfloat16*)x;
    auto* op_ = (__nv_bfloat16*)out;
    cudaStream_t st = (cudaStream_t)stream;
    switch (op) {
        case 0: return vtx::launch(elementwise_kernel<0>, dim3(blocks), dim3(256), 0, st, xp, op_, packed_row_count, max_rows, inner_size, a, b);
        case 1: return vtx::launch(elementwise_kernel<1>, dim3(blocks), dim3(256), 0, st, xp, op_, packed_row_count, max_rows, inner_size, a, b);
        case 2: return vtx::launch(elementwise_kernel<2>, dim3(blocks), dim3(256), 0, st, xp, op_, packed_row_count, max_rows, inner_size, a, b);
        case 3: return vtx::launch(elementwise_kernel<3>, dim3(blocks), dim3(256), 0, st, xp, op_, packed_row_count, max_rows, inner_size, a, b);
        default: return vtx::launch(elementwise_kernel<4>, dim3(blocks), dim3(256), 0, st, xp, op_, packed_row_count, max_rows, inner_size, a, b);
    }
}
