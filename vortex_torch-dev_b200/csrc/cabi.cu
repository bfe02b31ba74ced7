// Library-level entry points of the C ABI: version, status strings, last CUDA error text.
#include <string.h>

#include "vtx_common.cuh"

#include <atomic>
#include <mutex>

// Sticky status word of the kernels: a kernel that meets a condition it cannot report through its return
// code (the launch has already succeeded) sets a VTX_STATUS_* bit here with atomicOr and carries on with a
// well-defined result.  One word per device that loaded the library.
static __device__ uint32_t g_vtx_device_status = 0;

#ifdef VTX_CHECKED
// Limits and status bits of the index checks; visible to every translation unit (relocatable device code).
namespace vtx {
__device__ long long g_checked_limit[kNumLimits] = {-1, -1, -1, -1};
__device__ uint32_t g_checked_status = 0;
}
namespace {
__global__ void set_limits_kernel(long long kv_rows, long long summary_rows, long long loc_tokens,
                                  long long req_rows) {
    vtx::pdl_wait();
    vtx::pdl_trigger();
    vtx::g_checked_limit[vtx::kLimKvRows] = kv_rows;
    vtx::g_checked_limit[vtx::kLimSummaryRows] = summary_rows;
    vtx::g_checked_limit[vtx::kLimLocTokens] = loc_tokens;
    vtx::g_checked_limit[vtx::kLimReqRows] = req_rows;
}
}  // namespace
#endif

namespace {
thread_local char g_last_error[256] = "";
std::atomic<int> g_pdl{0};
std::mutex g_status_mu;
uint32_t* g_status_addr[64] = {};
}

namespace vtx {
void note_cuda_error(cudaError_t e) {
    const char* s = cudaGetErrorString(e);
    strncpy(g_last_error, s ? s : "unknown CUDA error", sizeof(g_last_error) - 1);
    g_last_error[sizeof(g_last_error) - 1] = '\0';
}
bool programmatic_launch_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }

// Device address of the status word on the current device (looked up once per device), or null.
uint32_t* device_status_word() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mu);
    if (g_status_addr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_vtx_device_status);
        if (e != cudaSuccess) {
            note_cuda_error(e);
            return nullptr;
        }
        g_status_addr[dev] = static_cast<uint32_t*>(p);
    }
    return g_status_addr[dev];
}
}  // namespace vtx

extern "C" int vtx_version(void) { return 100; /* 0.1.0 */ }

extern "C" const char* vtx_status_string(int status) {
    switch (status) {
        case VTX_OK: return "ok";
        case VTX_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, negative size or bad enum)";
        case VTX_ERR_UNSUPPORTED: return "shape or size not supported by the sm_100a kernels";
        case VTX_ERR_CUDA: return "CUDA runtime error at launch (see vtx_last_cuda_error)";
        case VTX_ERR_SCRATCH_LIMIT:
            return "the call needs more scratch than the library's built-in buffer holds "
                   "(VTX_NOALLOC_SCRATCH_BYTES): use fewer splits or the variant with a caller workspace";
        default: return "unknown status";
    }
}

extern "C" const char* vtx_last_cuda_error(void) { return g_last_error; }

extern "C" int vtx_set_programmatic_launch(int enable) {
    g_pdl.store(enable > 0 ? 1 : 0, std::memory_order_relaxed);
    return VTX_OK;
}

extern "C" void* vtx_device_status_word(void) { return vtx::device_status_word(); }

extern "C" int vtx_device_status_read(uint32_t* host_bits, int clear) {
    if (!host_bits) return VTX_ERR_INVALID_ARGUMENT;
    uint32_t* w = vtx::device_status_word();
    if (!w) return VTX_ERR_CUDA;
    cudaError_t e = cudaMemcpy(host_bits, w, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && clear) e = cudaMemset(w, 0, sizeof(uint32_t));
#ifdef VTX_CHECKED
    if (e == cudaSuccess) {  // the index checks keep their bits in a word of their own
        uint32_t chk = 0;
        e = cudaMemcpyFromSymbol(&chk, vtx::g_checked_status, sizeof(chk));
        *host_bits |= chk;
        if (e == cudaSuccess && clear) {
            chk = 0;
            e = cudaMemcpyToSymbol(vtx::g_checked_status, &chk, sizeof(chk));
        }
    }
#endif
    if (e != cudaSuccess) {
        vtx::note_cuda_error(e);
        return VTX_ERR_CUDA;
    }
    return VTX_OK;
}

extern "C" int vtx_checked_build(void) {
#ifdef VTX_CHECKED
    return 1;
#else
    return 0;
#endif
}

extern "C" int vtx_checked_set_limits(int64_t kv_rows, int64_t summary_rows, int64_t loc_tokens, int64_t req_rows,
                                      void* stream) {
#ifdef VTX_CHECKED
    return vtx::launch(set_limits_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(stream),
                       (long long)kv_rows, (long long)summary_rows, (long long)loc_tokens, (long long)req_rows);
#else
    (void)kv_rows; (void)summary_rows; (void)loc_tokens; (void)req_rows; (void)stream;
    return VTX_ERR_UNSUPPORTED;
#endif
}

extern "C" int vtx_checked_get_limits(int64_t* host_limits) {
    if (!host_limits) return VTX_ERR_INVALID_ARGUMENT;
#ifdef VTX_CHECKED
    long long v[vtx::kNumLimits];
    cudaError_t e = cudaMemcpyFromSymbol(v, vtx::g_checked_limit, sizeof(v));
    if (e != cudaSuccess) {
        vtx::note_cuda_error(e);
        return VTX_ERR_CUDA;
    }
    for (int i = 0; i < vtx::kNumLimits; ++i) host_limits[i] = v[i];
    return VTX_OK;
#else
    return VTX_ERR_UNSUPPORTED;
#endif
}
