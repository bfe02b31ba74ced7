// Library-level entry points of the C ABI: version, status strings, last CUDA error text.
#include <string.h>

#include "vtx_common.cuh"

#include <atomic>

namespace {
thread_local char g_last_error[256] = "";
std::atomic<int> g_pdl{0};
}

namespace vtx {
void note_cuda_error(cudaError_t e) {
    const char* s = cudaGetErrorString(e);
    strncpy(g_last_error, s ? s : "unknown CUDA error", sizeof(g_last_error) - 1);
    g_last_error[sizeof(g_last_error) - 1] = '\0';
}
bool programmatic_launch_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }
int programmatic_launch_mode() { return g_pdl.load(std::memory_order_relaxed); }
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
    g_pdl.store(enable < 0 ? 0 : (enable > 2 ? 2 : enable), std::memory_order_relaxed);
    return VTX_OK;
}
