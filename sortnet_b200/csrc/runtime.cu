// Library-wide host utilities: status strings, last CUDA error, device properties.
#include "common.cuh"
#include "launch.h"

namespace snb {

static thread_local cudaError_t g_last = cudaSuccess;

void set_last_cuda_error(cudaError_t e) { g_last = e; }

int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    int c = cached[dev & 63].load(std::memory_order_relaxed);
    if (c == 0) {
        if (cudaDeviceGetAttribute(&c, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || c <= 0) c = 148;
        cached[dev & 63].store(c, std::memory_order_relaxed);
    }
    return c;
}

}  // namespace snb

extern "C" const char* snb_status_string(int status) {
    switch (status) {
        case SNB_OK: return "ok";
        case SNB_ERR_NULL_POINTER: return "null pointer argument";
        case SNB_ERR_BAD_SHAPE: return "inconsistent or non-positive sizes";
        case SNB_ERR_UNSUPPORTED: return "unsupported configuration (p outside (0, inf), sort size outside 2..25, or groups on an entry point without scratch)";
        case SNB_ERR_TOO_LARGE: return "tensor too large for 31-bit indexing";
        case SNB_ERR_CUDA: return "CUDA runtime error";
        case SNB_ERR_ALIGNMENT: return "pointer not aligned to its element type";
        case SNB_ERR_STATIC_CAPACITY:
            return "B * CO exceeds the built-in scratch of snb_inf_dist_forward_noalloc (1048576 outputs); "
                   "use snb_inf_dist_forward or snb_inf_dist_forward_ws";
        case SNB_ERR_INDEX_RANGE: return "an index list holds an entry outside [0, channels)";
        default: return "unknown status";
    }
}

extern "C" const char* snb_last_cuda_error(void) { return cudaGetErrorString(snb::g_last); }

extern "C" int snb_version(void) { return 100; }
