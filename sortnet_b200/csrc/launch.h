// Host-side helpers shared by the entry points.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

namespace snb {

// Records the last CUDA runtime error seen by an entry point of this thread.
void set_last_cuda_error(cudaError_t e);

// Number of SMs of the current device (cached per device).
int sm_count();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace snb

#define SNB_CUDA(...)                          \
    do {                                       \
        cudaError_t _e = (__VA_ARGS__);        \
        if (_e != cudaSuccess) {               \
            snb::set_last_cuda_error(_e);      \
            return SNB_ERR_CUDA;               \
        }                                      \
    } while (0)
