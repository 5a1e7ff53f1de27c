// Library-wide host utilities: status strings, last CUDA error, device properties.
#include "common.cuh"
#include "launch.h"

namespace snb {

static thread_local cudaError_t g_last = cudaSuccess;

void set_last_cuda_error(cudaError_t e) { g_last = e; }

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    int& c = cached[dev & 63];
    if (c == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        c = v;
    }
    return c;
}

}  // namespace snb

extern "C" const char* snb_status_string(int status) {
    switch (status) {
        case SNB_OK: return "ok";
        case SNB_ERR_NULL_POINTER: return "null pointer argument";
        case SNB_ERR_BAD_SHAPE: return "inconsistent or non-positive sizes";
        case SNB_ERR_UNSUPPORTED: return "unsupported configuration (only G = 1, HW = 1, 0 < p)";
        case SNB_ERR_TOO_LARGE: return "tensor too large for 31-bit indexing";
        case SNB_ERR_CUDA: return "CUDA runtime error";
        case SNB_ERR_ALIGNMENT: return "pointer not aligned to its element type";
        default: return "unknown status";
    }
}

extern "C" const char* snb_last_cuda_error(void) { return cudaGetErrorString(snb::g_last); }

extern "C" int snb_version(void) { return 100; }

// ---- FP32 peak probe ---------------------------------------------------------------------
// A register-only chain of fused multiply-adds, 16 independent accumulators per thread.  The
// benchmark times it with CUDA events to obtain the CUDA-core FP32 peak (2 flops per FMA) of
// the GPU it runs on, the denominator of the FP32 roofline fractions it reports.
__global__ void __launch_bounds__(256) fp32_probe_kernel(float* out, int iters, float a, float b) {
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; i++) acc[i] = (float)(threadIdx.x + i);
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 16; i++) acc[i] = fmaf(acc[i], a, b);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i++) s += acc[i];
    if (s == 123.456f) out[0] = s;  // never true; keeps the chain alive
}

// Launches the probe; *flops receives the number of floating-point operations it performs.
extern "C" int snb_probe_fp32(float* scratch, int iters, double* flops, void* stream) {
    if (!scratch || !flops || iters <= 0) return SNB_ERR_NULL_POINTER;
    const int blocks = snb::sm_count() * 8;
    fp32_probe_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(scratch, iters, 1.000001f, 1e-7f);
    SNB_CUDA(cudaGetLastError());
    *flops = 2.0 * 16.0 * (double)iters * 256.0 * (double)blocks;
    return SNB_OK;
}
