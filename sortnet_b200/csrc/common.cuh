// Shared device helpers for the norm-distance kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define SNB_EPS 1e-10f
#define SNB_SUB_BATCH 32
#define SNB_SIGN_BIT 0x80000000u
#define SNB_NO_GRAD_ID 0xffffffffu

// Status codes returned by every exported entry point (0 = ok).
enum {
    SNB_OK = 0,
    SNB_ERR_NULL_POINTER = 1,
    SNB_ERR_BAD_SHAPE = 2,
    SNB_ERR_UNSUPPORTED = 3,      // a p outside (0, inf), a sort size outside 2..25, groups without scratch
    SNB_ERR_TOO_LARGE = 4,        // an index would not fit 31 bits
    SNB_ERR_CUDA = 5,             // a CUDA runtime call failed (see snb_last_cuda_error)
    SNB_ERR_ALIGNMENT = 6,
    SNB_ERR_STATIC_CAPACITY = 7,  // B * CO exceeds the built-in scratch of the no-allocation entry point
    SNB_ERR_INDEX_RANGE = 8,      // an index list holds an entry outside [0, channels) (snb_check_index_lists)
};

namespace snb {

// ---- packed fp32 and 3-input min/max (Blackwell) -------------------------------------
// Two IEEE fp32 subtractions in one instruction on a 64-bit register pair.
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// max(|a|, |b|, |c|); NaN operands are ignored like fmaxf.
__device__ __forceinline__ float max3abs(float a, float b, float c) {
    float d;
    asm("max.abs.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float min3(float a, float b, float c) {
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// ---- asynchronous global -> shared copies ---------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
// 16-byte copy through L2 only; src_bytes = 0 writes zeros without reading.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

}  // namespace snb
