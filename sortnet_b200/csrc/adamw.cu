// Fused AdamW over one flat fp32 parameter buffer.
//
// The reference trains with torch.optim.AdamW over the model parameters (main.py:429-432, weight
// decay 0 on the norm-distance weights) after DistributedDataParallel has averaged the gradients
// (main.py:402).  Here parameters, gradients and both moments live in four flat buffers, so one
// pass updates everything: 4 reads + 3 writes of 4 bytes per parameter, HBM-bound.
// Arithmetic follows torch.optim.AdamW (decoupled weight decay, bias-corrected moments):
//   w  *= 1 - lr * wd
//   m   = b1 m + (1 - b1) g ;  v = b2 v + (1 - b2) g^2
//   w  -= (lr / (1 - b1^t)) * m / (sqrt(v) / sqrt(1 - b2^t) + eps)
// grad_scale multiplies g first (e.g. 1 / world size when the exchange summed the gradients).
#include "common.cuh"
#include "launch.h"

namespace snb {

__global__ void __launch_bounds__(256) adamw_kernel(float4* __restrict__ w, const float4* __restrict__ g,
                                                    float4* __restrict__ m, float4* __restrict__ v, size_t n4,
                                                    float decay, float b1, float b2, float step_size,
                                                    float inv_sqrt_bc2, float eps, float grad_scale) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 wv = w[i], gv = g[i], mv = m[i], vv = v[i];
        float* wp = reinterpret_cast<float*>(&wv);
        const float* gp = reinterpret_cast<const float*>(&gv);
        float* mp = reinterpret_cast<float*>(&mv);
        float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float gk = gp[k] * grad_scale;
            mp[k] = b1 * mp[k] + (1.0f - b1) * gk;
            vp[k] = b2 * vp[k] + (1.0f - b2) * gk * gk;
            const float denom = sqrtf(vp[k]) * inv_sqrt_bc2 + eps;
            wp[k] = wp[k] * decay - step_size * (mp[k] / denom);
        }
        w[i] = wv;
        m[i] = mv;
        v[i] = vv;
    }
}

constexpr int ADAMW_MAX_PARTS = 16;
struct GradParts {
    const float4* g[ADAMW_MAX_PARTS];
};

// The same update with the gradient given as PARTS partial buffers (summed in index order) and
// the new values written to a second parameter buffer: the local half of a data-parallel step
// whose reduce-scatter and all-gather are plain device-to-device copies.  PARTS is a template
// parameter so that the part pointers are compile-time-indexed kernel parameters (a run-time index
// sends the pointer table to local memory and serialises the loads behind it: 0.72 ms instead of
// 0.2 ms for 30 M values in four parts); all loads of an element are issued before the first use.
template <int PARTS>
__global__ void __launch_bounds__(256) adamw_reduce_kernel(const float4* __restrict__ w_src, float4* __restrict__ w_dst,
                                                           const GradParts parts, float4* __restrict__ m,
                                                           float4* __restrict__ v, size_t n4, float decay, float b1,
                                                           float b2, float step_size, float inv_sqrt_bc2, float eps,
                                                           float grad_scale) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 t[PARTS];
#pragma unroll
        for (int r = 0; r < PARTS; r++) t[r] = __ldcs(parts.g[r] + i);     // read once: streaming loads
        float4 wv = w_src[i], mv = m[i], vv = v[i];
        float4 gv = t[0];
#pragma unroll
        for (int r = 1; r < PARTS; r++) {
            gv.x += t[r].x;
            gv.y += t[r].y;
            gv.z += t[r].z;
            gv.w += t[r].w;
        }
        float* wp = reinterpret_cast<float*>(&wv);
        const float* gp = reinterpret_cast<const float*>(&gv);
        float* mp = reinterpret_cast<float*>(&mv);
        float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float gk = gp[k] * grad_scale;
            mp[k] = b1 * mp[k] + (1.0f - b1) * gk;
            vp[k] = b2 * vp[k] + (1.0f - b2) * gk * gk;
            const float denom = sqrtf(vp[k]) * inv_sqrt_bc2 + eps;
            wp[k] = wp[k] * decay - step_size * (mp[k] / denom);
        }
        w_dst[i] = wv;
        m[i] = mv;
        v[i] = vv;
    }
}

}  // namespace snb

using namespace snb;

extern "C" int snb_adamw_reduce_step(const float* w_src, float* w_dst, const void* const* grad_parts, int parts,
                                     float* m, float* v, long long n, float lr, float beta1, float beta2, float eps,
                                     float weight_decay, int step, float grad_scale, void* stream) {
    if (!w_src || !w_dst || !grad_parts || !m || !v) return SNB_ERR_NULL_POINTER;
    if (parts < 1 || parts > ADAMW_MAX_PARTS) return SNB_ERR_UNSUPPORTED;
    if (n <= 0 || step <= 0 || (n & 3)) return SNB_ERR_BAD_SHAPE;
    if (!aligned16(w_src) || !aligned16(w_dst) || !aligned16(m) || !aligned16(v)) return SNB_ERR_ALIGNMENT;
    GradParts gp{};
    for (int r = 0; r < parts; r++) {
        if (!grad_parts[r]) return SNB_ERR_NULL_POINTER;
        if (!aligned16(grad_parts[r])) return SNB_ERR_ALIGNMENT;
        gp.g[r] = reinterpret_cast<const float4*>(grad_parts[r]);
    }
    const double bc1 = 1.0 - pow((double)beta1, step), bc2 = 1.0 - pow((double)beta2, step);
    const float step_size = (float)(lr / bc1), inv_sqrt_bc2 = (float)(1.0 / sqrt(bc2));
    const int blocks = sm_count() * 8;
    cudaStream_t st = (cudaStream_t)stream;
#define SNB_REDUCE_CASE(P)                                                                                          \
    case P:                                                                                                         \
        adamw_reduce_kernel<P><<<blocks, 256, 0, st>>>(reinterpret_cast<const float4*>(w_src),                      \
                                                       reinterpret_cast<float4*>(w_dst), gp, reinterpret_cast<float4*>(m), \
                                                       reinterpret_cast<float4*>(v), (size_t)n / 4,                 \
                                                       1.0f - lr * weight_decay, beta1, beta2, step_size,           \
                                                       inv_sqrt_bc2, eps, grad_scale);                              \
        break;
    switch (parts) {
        SNB_REDUCE_CASE(1) SNB_REDUCE_CASE(2) SNB_REDUCE_CASE(3) SNB_REDUCE_CASE(4) SNB_REDUCE_CASE(5)
        SNB_REDUCE_CASE(6) SNB_REDUCE_CASE(7) SNB_REDUCE_CASE(8) SNB_REDUCE_CASE(9) SNB_REDUCE_CASE(10)
        SNB_REDUCE_CASE(11) SNB_REDUCE_CASE(12) SNB_REDUCE_CASE(13) SNB_REDUCE_CASE(14) SNB_REDUCE_CASE(15)
        SNB_REDUCE_CASE(16)
    }
#undef SNB_REDUCE_CASE
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

extern "C" int snb_adamw_step(float* w, const float* g, float* m, float* v, long long n, float lr, float beta1,
                              float beta2, float eps, float weight_decay, int step, float grad_scale,
                              void* stream) {
    if (!w || !g || !m || !v) return SNB_ERR_NULL_POINTER;
    if (n <= 0 || step <= 0 || (n & 3)) return SNB_ERR_BAD_SHAPE;  // buffers are padded to 4 elements
    if (!aligned16(w) || !aligned16(g) || !aligned16(m) || !aligned16(v)) return SNB_ERR_ALIGNMENT;
    const double bc1 = 1.0 - pow((double)beta1, step), bc2 = 1.0 - pow((double)beta2, step);
    const float step_size = (float)(lr / bc1), inv_sqrt_bc2 = (float)(1.0 / sqrt(bc2));
    const int blocks = sm_count() * 8;
    adamw_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<float4*>(w), reinterpret_cast<const float4*>(g), reinterpret_cast<float4*>(m),
        reinterpret_cast<float4*>(v), (size_t)n / 4, 1.0f - lr * weight_decay, beta1, beta2, step_size,
        inv_sqrt_bc2, eps, grad_scale);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}
