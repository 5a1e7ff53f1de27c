// Data-parallel optimiser step fused with the gradient exchange over NVLink peer memory.
//
// The reference averages gradients with DistributedDataParallel's bucketed NCCL all-reduce
// (main.py:402) and then runs AdamW on every rank over all parameters (main.py:95,429-432).
// Here the flat gradient and parameter buffers of all ranks of one node are mapped into every
// rank's address space (symmetric memory), and ONE kernel per rank does, for its 1/world shard:
//     g   = (sum over ranks r of grad_r[i]) / world        plain peer loads over NVLink, fixed order
//     w,m,v <- AdamW(w, g, m, v)                            moments exist for the shard only
//     param_r[i] = w for every rank r                       plain peer stores over NVLink
// i.e. reduce-scatter + optimiser + all-gather without a separate collective and without a
// second pass over the gradients; each parameter element is reduced and updated by exactly one
// rank, so all replicas stay bit-identical.  Ordering between ranks (gradients complete before
// they are read, parameters complete before the next forward reads them) is provided by the
// caller with stream-ordered barriers around the launch; the kernel itself never waits.
// Only ordinary ld / st instructions touch peer pointers.
#include "common.cuh"
#include "launch.h"

#define SNB_MAX_PEERS 16

namespace snb {

struct PeerBuffers {
    const float4* grad[SNB_MAX_PEERS];
    float4* param[SNB_MAX_PEERS];
};

// WORLD is a template parameter so that the peer pointers are compile-time-indexed kernel parameters
// (a run-time index sends the pointer table to local memory and serialises the loads behind it) and
// all peer loads of an element are in flight together.
template <int WORLD>
__global__ void __launch_bounds__(256) dp_adamw_kernel(const PeerBuffers pb, float4* __restrict__ m,
                                                       float4* __restrict__ v, const float4* own_param,
                                                       size_t lo4, size_t hi4, float decay, float b1, float b2,
                                                       float step_size, float inv_sqrt_bc2, float eps, float inv_world) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = lo4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < hi4; i += stride) {
        float4 t[WORLD];
#pragma unroll
        for (int r = 0; r < WORLD; r++) t[r] = pb.grad[r][i];
        float4 gs = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < WORLD; r++) {
            gs.x += t[r].x;
            gs.y += t[r].y;
            gs.z += t[r].z;
            gs.w += t[r].w;
        }
        float4 wv = own_param[i], mv = m[i - lo4], vv = v[i - lo4];
        float* wp = reinterpret_cast<float*>(&wv);
        const float* gp = reinterpret_cast<const float*>(&gs);
        float* mp = reinterpret_cast<float*>(&mv);
        float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float gk = gp[k] * inv_world;
            mp[k] = b1 * mp[k] + (1.0f - b1) * gk;
            vp[k] = b2 * vp[k] + (1.0f - b2) * gk * gk;
            const float denom = sqrtf(vp[k]) * inv_sqrt_bc2 + eps;
            wp[k] = wp[k] * decay - step_size * (mp[k] / denom);
        }
        m[i - lo4] = mv;
        v[i - lo4] = vv;
#pragma unroll
        for (int r = 0; r < WORLD; r++) pb.param[r][i] = wv;
    }
}

}  // namespace snb

using namespace snb;

// grad_ptrs / param_ptrs: `world` device pointers each (host arrays), the same flat buffers on
// every rank, entry `rank` being this GPU's own.  [lo, hi) is this rank's shard in elements
// (multiples of 4); m and v hold hi - lo elements.
extern "C" int snb_dp_adamw_step(const void* const* grad_ptrs, void* const* param_ptrs, float* m, float* v,
                                 int rank, int world, long long lo, long long hi, float lr, float beta1,
                                 float beta2, float eps, float weight_decay, int step, void* stream) {
    if (!grad_ptrs || !param_ptrs || !m || !v) return SNB_ERR_NULL_POINTER;
    if (world < 1 || world > SNB_MAX_PEERS || rank < 0 || rank >= world) return SNB_ERR_UNSUPPORTED;
    if (lo < 0 || hi < lo || (lo & 3) || (hi & 3) || step <= 0) return SNB_ERR_BAD_SHAPE;
    PeerBuffers pb;
    for (int r = 0; r < SNB_MAX_PEERS; r++) {
        pb.grad[r] = nullptr;
        pb.param[r] = nullptr;
    }
    for (int r = 0; r < world; r++) {
        if (!grad_ptrs[r] || !param_ptrs[r]) return SNB_ERR_NULL_POINTER;
        if (!aligned16(grad_ptrs[r]) || !aligned16(param_ptrs[r])) return SNB_ERR_ALIGNMENT;
        pb.grad[r] = static_cast<const float4*>(grad_ptrs[r]);
        pb.param[r] = static_cast<float4*>(param_ptrs[r]);
    }
    if (!aligned16(m) || !aligned16(v)) return SNB_ERR_ALIGNMENT;
    if (hi == lo) return SNB_OK;
    const double bc1 = 1.0 - pow((double)beta1, step), bc2 = 1.0 - pow((double)beta2, step);
    const int blocks = sm_count() * 4;
    cudaStream_t st = (cudaStream_t)stream;
#define SNB_DP_CASE(W)                                                                                              \
    case W:                                                                                                         \
        dp_adamw_kernel<W><<<blocks, 256, 0, st>>>(pb, reinterpret_cast<float4*>(m), reinterpret_cast<float4*>(v),   \
                                                   pb.param[rank], (size_t)lo / 4, (size_t)hi / 4,                   \
                                                   1.0f - lr * weight_decay, beta1, beta2, (float)(lr / bc1),        \
                                                   (float)(1.0 / sqrt(bc2)), eps, 1.0f / (float)world);              \
        break;
    switch (world) {
        SNB_DP_CASE(1) SNB_DP_CASE(2) SNB_DP_CASE(3) SNB_DP_CASE(4) SNB_DP_CASE(5) SNB_DP_CASE(6) SNB_DP_CASE(7)
        SNB_DP_CASE(8) SNB_DP_CASE(9) SNB_DP_CASE(10) SNB_DP_CASE(11) SNB_DP_CASE(12) SNB_DP_CASE(13)
        SNB_DP_CASE(14) SNB_DP_CASE(15) SNB_DP_CASE(16)
    }
#undef SNB_DP_CASE
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}
