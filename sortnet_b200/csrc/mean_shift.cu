// Mean-shift normalisation that follows every hidden norm-distance layer.
//
// Replaces the ~12 PyTorch element-wise / scatter launches of MeanShiftDropout.forward in
// zbh2047/SortNet core/models/bound_basic_module.py:123-157 (no native counterpart there).
//
//   stats : mean[c] = sum over rows b whose 32-row sub-batch kept channel c of x[b, slot(c)]
//                     / max(number of such rows, 1e-10)           (0 for never-kept channels)
//           running_mean = (1 - momentum) * running_mean + momentum * mean      (optional)
//   apply : y[b, j] = x[b, j] - mean[index[s_b][j]]                (index NULL = identity)
//
// The training-mode backward is the same pair applied to the incoming gradient, because the
// reference differentiates through the batch mean.  Both kernels are deterministic: sums run
// in a fixed order (rows ascending inside a sub-batch, sub-batches combined in a fixed tree).
#include "common.cuh"
#include "launch.h"

namespace snb {

// CTA = 16 channels x 16 sub-batch lanes.  Lane (cx, sg) sums channel c over the sub-batches
// sg, sg + 16, ...; the 16 partial sums are then added in index order.  The kernel is bound by the
// latency of each lane's chain (a binary search in the sorted list, then 32 rows), hence many short
// chains.
__global__ void __launch_bounds__(256) mean_shift_stats_kernel(const float* __restrict__ x,
                                                               const int* __restrict__ index, int B,
                                                               int C, int C_full, float* __restrict__ mean,
                                                               float* __restrict__ running_mean,
                                                               float momentum) {
    __shared__ float ssum[16][17];
    __shared__ float scnt[16][17];
    const int cx = threadIdx.x & 15, sg = threadIdx.x >> 4;
    const int c = blockIdx.x * 16 + cx;
    const int S = (B + SNB_SUB_BATCH - 1) / SNB_SUB_BATCH;
    float sum = 0.f, cnt = 0.f;
    if (c < C_full) {
        for (int s = sg; s < S; s += 16) {
            int slot = c;
            if (index) {
                // lower bound of c in the sorted kept-channel list of sub-batch s
                const int* idx = index + (size_t)s * C;
                int lo = 0, hi = C;
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (idx[mid] < c) lo = mid + 1;
                    else hi = mid;
                }
                slot = (lo < C && idx[lo] == c) ? lo : -1;
            } else if (c >= C) {
                slot = -1;
            }
            if (slot < 0) continue;
            const int b0 = s * SNB_SUB_BATCH, b1 = min(B, b0 + SNB_SUB_BATCH);
            float part = 0.f;
            for (int b = b0; b < b1; b++) part += x[(size_t)b * C + slot];
            sum += part;
            cnt += (float)(b1 - b0);
        }
    }
    ssum[sg][cx] = sum;
    scnt[sg][cx] = cnt;
    __syncthreads();
    if (sg == 0 && c < C_full) {
        float t = 0.f, n = 0.f;
#pragma unroll
        for (int k = 0; k < 16; k++) {
            t += ssum[k][cx];
            n += scnt[k][cx];
        }
        const float m = t / fmaxf(n, 1e-10f);
        mean[c] = m;
        if (running_mean) running_mean[c] = running_mean[c] * (1.0f - momentum) + momentum * m;
    }
}

__global__ void __launch_bounds__(256) mean_shift_apply_kernel(const float* __restrict__ x,
                                                               const float* __restrict__ mean,
                                                               const int* __restrict__ index, int B,
                                                               int C, float* __restrict__ y) {
    const int j = blockIdx.x * 256 + threadIdx.x;
    if (j >= C) return;
    const int s = blockIdx.y;
    const float m = mean[index ? index[(size_t)s * C + j] : j];
    const int b0 = s * SNB_SUB_BATCH, b1 = min(B, b0 + SNB_SUB_BATCH);
    for (int b = b0; b < b1; b++) y[(size_t)b * C + j] = x[(size_t)b * C + j] - m;
}

}  // namespace snb

using namespace snb;

extern "C" int snb_mean_shift_stats(const float* x, const int* index, int B, int C, int C_full,
                                    float* mean, float* running_mean, float momentum, void* stream) {
    if (!x || !mean) return SNB_ERR_NULL_POINTER;
    if (B <= 0 || C <= 0 || C_full < C || (!index && C_full != C)) return SNB_ERR_BAD_SHAPE;
    if ((long long)B * C >= (1ll << 31)) return SNB_ERR_TOO_LARGE;
    mean_shift_stats_kernel<<<(C_full + 15) / 16, 256, 0, (cudaStream_t)stream>>>(
        x, index, B, C, C_full, mean, running_mean, momentum);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

extern "C" int snb_mean_shift_apply(const float* x, const float* mean, const int* index, int B, int C,
                                    float* y, void* stream) {
    if (!x || !mean || !y) return SNB_ERR_NULL_POINTER;
    if (B <= 0 || C <= 0) return SNB_ERR_BAD_SHAPE;
    if ((long long)B * C >= (1ll << 31)) return SNB_ERR_TOO_LARGE;
    dim3 grid((C + 255) / 256, (B + SNB_SUB_BATCH - 1) / SNB_SUB_BATCH);
    mean_shift_apply_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, mean, index, B, C, y);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}
