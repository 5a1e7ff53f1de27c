// Layer-level entry points: one call per fully connected norm-distance layer and direction, and
// the head of the SortNet-MLP (margin + mixture loss, certified fraction, input box).
//
// In the reference one layer of the forward is a chain of Python calls: the distance operator
// (core/norm_dist.py:56-99), MeanShiftDropout (core/models/bound_basic_module.py:123-157, about a
// dozen PyTorch launches), the bias add (core/models/norm_dist.py:102-103); the model tail is
// ell_inf_models.py:45-50 (margin) followed by the loss (main.py:357-364).  At 64-128 rows per GPU
// the host time of those chains exceeds the GPU time of the layer.  Each function below enqueues
// the kernels of one such chain from C, so the host pays for one call; the arithmetic is that of
// the separate entry points, in the same order (results are bit-identical to calling them one by
// one).
#include "../../include/sortnet_b200.h"
#include "common.cuh"
#include "launch.h"

namespace snb {

// out[b, j] = (x[b, j] - mean[idx]) + bias[idx], idx = index[s_b][j] or j; mean / bias may be null.
// The two additions are separate fp32 operations in this order, as in the reference.
// y may be x (in place).
__global__ void __launch_bounds__(256) shift_bias_kernel(const float* x, const float* __restrict__ mean,
                                                         const float* __restrict__ bias,
                                                         const int* __restrict__ index, int B, int C, float* y) {
    const int j = blockIdx.x * 256 + threadIdx.x;
    if (j >= C) return;
    const int s = blockIdx.y;
    const int c = index ? index[(size_t)s * C + j] : j;
    const float m = mean ? mean[c] : 0.f, bv = bias ? bias[c] : 0.f;
    const int b0 = s * SNB_SUB_BATCH, b1 = min(B, b0 + SNB_SUB_BATCH);
    for (int b = b0; b < b1; b++) {
        float v = x[(size_t)b * C + j];
        if (mean) v = v - m;
        if (bias) v = v + bv;
        y[(size_t)b * C + j] = v;
    }
}

// The same for the three tensors of an evaluation-mode bound pass (no index lists there), in place.
__global__ void __launch_bounds__(256) shift_bias3_kernel(float* __restrict__ y, float* __restrict__ yl,
                                                          float* __restrict__ yu, const float* __restrict__ mean,
                                                          const float* __restrict__ bias, int B, int C) {
    const size_t n = (size_t)B * C;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
        const int c = (int)(i % C);
        const float m = mean ? mean[c] : 0.f, bv = bias ? bias[c] : 0.f;
        float* ptrs[3] = {y, yl, yu};
#pragma unroll
        for (int k = 0; k < 3; k++) {
            if (!ptrs[k]) continue;
            float v = ptrs[k][i];
            if (mean) v = v - m;
            if (bias) v = v + bv;
            ptrs[k][i] = v;
        }
    }
}

// sum[c] = sum over the rows whose sub-batch kept channel c of g[b, slot(c)] (bias gradient).
// Fixed summation order: rows ascending inside a sub-batch, then the sub-batches' partial sums
// ascending.  CTA = 16 channels x 16 lanes; lane sg takes the sub-batches sg, sg + 16, ..., leaves
// their partial sums in shared memory, and lane 0 adds them in order (up to COLSUM_MAX_S
// sub-batches; beyond that the partial sums are added as they come, by one thread per channel).
constexpr int COLSUM_MAX_S = 64;

__device__ __forceinline__ float column_part(const float* __restrict__ g, const int* __restrict__ index, int B, int C,
                                             int c, int s, bool* kept) {
    int slot = c;
    if (index) {
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
    *kept = slot >= 0;
    if (slot < 0) return 0.f;
    const int b0 = s * SNB_SUB_BATCH, b1 = min(B, b0 + SNB_SUB_BATCH);
    float part = 0.f;
    for (int b = b0; b < b1; b++) part += g[(size_t)b * C + slot];
    return part;
}

__global__ void __launch_bounds__(256) column_sum_kernel(const float* __restrict__ g, const int* __restrict__ index,
                                                         int B, int C, int C_full, float* __restrict__ sum) {
    __shared__ float parts[COLSUM_MAX_S][17];
    __shared__ unsigned char have[COLSUM_MAX_S][17];
    const int cx = threadIdx.x & 15, sg = threadIdx.x >> 4;
    const int c = blockIdx.x * 16 + cx;
    const int S = (B + SNB_SUB_BATCH - 1) / SNB_SUB_BATCH;
    if (S > COLSUM_MAX_S) {
        if (sg != 0 || c >= C_full) return;
        float total = 0.f;
        for (int s = 0; s < S; s++) {
            bool kept;
            const float part = column_part(g, index, B, C, c, s, &kept);
            if (kept) total += part;
        }
        sum[c] = total;
        return;
    }
    if (c < C_full)
        for (int s = sg; s < S; s += 16) {
            bool kept;
            parts[s][cx] = column_part(g, index, B, C, c, s, &kept);
            have[s][cx] = kept;
        }
    __syncthreads();
    if (sg == 0 && c < C_full) {
        float total = 0.f;
        for (int s = 0; s < S; s++)
            if (have[s][cx]) total += parts[s][cx];
        sum[c] = total;
    }
}

// lower = max(x - eps, down), upper = min(x + eps, up) (ell_inf_models.py:35-36 with scalar bounds).
__global__ void __launch_bounds__(256) input_box_kernel(const float* __restrict__ x, float eps, float down, float up,
                                                        size_t n, float* __restrict__ xl, float* __restrict__ xu) {
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
        const float v = x[i];
        xl[i] = fmaxf(v - eps, down);
        xu[i] = fminf(v + eps, up);
    }
}

// One warp per row.  d [B, K] are the head's outputs (distances).  Margin of the training forward
// (ell_inf_models.py:45-50 with lower = d - eps, upper = d + eps):
//     margin[b, c] = ((d[b, t] + eps) - (d[b, c] - eps)) / (2 eps),   margin[b, t] = 0
// loss row = max_c clamp(margin, 0, clip) + lam * (logsumexp(-scale * d[b, :]) + scale * d[b, t])
// (main.py:357-364 `mixture`), and its gradient with respect to d for a unit upstream gradient
// and mean reduction over the B rows.
__global__ void __launch_bounds__(256) margin_loss_kernel(const float* __restrict__ d, const long long* __restrict__ target,
                                                          int B, int K, float eps, float two_eps, float clip, float lam,
                                                          float scale, float* __restrict__ margin_out,
                                                          float* __restrict__ row_loss, float* __restrict__ grad_d) {
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (b >= B) return;
    const float* dr = d + (size_t)b * K;
    const int t = (int)target[b];
    const float upper_t = dr[t] + eps;
    // pass 1: worst clamped margin (first index attaining it), max logit
    float worst = -1.f, best_margin = 0.f, zmax = -INFINITY;
    int worst_c = K;
    for (int c = lane; c < K; c += 32) {
        const float dv = dr[c];
        float m = (upper_t - (dv - eps)) / two_eps;
        if (c == t) m = 0.f;
        if (margin_out) margin_out[(size_t)b * K + c] = m;
        const float r = fminf(fmaxf(m, 0.f), clip);
        if (r > worst) {
            worst = r;
            worst_c = c;
            best_margin = m;
        }
        zmax = fmaxf(zmax, -scale * dv);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ow = __shfl_xor_sync(0xffffffffu, worst, o);
        const int oc = __shfl_xor_sync(0xffffffffu, worst_c, o);
        const float om = __shfl_xor_sync(0xffffffffu, best_margin, o);
        if (ow > worst || (ow == worst && oc < worst_c)) {
            worst = ow;
            worst_c = oc;
            best_margin = om;
        }
        zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, o));
    }
    // pass 2: softmax denominator
    float zsum = 0.f;
    for (int c = lane; c < K; c += 32) zsum += expf(-scale * dr[c] - zmax);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) zsum += __shfl_xor_sync(0xffffffffu, zsum, o);
    const float lse = zmax + logf(zsum);
    if (lane == 0) row_loss[b] = worst + lam * (lse + scale * dr[t]);
    if (!grad_d) return;
    // gradient: the margin term flows to (worst_c, t) when its margin lies inside the clamp range
    const float invB = 1.0f / (float)B, inv2eps = 1.0f / two_eps;
    const bool live = worst_c != t && best_margin >= 0.f && best_margin <= clip;
    for (int c = lane; c < K; c += 32) {
        const float soft = expf(-scale * dr[c] - lse);
        float gval = -scale * lam * (soft - (c == t ? 1.f : 0.f));
        if (live && c == worst_c) gval -= inv2eps;
        if (live && c == t) gval += inv2eps;
        grad_d[(size_t)b * K + c] = gval * invB;
    }
}

// loss = mean of row_loss in index order (deterministic); one block.
__global__ void __launch_bounds__(256) mean_rows_kernel(const float* __restrict__ row, int B, float* __restrict__ out) {
    __shared__ float part[256];
    float s = 0.f;
    const int per = (B + 255) / 256, b0 = threadIdx.x * per, b1 = min(B, b0 + per);
    for (int b = b0; b < b1; b++) s += row[b];
    part[threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int k = 0; k < 256; k++) t += part[k];
        *out = t / (float)B;
    }
}

// flag[b] = 1 when every wrong class's worst-case margin is negative:
// max_{c != t} ((-yl[b, c]) - (-yu[b, t])) < 0 (ell_inf_models.py:45-50 on the bounds; main.py:225-227).
__global__ void __launch_bounds__(256) certified_rows_kernel(const float* __restrict__ yl, const float* __restrict__ yu,
                                                             const long long* __restrict__ target, int B, int K,
                                                             float* __restrict__ flag) {
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (b >= B) return;
    const int t = (int)target[b];
    const float lo_t = -yu[(size_t)b * K + t];
    float worst = -INFINITY;
    for (int c = lane; c < K; c += 32)
        if (c != t) worst = fmaxf(worst, (-yl[(size_t)b * K + c]) - lo_t);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) worst = fmaxf(worst, __shfl_xor_sync(0xffffffffu, worst, o));
    if (lane == 0) flag[b] = worst < 0.f ? 1.f : 0.f;
}

}  // namespace snb

using namespace snb;

static int check2d(int B, int CO, int CI) {
    if (B <= 0 || CO <= 0 || CI <= 0) return SNB_ERR_BAD_SHAPE;
    if ((long long)B * CO >= (1ll << 31) || (long long)B * CI >= (1ll << 31)) return SNB_ERR_TOO_LARGE;
    return SNB_OK;
}

extern "C" int snb_layer_forward(const float* x, const float* w, int B, int CO, int CI, float p,
                                 const int* w_index_ci, const int* w_index_co, int W_CO, int W_CI, float* y_dist,
                                 int* pos, void* workspace, size_t workspace_bytes, float* running_mean,
                                 float momentum, float* mean, const float* bias, float* out, void* stream) {
    if (!x || !w || !y_dist || !out) return SNB_ERR_NULL_POINTER;
    int rc = check2d(B, CO, CI);
    if (rc) return rc;
    if (isinf(p)) {
        if (pos)
            rc = snb_inf_dist_forward_sorted_ws(x, w, B, CO, CI, 1, 1, y_dist, pos, w_index_ci, w_index_co, W_CO, W_CI,
                                                workspace, workspace_bytes, stream);
        else if (!w_index_ci && !w_index_co)
            rc = snb_inf_dist_forward_nograd(x, w, B, CO, CI, 1, 1, y_dist, stream);
        else
            return SNB_ERR_NULL_POINTER;      // masked forward always records positions
    } else {
        rc = snb_norm_dist_forward_ws(x, w, B, CO, CI, 1, 1, y_dist, p, w_index_ci, w_index_co, W_CO, W_CI, workspace,
                                      workspace_bytes, stream);
    }
    if (rc) return rc;
    const bool shift = mean != nullptr;
    if (shift) {
        rc = snb_mean_shift_stats(y_dist, w_index_co, B, CO, W_CO, mean, running_mean, momentum, stream);
        if (rc) return rc;
    }
    if (shift || bias || out != y_dist) {
        dim3 grid((CO + 255) / 256, (B + SNB_SUB_BATCH - 1) / SNB_SUB_BATCH);
        shift_bias_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(y_dist, shift ? mean : nullptr, bias, w_index_co, B,
                                                                  CO, out);
        SNB_CUDA(cudaGetLastError());
    }
    return SNB_OK;
}

extern "C" int snb_layer_backward(const float* grad_out, const float* x, const float* w, const float* y_dist,
                                  const int* pos, int B, int CO, int CI, float p, const int* w_index_ci,
                                  const int* w_index_co, int W_CO, int W_CI, int mean_shift, float* mean,
                                  float* grad_centred, float* grad_bias, float* grad_x, float* grad_w,
                                  void* stream) {
    if (!grad_out) return SNB_ERR_NULL_POINTER;
    int rc = check2d(B, CO, CI);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (grad_bias) {
        column_sum_kernel<<<(W_CO + 15) / 16, 256, 0, st>>>(grad_out, w_index_co, B, CO, W_CO, grad_bias);
        SNB_CUDA(cudaGetLastError());
    }
    const float* g = grad_out;
    if (mean_shift) {
        // the reference differentiates through the batch mean: the gradient is centred the same way
        if (!mean || !grad_centred) return SNB_ERR_NULL_POINTER;
        rc = snb_mean_shift_stats(grad_out, w_index_co, B, CO, W_CO, mean, nullptr, 0.f, stream);
        if (rc) return rc;
        rc = snb_mean_shift_apply(grad_out, mean, w_index_co, B, CO, grad_centred, stream);
        if (rc) return rc;
        g = grad_centred;
    }
    if (!grad_x) return grad_w ? SNB_ERR_NULL_POINTER : SNB_OK;
    if (isinf(p)) {
        if (!pos) return SNB_ERR_NULL_POINTER;
        return grad_w ? snb_inf_dist_backward_input_weight(g, pos, B, CO, CI, 1, 1, grad_x, grad_w, w_index_ci,
                                                           w_index_co, W_CO, W_CI, stream)
                      : snb_inf_dist_backward_input(g, pos, B, CO, CI, 1, 1, grad_x, stream);
    }
    return grad_w ? snb_norm_dist_backward_input_weight(g, x, w, y_dist, B, CO, CI, 1, 1, grad_x, grad_w, p,
                                                        w_index_ci, w_index_co, W_CO, W_CI, stream)
                  : snb_norm_dist_backward_input(g, x, w, y_dist, B, CO, CI, 1, 1, grad_x, p, w_index_ci, w_index_co,
                                                 W_CO, W_CI, stream);
}

extern "C" int snb_layer_bound_forward(const float* x, const float* xl, const float* xu, const float* w, int B, int CO,
                                       int CI, const float* running_mean, const float* bias, float* y, float* yl,
                                       float* yu, void* stream) {
    if (!w || (!x && !xl)) return SNB_ERR_NULL_POINTER;
    int rc = check2d(B, CO, CI);
    if (rc) return rc;
    if (x) {
        if (!y) return SNB_ERR_NULL_POINTER;
        rc = snb_inf_dist_forward_nograd(x, w, B, CO, CI, 1, 1, y, stream);
        if (rc) return rc;
    }
    if (xl) {
        if (!xu || !yl || !yu) return SNB_ERR_NULL_POINTER;
        rc = snb_bound_inf_dist_forward_nograd(xl, xu, w, B, CO, CI, 1, 1, yl, yu, stream);
        if (rc) return rc;
    }
    if (running_mean || bias) {
        const size_t n = (size_t)B * CO;
        const int blocks = (int)((n + 255) / 256 < 2368 ? (n + 255) / 256 : 2368);
        shift_bias3_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x ? y : nullptr, xl ? yl : nullptr,
                                                                     xl ? yu : nullptr, running_mean, bias, B, CO);
        SNB_CUDA(cudaGetLastError());
    }
    return SNB_OK;
}

extern "C" int snb_input_box(const float* x, float eps, float down, float up, long long n, float* xl, float* xu,
                             void* stream) {
    if (!x || !xl || !xu) return SNB_ERR_NULL_POINTER;
    if (n <= 0) return SNB_ERR_BAD_SHAPE;
    const int blocks = (int)((n + 255) / 256 < 2368 ? (n + 255) / 256 : 2368);
    input_box_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, eps, down, up, (size_t)n, xl, xu);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

extern "C" int snb_margin_loss(const float* d, const long long* target, int B, int K, float eps, float clip, float lam,
                               float scale, float* margin, float* row_loss, float* loss, float* grad_d, void* stream) {
    if (!d || !target || !row_loss || !loss) return SNB_ERR_NULL_POINTER;
    if (B <= 0 || K <= 0 || !(eps > 0.f)) return SNB_ERR_BAD_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    margin_loss_kernel<<<(B + 7) / 8, 256, 0, st>>>(d, target, B, K, eps, 2.0f * eps, clip, lam, scale, margin, row_loss,
                                                    grad_d);
    SNB_CUDA(cudaGetLastError());
    mean_rows_kernel<<<1, 256, 0, st>>>(row_loss, B, loss);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

extern "C" int snb_certified_fraction(const float* yl, const float* yu, const long long* target, int B, int K,
                                      float* row_flag, float* fraction, void* stream) {
    if (!yl || !yu || !target || !row_flag || !fraction) return SNB_ERR_NULL_POINTER;
    if (B <= 0 || K <= 0) return SNB_ERR_BAD_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    certified_rows_kernel<<<(B + 7) / 8, 256, 0, st>>>(yl, yu, target, B, K, row_flag);
    SNB_CUDA(cudaGetLastError());
    mean_rows_kernel<<<1, 256, 0, st>>>(row_flag, B, fraction);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}
