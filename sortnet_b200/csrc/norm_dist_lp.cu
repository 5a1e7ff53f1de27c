// l-p distance neuron (finite p): forward and the dense fused backward.
//
// Replaces zbh2047/SortNet core/cuda/norm_dist_cuda.cu (forward kernels :36-160 and :163-259,
// backward kernels :269-367 and :370-504; launchers :511-594) and the p dispatch of
// core/cuda/norm_dist.cpp:43-129.
//
//   p <= 10 :  y = max(sum_c |t|^p, FLT_MIN)^(1/p)                         t = x - w (fp32)
//   p  > 10 :  y = M * (sum_c (|t|/M)^p + (1e-10/M)^p)^(1/p),  M = max(1e-10, max_c |t|)
//   backward:  term = g * sgn(t) * (|t| / y)^(p-1);  grad_x[b,c] = sum_j term;
//              grad_w[co[s][j], ci[s][c]] -= sum_{b in sub-batch s} term
//
// The reference reaches the p > 10 value with an online running maximum that may lag the true
// maximum by 1e-6 relative; here M is the exact maximum, computed first by the l-infinity
// kernel into y, so the result is the exact-math value up to fp32 rounding.  Integer p in
// [1, 8] uses multiply chains (as the reference does), any other p uses exp2(p * log2 r) with
// the full-precision log2f / exp2f so that the p-fold error amplification stays inside 1e-5.
#include <float.h>
#include "tile.cuh"
#include "launch.h"

namespace snb {

// defined in inf_dist.cu: y = max(1e-10, max_c |x - w|) with optional index lists, no argmax
cudaError_t inf_forward_values(const float* x, const float* w, float* y, const int* ci, const int* co,
                               int B, int CO, int CI, int W_CI, cudaStream_t st);

// |r|^IP for integer IP (multiply chain) or r^e for IP < 0 (r >= 0).
template <int IP>
__device__ __forceinline__ float pow_abs(float r, float e) {
    if (IP == 0) return 1.0f;
    if (IP == 1) return fabsf(r);
    if (IP == 2) return r * r;
    if (IP == 3) return fabsf(r) * r * r;
    if (IP == 4) { float a = r * r; return a * a; }
    if (IP == 5) { float a = r * r; return fabsf(r) * a * a; }
    if (IP == 6) { float a = r * r; return a * a * a; }
    if (IP == 7) { float a = r * r; return fabsf(r) * a * a * a; }
    if (IP == 8) { float a = r * r; a = a * a; return a * a; }
    return exp2f(e * log2f(fabsf(r)));
}

// sgn(r) * |r|^IP.
template <int IP>
__device__ __forceinline__ float pow_signed(float r, float e) {
    if (IP == 0) return r >= 0 ? 1.0f : -1.0f;
    if (IP == 1) return r;
    if (IP == 2) return fabsf(r) * r;
    if (IP == 3) return r * r * r;
    if (IP == 4) { float a = r * r; return fabsf(r) * r * a; }
    if (IP == 5) { float a = r * r; return a * a * r; }
    if (IP == 6) { float a = r * r; return fabsf(r) * r * a * a; }
    if (IP == 7) { float a = r * r; return a * a * a * r; }
    return copysignf(exp2f(e * log2f(fabsf(r))), r);
}

struct LpFwdParams {
    const float* x;
    const float* w;
    float* y;  // NORMALISED: holds M on entry
    const int* ci;
    const int* co;
    int B, CO, CI, W_CI;
    float p;
};

enum { MODE_VEC = 0, MODE_SCALAR = 1, MODE_GATHER = 2 };

// 32 x (64 * WN) tile per CTA (one sub-batch of rows), 8x8 outputs per thread.
template <int WN, int MODE, int IP, bool NORMALISED>
__global__ void __launch_bounds__(WN * 32) lp_fwd_kernel(const LpFwdParams p) {
    constexpr int BM = 32, BN = 64 * WN, NT = WN * 32;
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;
    float* ws = smem + 2 * BM * LDS;
    const int tid = threadIdx.x, lane = tid & 31, wn = tid >> 5, tb = lane >> 3, tj = lane & 7;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int nk = (p.CI + BK - 1) / BK;

    GatherW<BN, NT> gw;
    const int* ci_s = nullptr;
    if (MODE == MODE_GATHER) {
        const int s = m0 / SNB_SUB_BATCH;
        ci_s = p.ci ? p.ci + (size_t)s * p.CI : nullptr;
        gw.init_rows(p.co ? p.co + (size_t)s * p.CO : nullptr, n0, p.CO, p.W_CI, tid);
        gw.fetch_cols(ci_s, 0, p.CI, tid);
    }
    auto stage = [&](int kt, int st) {
        float* xd = xs + st * BM * LDS;
        float* wd = ws + st * BN * LDS;
        if (MODE == MODE_VEC) {
            stage_dense_vec<BM, NT>(xd, p.x, m0, p.B, p.CI, kt * BK, p.CI, tid);
            stage_dense_vec<BN, NT>(wd, p.w, n0, p.CO, p.W_CI, kt * BK, p.CI, tid);
        } else if (MODE == MODE_SCALAR) {
            stage_dense_scalar<BM, NT>(xd, p.x, m0, p.B, p.CI, kt * BK, p.CI, tid);
            stage_dense_scalar<BN, NT>(wd, p.w, n0, p.CO, p.W_CI, kt * BK, p.CI, tid);
        } else {
            stage_dense_scalar<BM, NT>(xd, p.x, m0, p.B, p.CI, kt * BK, p.CI, tid);
            gw.stage(wd, p.w, tid);
        }
    };

    float acc[8][8], rm[NORMALISED ? 8 : 1][NORMALISED ? 8 : 1];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            acc[i][j] = 0.f;
            if (NORMALISED) {
                const int m = m0 + tb + 4 * i, n = n0 + wn * 64 + tj + 8 * j;
                const float mx = (m < p.B && n < p.CO) ? p.y[(size_t)m * p.CO + n] : 1.0f;
                rm[i][j] = 1.0f / mx;
                acc[i][j] = pow_abs<IP>(SNB_EPS * rm[i][j], p.p);  // the (EPS / M)^p seed term
            }
        }

    stage(0, 0);
    cp_async_commit();
    for (int kt = 0; kt < nk; kt++) {
        cp_async_wait<0>();
        __syncthreads();
        if (kt + 1 < nk) {
            if (MODE == MODE_GATHER) gw.fetch_cols(ci_s, (kt + 1) * BK, p.CI, tid);
            stage(kt + 1, (kt + 1) & 1);
        }
        cp_async_commit();
        const float* xr = xs + (kt & 1) * BM * LDS + tb * LDS;
        const float* wr = ws + (kt & 1) * BN * LDS + (wn * 64 + tj) * LDS;
        // zero-filled padding (x = w = 0) contributes |0|^p = 0 for every p > 0
#pragma unroll 2
        for (int kk = 0; kk < BK / 2; kk++) {
            float2 xf[8], wf[8];
#pragma unroll
            for (int i = 0; i < 8; i++) xf[i] = *reinterpret_cast<const float2*>(xr + i * 4 * LDS + kk * 2);
#pragma unroll
            for (int j = 0; j < 8; j++) wf[j] = *reinterpret_cast<const float2*>(wr + j * 8 * LDS + kk * 2);
#pragma unroll
            for (int i = 0; i < 8; i++) {
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    float t0 = xf[i].x - wf[j].x, t1 = xf[i].y - wf[j].y;
                    if (NORMALISED) {
                        t0 *= rm[i][j];
                        t1 *= rm[i][j];
                    }
                    acc[i][j] += pow_abs<IP>(t0, p.p);
                    acc[i][j] += pow_abs<IP>(t1, p.p);
                }
            }
        }
    }
    const float rp = 1.0f / p.p;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int m = m0 + tb + 4 * i;
        if (m >= p.B) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int n = n0 + wn * 64 + tj + 8 * j;
            if (n >= p.CO) continue;
            float r;
            if (NORMALISED) r = exp2f(rp * log2f(acc[i][j])) / rm[i][j];
            else r = exp2f(rp * log2f(fmaxf(acc[i][j], FLT_MIN)));
            p.y[(size_t)m * p.CO + n] = r;
        }
    }
}

struct LpBwdParams {
    const float* g;
    const float* x;
    const float* w;
    const float* y;
    float* gx;
    float* gw;  // may be null: grad_x only
    const int* ci;
    const int* co;
    int B, CO, CI, W_CI;
    float pm1;  // p - 1
};

// One CTA = one 32-row sub-batch x 256 compact input columns; it walks all outputs j.
// Thread (tb, tc): rows tb*8 .. tb*8+7, columns 4*tc .. 4*tc+3; the four tb lanes that share
// tc sit in one warp (lane = (tc % 8) * 4 + tb), so the per-(j, c) sums over the 32 rows
// finish with two shuffles and one global reduction.
template <int IP>
__global__ void __launch_bounds__(256) lp_bwd_kernel(const LpBwdParams p) {
    constexpr int JT = 32;
    __shared__ float2 gr[JT][32 + 1];  // (g, 1/y) for [j][b]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tb = lane & 3, tc = warp * 8 + (lane >> 2);
    const int s = blockIdx.x, b0 = s * SNB_SUB_BATCH;
    const int c0 = blockIdx.y * 256 + tc * 4;
    const int* ci_s = p.ci ? p.ci + (size_t)s * p.CI : nullptr;
    const int* co_s = p.co ? p.co + (size_t)s * p.CO : nullptr;

    int col[4];
    float xv[8][4], gx[8][4];
#pragma unroll
    for (int k = 0; k < 4; k++) col[k] = (c0 + k < p.CI) ? (ci_s ? ci_s[c0 + k] : c0 + k) : -1;
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int b = b0 + tb * 8 + i;
            xv[i][k] = (b < p.B && col[k] >= 0) ? p.x[(size_t)b * p.CI + c0 + k] : 0.f;
            gx[i][k] = 0.f;
        }

    for (int j0 = 0; j0 < p.CO; j0 += JT) {
        __syncthreads();
        for (int e = tid; e < JT * 32; e += 256) {
            const int jj = e & 31, bb = e >> 5;  // consecutive threads -> consecutive j (coalesced)
            const int b = b0 + bb, j = j0 + jj;
            float2 v = make_float2(0.f, 0.f);
            if (b < p.B && j < p.CO) {
                v.x = p.g[(size_t)b * p.CO + j];
                v.y = 1.0f / p.y[(size_t)b * p.CO + j];
            }
            gr[jj][bb] = v;
        }
        __syncthreads();
        const int jn = min(JT, p.CO - j0);
        for (int jj = 0; jj < jn; jj++) {
            const int row = co_s ? co_s[j0 + jj] : j0 + jj;
            const float* wrow = p.w + (size_t)row * p.W_CI;
            float wv[4], gwp[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                wv[k] = col[k] >= 0 ? wrow[col[k]] : 0.f;
                gwp[k] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float2 gy = gr[jj][tb * 8 + i];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float u = (xv[i][k] - wv[k]) * gy.y;
                    const float term = gy.x * pow_signed<IP>(u, p.pm1);
                    gx[i][k] += term;
                    gwp[k] += term;
                }
            }
            if (p.gw) {
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    gwp[k] += __shfl_xor_sync(0xffffffffu, gwp[k], 1);
                    gwp[k] += __shfl_xor_sync(0xffffffffu, gwp[k], 2);
                }
                if (tb == 0) {
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        if (col[k] >= 0) atomicAdd(p.gw + (size_t)row * p.W_CI + col[k], -gwp[k]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int b = b0 + tb * 8 + i;
        if (b >= p.B) continue;
#pragma unroll
        for (int k = 0; k < 4; k++)
            if (col[k] >= 0) p.gx[(size_t)b * p.CI + c0 + k] = gx[i][k];
    }
}

template <int WN, int MODE, int IP, bool NORM>
static cudaError_t launch_lp_fwd(const LpFwdParams& p, cudaStream_t st) {
    constexpr int BN = 64 * WN;
    constexpr int SMEM = 2 * (32 + BN) * LDS * (int)sizeof(float);
    auto kern = lp_fwd_kernel<WN, MODE, IP, NORM>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        configured[dev & 63] = true;
    }
    dim3 grid((p.B + 31) / 32, (p.CO + BN - 1) / BN);
    kern<<<grid, WN * 32, SMEM, st>>>(p);
    return cudaGetLastError();
}

template <int IP, bool NORM>
static cudaError_t dispatch_lp_mode(const LpFwdParams& p, cudaStream_t st) {
    if (p.ci || p.co) return launch_lp_fwd<4, MODE_GATHER, IP, NORM>(p, st);
    const bool vec = (p.CI % 4 == 0) && (p.W_CI % 4 == 0) && aligned16(p.x) && aligned16(p.w);
    return vec ? launch_lp_fwd<4, MODE_VEC, IP, NORM>(p, st) : launch_lp_fwd<4, MODE_SCALAR, IP, NORM>(p, st);
}

static int integer_power(float p) {
    const int ip = (int)p;
    return (p == (float)ip && ip >= 0 && ip <= 8) ? ip : -1;
}

}  // namespace snb

using namespace snb;

extern "C" int snb_norm_dist_forward(const float* x, const float* w, int B, int CO, int CI, int G,
                                     int HW, float* y, float p, const int* w_index_ci,
                                     const int* w_index_co, int W_CO, int W_CI, void* stream) {
    if (!x || !w || !y) return SNB_ERR_NULL_POINTER;
    if (G != 1 || HW != 1 || !(p > 0) || isinf(p)) return SNB_ERR_UNSUPPORTED;
    if (B <= 0 || CO <= 0 || CI <= 0 || W_CO <= 0 || W_CI <= 0) return SNB_ERR_BAD_SHAPE;
    if ((!w_index_ci && W_CI != CI) || (!w_index_co && W_CO != CO) || CI > W_CI || CO > W_CO)
        return SNB_ERR_BAD_SHAPE;
    if ((long long)W_CO * W_CI >= (1ll << 31) || (long long)B * CO >= (1ll << 31) || (long long)B * CI >= (1ll << 31))
        return SNB_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    LpFwdParams q{x, w, y, w_index_ci, w_index_co, B, CO, CI, W_CI, p};
    if (p > 10.0f) {
        SNB_CUDA(inf_forward_values(x, w, y, w_index_ci, w_index_co, B, CO, CI, W_CI, st));
        SNB_CUDA(dispatch_lp_mode<-1, true>(q, st));
        return SNB_OK;
    }
    switch (integer_power(p)) {
        case 1: SNB_CUDA(dispatch_lp_mode<1, false>(q, st)); break;
        case 2: SNB_CUDA(dispatch_lp_mode<2, false>(q, st)); break;
        case 3: SNB_CUDA(dispatch_lp_mode<3, false>(q, st)); break;
        case 4: SNB_CUDA(dispatch_lp_mode<4, false>(q, st)); break;
        case 5: SNB_CUDA(dispatch_lp_mode<5, false>(q, st)); break;
        case 6: SNB_CUDA(dispatch_lp_mode<6, false>(q, st)); break;
        case 7: SNB_CUDA(dispatch_lp_mode<7, false>(q, st)); break;
        case 8: SNB_CUDA(dispatch_lp_mode<8, false>(q, st)); break;
        default: SNB_CUDA(dispatch_lp_mode<-1, false>(q, st)); break;
    }
    return SNB_OK;
}

static int lp_backward(const float* g, const float* x, const float* w, const float* y, int B, int CO,
                       int CI, int G, int HW, float* gx, float* gw, float p, const int* ci,
                       const int* co, int W_CO, int W_CI, cudaStream_t st) {
    if (!g || !x || !w || !y || !gx) return SNB_ERR_NULL_POINTER;
    if (G != 1 || HW != 1 || !(p > 0) || isinf(p)) return SNB_ERR_UNSUPPORTED;
    if (B <= 0 || CO <= 0 || CI <= 0 || W_CO <= 0 || W_CI <= 0) return SNB_ERR_BAD_SHAPE;
    if ((!ci && W_CI != CI) || (!co && W_CO != CO) || CI > W_CI || CO > W_CO) return SNB_ERR_BAD_SHAPE;
    if ((long long)W_CO * W_CI >= (1ll << 31) || (long long)B * CO >= (1ll << 31) || (long long)B * CI >= (1ll << 31))
        return SNB_ERR_TOO_LARGE;
    if (gw) SNB_CUDA(cudaMemsetAsync(gw, 0, sizeof(float) * (size_t)W_CO * W_CI, st));
    LpBwdParams q{g, x, w, y, gx, gw, ci, co, B, CO, CI, W_CI, p - 1.0f};
    dim3 grid((B + 31) / 32, (CI + 255) / 256);
    switch (integer_power(p - 1.0f)) {
        case 0: lp_bwd_kernel<0><<<grid, 256, 0, st>>>(q); break;
        case 1: lp_bwd_kernel<1><<<grid, 256, 0, st>>>(q); break;
        case 2: lp_bwd_kernel<2><<<grid, 256, 0, st>>>(q); break;
        case 3: lp_bwd_kernel<3><<<grid, 256, 0, st>>>(q); break;
        case 4: lp_bwd_kernel<4><<<grid, 256, 0, st>>>(q); break;
        case 5: lp_bwd_kernel<5><<<grid, 256, 0, st>>>(q); break;
        case 6: lp_bwd_kernel<6><<<grid, 256, 0, st>>>(q); break;
        case 7: lp_bwd_kernel<7><<<grid, 256, 0, st>>>(q); break;
        default: lp_bwd_kernel<-1><<<grid, 256, 0, st>>>(q); break;
    }
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

extern "C" int snb_norm_dist_backward_input(const float* grad_output, const float* x, const float* w,
                                            const float* y, int B, int CO, int CI, int G, int HW,
                                            float* grad_input, float p, const int* w_index_ci,
                                            const int* w_index_co, int W_CO, int W_CI, void* stream) {
    return lp_backward(grad_output, x, w, y, B, CO, CI, G, HW, grad_input, nullptr, p, w_index_ci,
                       w_index_co, W_CO, W_CI, (cudaStream_t)stream);
}

extern "C" int snb_norm_dist_backward_input_weight(const float* grad_output, const float* x,
                                                   const float* w, const float* y, int B, int CO,
                                                   int CI, int G, int HW, float* grad_input,
                                                   float* grad_weight, float p, const int* w_index_ci,
                                                   const int* w_index_co, int W_CO, int W_CI,
                                                   void* stream) {
    if (!grad_weight) return SNB_ERR_NULL_POINTER;
    return lp_backward(grad_output, x, w, y, B, CO, CI, G, HW, grad_input, grad_weight, p, w_index_ci,
                       w_index_co, W_CO, W_CI, (cudaStream_t)stream);
}
