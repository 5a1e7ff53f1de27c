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
// [1, 8] uses multiply chains (as the reference does), any other p uses ex2(p * log2 r) on the
// special-function unit with a series for log2 near r = 1 (log2_rel), which keeps the p-fold
// amplification of the logarithm's error at the level of the fp32 rounding of r itself.
#include <float.h>
#include "tile.cuh"
#include "launch.h"
#include "general_shapes.h"

namespace snb {

// defined in inf_dist.cu: y = max(1e-10, max_c |x - w|) with optional index lists, no argmax
cudaError_t inf_forward_values(const float* x, const float* w, float* y, const int* ci, const int* co,
                               int B, int CO, int CI, int W_CI, cudaStream_t st);

// Special-function-unit exp2 / log2.  The .ftz forms skip the denormal fix-up code: a denormal
// argument of log2 reads as 0 (its power is 0 to fp32 anyway) and results below 2^-126 flush to 0.
__device__ __forceinline__ float ex2_approx(float z) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(z));
    return r;
}
__device__ __forceinline__ float lg2_approx(float a) {
    float r;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
    return r;
}

// log2(a) by a degree-8 series in d = a - 1 (exact subtraction), for |d| <= 0.125.  The hardware
// approximation has an absolute error of 2^-22, i.e. no relative accuracy near a = 1; the series
// keeps the relative error of log2 at fp32 level there, so that a^e for large e is as accurate as
// the fp32 rounding of a allows.
__device__ __forceinline__ float log2_series(float a) {
    const float d = a - 1.0f;
    float s = fmaf(d, -0.125f, 1.0f / 7.0f);
    s = fmaf(d, s, -1.0f / 6.0f);
    s = fmaf(d, s, 0.2f);
    s = fmaf(d, s, -0.25f);
    s = fmaf(d, s, 1.0f / 3.0f);
    s = fmaf(d, s, -0.5f);
    s = fmaf(d, s, 1.0f);
    return d * 1.4426950408889634f * s;
}
__device__ __forceinline__ bool near_one(float a) { return fabsf(a - 1.0f) <= 0.125f; }

// a^e for a >= 0, accurate per value (used once per output and in the backward).
__device__ __forceinline__ float pow_pos(float a, float e) {
    return ex2_approx(e * (near_one(a) ? log2_series(a) : lg2_approx(a)));
}
// a^e where only the *sum* of many such terms matters (forward): the absolute error of the
// hardware log2 perturbs the sum by ~1.7e-7 * e relative, and the e-th root taken afterwards
// divides that by e.
__device__ __forceinline__ float pow_pos_sum(float a, float e) { return ex2_approx(e * lg2_approx(a)); }

// |r|^IP for integer IP (multiply chain) or |r|^e for IP < 0; forward terms.
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
    return pow_pos_sum(fabsf(r), e);
}

// sgn(r) * |r|^IP; backward terms.
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
    return copysignf(pow_pos(fabsf(r), e), r);
}

struct LpFwdParams {
    const float* x;
    const float* w;
    float* y;
    const float* m;  // NORMALISED: the maxima M (may be y itself when direct)
    const int* ci;
    const int* co;
    int B, CO, CI, W_CI;
    float p;
    int direct;      // 1: one CTA per output tile, finished in the kernel; 0: shared tiles, lp_finish_kernel follows
};

enum { MODE_VEC = 0, MODE_SCALAR = 1, MODE_GATHER = 2 };

// 32 x (64 * WN) output tiles (one sub-batch of rows), 8x8 outputs per thread.  The (tile, k-tile)
// pairs of the whole problem form one sequence that is cut into gridDim.x equal ranges (see
// StreamK), so all SMs stay busy whatever the shape and the mask sizes.  With `direct` the grid
// has one CTA per tile and each CTA turns its sums into distances itself; otherwise every range
// adds its partial sums into the zero-filled y with atomics and lp_finish_kernel takes the root.
template <int WN, int MODE, int IP, bool NORMALISED>
__global__ void __launch_bounds__(WN * 32) lp_fwd_kernel(const LpFwdParams p) {
    constexpr int BM = 32, BN = 64 * WN, NT = WN * 32;
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;
    float* ws = smem + 2 * BM * LDS;
    const int tid = threadIdx.x, lane = tid & 31, wn = tid >> 5, tb = lane >> 3, tj = lane & 7;
    const int nk = (p.CI + BK - 1) / BK;
    const StreamK sk{(p.B + BM - 1) / BM, (p.CO + BN - 1) / BN, nk};
    long long u, u_end;
    sk.range(u, u_end);
    // worth testing only when most elements qualify: at p >= 48 the cut is |t|/M < 0.56
    const bool use_skip = NORMALISED && p.p >= 48.0f;
    const float skip_below = exp2f(-40.0f / p.p);

  while (u < u_end) {
    const int tile = (int)(u / nk), kt_begin = (int)(u % nk);
    const int kt_end = (int)min((long long)nk, kt_begin + (u_end - u));
    const int m0 = (tile / sk.tiles_n) * BM, n0 = (tile % sk.tiles_n) * BN;

    GatherW<BN, NT> gw;
    const int* ci_s = nullptr;
    if (MODE == MODE_GATHER) {
        const int s = m0 / SNB_SUB_BATCH;
        ci_s = p.ci ? p.ci + (size_t)s * p.CI : nullptr;
        gw.init_rows(p.co ? p.co + (size_t)s * p.CO : nullptr, n0, p.CO, p.W_CI, tid);
        gw.fetch_cols(ci_s, kt_begin * BK, p.CI, tid);
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
                const float mx = (m < p.B && n < p.CO) ? p.m[(size_t)m * p.CO + n] : 1.0f;
                rm[i][j] = 1.0f / mx;
                // the (EPS / M)^p seed term, once per output
                if (kt_begin == 0) acc[i][j] = pow_abs<IP>(SNB_EPS * rm[i][j], p.p);
            }
        }

    __syncthreads();                           // everyone is done with the previous range's tiles
    stage(kt_begin, 0);
    cp_async_commit();
    if (MODE == MODE_GATHER && kt_begin + 1 < kt_end) gw.fetch_cols(ci_s, (kt_begin + 1) * BK, p.CI, tid);
    for (int kt = kt_begin; kt < kt_end; kt++) {
        const int cur = (kt - kt_begin) & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (kt + 1 < kt_end) {
            stage(kt + 1, cur ^ 1);
            if (MODE == MODE_GATHER && kt + 2 < kt_end) gw.fetch_cols(ci_s, (kt + 2) * BK, p.CI, tid);
        }
        cp_async_commit();
        const float* xr = xs + cur * BM * LDS + tb * LDS;
        const float* wr = ws + cur * BN * LDS + (wn * 64 + tj) * LDS;
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
                if (NORMALISED) {
                    // 16 normalised magnitudes at a time: one warp vote decides whether any of them
                    // can matter, and the special-function chains of the 16 stay independent
                    float a0[8], a1[8], big = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        a0[j] = fabsf(xf[i].x - wf[j].x) * rm[i][j];
                        a1[j] = fabsf(xf[i].y - wf[j].y) * rm[i][j];
                        big = fmaxf(big, fmaxf(a0[j], a1[j]));
                    }
                    // (|t|/M)^p < 2^-40 for every element and lane: nothing to add (the sum is >= 1)
                    if (use_skip && __all_sync(0xffffffffu, big < skip_below)) continue;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        acc[i][j] += pow_abs<IP>(a0[j], p.p);
                        acc[i][j] += pow_abs<IP>(a1[j], p.p);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        acc[i][j] += pow_abs<IP>(xf[i].x - wf[j].x, p.p);
                        acc[i][j] += pow_abs<IP>(xf[i].y - wf[j].y, p.p);
                    }
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
            float* dst = p.y + (size_t)m * p.CO + n;
            if (!p.direct) {
                atomicAdd(dst, acc[i][j]);
                continue;
            }
            float r;
            if (NORMALISED) r = pow_pos(acc[i][j], rp) / rm[i][j];
            else r = pow_pos(fmaxf(acc[i][j], FLT_MIN), rp);
            *dst = r;
        }
    }
    u += kt_end - kt_begin;
  }
}

// Sums -> distances after a shared-tile forward: y = M * S^(1/p) or max(S, FLT_MIN)^(1/p).
__global__ void lp_finish_kernel(float* __restrict__ y, const float* __restrict__ m, long long n, float rp) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float sum = y[i];
        y[i] = m ? pow_pos(sum, rp) * m[i] : pow_pos(fmaxf(sum, FLT_MIN), rp);
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

// Work unit: one 32-row sub-batch x NT compact input columns x one tile of 32 outputs j.  The units
// of the whole problem form one sequence (sub-batch, column tile, j tile) that is cut into
// gridDim.x equal ranges, so every CTA does the same amount of work whatever the shape; a range
// that covers all j tiles of a (sub-batch, column tile) pair stores its grad_x block, a partial one
// adds it with atomics into the zero-filled grad_x.  Thread (tb, tc): rows tb*8 .. tb*8+7,
// columns 4*tc .. 4*tc+3; the four tb lanes that share tc sit in one warp (lane = (tc % 8) * 4 +
// tb), so the per-(j, c) sums over the 32 rows finish with two shuffles and one global reduction.
// The gathered W tile [32 j][NT c] and the (g, y) tile of the next j tile are fetched with
// cp.async while the current one is consumed.
constexpr int LPB_JT = 32;
// floats per row of the (g, 1/y) tiles [j][row]: 16-byte aligned rows, so that a thread's eight rows
// are two vector loads (all lanes of a warp that share tb read the same words: broadcast)
constexpr int LPB_GLD = 36;

// FINE (general exponent only): the two warp votes per 16-term batch ("all terms negligible",
// "some ratio near 1 -> accurate log2 series").  They pay from p - 1 >= 40: below that no term is
// negligible and the hardware log2's absolute error of 2^-22, multiplied by p - 1, stays under
// 7e-6 of a term; without the votes nothing separates the batches and the compiler overlaps
// their log2 / exp2 chains.
template <int IP, int NT, bool FINE>
__global__ void __launch_bounds__(NT, IP < 0 ? 4 : 3) lp_bwd_kernel(const LpBwdParams p) {
    constexpr int LPB_WLD = NT + 4;  // floats per W-tile row (+4: keeps 16-byte alignment, shifts banks)
    extern __shared__ __align__(16) float smem[];
    float* wt = smem;                                   // [2][JT][WLD]
    float* gt = smem + 2 * LPB_JT * LPB_WLD;            // [2][JT][GLD]  g
    float* yt = gt + 2 * LPB_JT * LPB_GLD;                   // [2][JT][GLD]  y, turned into 1/y in place
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tb = lane & 3, tc = warp * 8 + (lane >> 2);
    const int ntiles = (p.CO + LPB_JT - 1) / LPB_JT;
    const int col_tiles = (p.CI + NT - 1) / NT;
    const long long total = (long long)((p.B + SNB_SUB_BATCH - 1) / SNB_SUB_BATCH) * col_tiles * ntiles;
    long long u = total * blockIdx.x / gridDim.x;
    const long long u_end = total * (blockIdx.x + 1) / gridDim.x;
    // |u|^(p-1) < 2^-40 for a whole warp: the terms are dropped (the largest terms are ~1)
    const bool use_skip = p.pm1 >= 48.0f;
    const float skip_below = IP < 0 ? exp2f(-40.0f / fmaxf(p.pm1, 1e-3f)) : 0.f;

  while (u < u_end) {
    const int unit = (int)(u / ntiles), t_begin = (int)(u % ntiles);
    const int t_end = (int)min((long long)ntiles, t_begin + (u_end - u));
    const int s = unit / col_tiles, b0 = s * SNB_SUB_BATCH;
    const int c0 = (unit % col_tiles) * NT + tc * 4;
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

    const int mycol = tb == 0 ? col[0] : tb == 1 ? col[1] : tb == 2 ? col[2] : col[3];
    // this thread stages rows jj = tb, tb + 4, ... of the W tile (its own four columns) and
    // elements e = tid, tid + NT, ... of the 32 x 32 (g, y) tiles
    auto stage = [&](int t, int st) {
        const int j0 = t * LPB_JT;
#pragma unroll
        for (int r = 0; r < 8; r++) {
            const int jj = tb + 4 * r, j = j0 + jj;
            const bool jok = j < p.CO;
            const int row = jok ? (co_s ? co_s[j] : j) : 0;
            const float* wrow = p.w + (size_t)row * p.W_CI;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const bool ok = jok && col[k] >= 0;
                cp_async4(smem_u32(wt + (st * LPB_JT + jj) * LPB_WLD + tc * 4 + k), ok ? wrow + col[k] : p.w, ok ? 4 : 0);
            }
        }
#pragma unroll
        for (int r = 0; r < 1024 / NT; r++) {
            const int e = tid + NT * r;
            const int jj = e & 31, bb = e >> 5;  // consecutive threads -> consecutive j (coalesced)
            const int b = b0 + bb, j = j0 + jj;
            const bool ok = b < p.B && j < p.CO;
            const size_t o = ok ? (size_t)b * p.CO + j : 0;
            cp_async4(smem_u32(gt + (st * LPB_JT + jj) * LPB_GLD + bb), p.g + o, ok ? 4 : 0);
            cp_async4(smem_u32(yt + (st * LPB_JT + jj) * LPB_GLD + bb), p.y + o, ok ? 4 : 0);
        }
    };

    __syncthreads();                           // everyone is done with the previous range's tiles
    stage(t_begin, 0);
    cp_async_commit();
    for (int t = t_begin; t < t_end; t++) {
        const int st = (t - t_begin) & 1;
        cp_async_wait<0>();
        __syncthreads();                       // tile t landed; everyone is done with tile t - 1
        if (t + 1 < t_end) stage(t + 1, st ^ 1);
        cp_async_commit();
#pragma unroll
        for (int r = 0; r < 1024 / NT; r++) {  // y -> 1/y (0 for padding), each thread its own elements
            const int e = tid + NT * r;
            const int o = (st * LPB_JT + (e & 31)) * LPB_GLD + (e >> 5);
            const float v = yt[o];
            const float ry = v > 0.f ? 1.0f / v : 0.f;
            yt[o] = ry;
            // integer exponents: g * (|t| / y)^IP = (g / y^IP) * |t|^IP, so the division by y is
            // folded into g once per (row, output) instead of once per term
            if (IP >= 0) gt[o] *= pow_abs<IP>(ry, 0.f);
            // large general exponents: 1 / y = ry * (1 + e) with e = 1 - y * ry known exactly (one
            // fma); (1 + e)^(p-1) = 1 + (p-1) e to first order goes into g, so that the rounding of
            // the reciprocal is not amplified by the exponent in every term
            if (IP < 0 && FINE) gt[o] = fmaf(gt[o], p.pm1 * fmaf(-v, ry, 1.0f), gt[o]);
        }
        __syncthreads();
        const int j0 = t * LPB_JT;
        const int jn = min(LPB_JT, p.CO - j0);
        for (int jj = 0; jj < jn; jj++) {
            const float4 wv4 = *reinterpret_cast<const float4*>(wt + (st * LPB_JT + jj) * LPB_WLD + tc * 4);
            const float wv[4] = {wv4.x, wv4.y, wv4.z, wv4.w};
            float gwp[4] = {0.f, 0.f, 0.f, 0.f};
            float gp[8], yp[8];
            {
                const float4* g4 = reinterpret_cast<const float4*>(gt + (st * LPB_JT + jj) * LPB_GLD + tb * 8);
                const float4* y4 = reinterpret_cast<const float4*>(yt + (st * LPB_JT + jj) * LPB_GLD + tb * 8);
                const float4 ga = g4[0], gb = g4[1];
                gp[0] = ga.x; gp[1] = ga.y; gp[2] = ga.z; gp[3] = ga.w;
                gp[4] = gb.x; gp[5] = gb.y; gp[6] = gb.z; gp[7] = gb.w;
                if (IP < 0) {
                    const float4 ya = y4[0], yb = y4[1];
                    yp[0] = ya.x; yp[1] = ya.y; yp[2] = ya.z; yp[3] = ya.w;
                    yp[4] = yb.x; yp[5] = yb.y; yp[6] = yb.z; yp[7] = yb.w;
                }
            }
            if (IP >= 0) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float gv = gp[i];   // already divided by y^IP
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const float ps = pow_signed<IP>(xv[i][k] - wv[k], p.pm1);
                        gx[i][k] = fmaf(gv, ps, gx[i][k]);
                        gwp[k] = fmaf(gv, ps, gwp[k]);
                    }
                }
            } else {
                // general exponent: 16 terms at a time so that their log2 / exp2 chains overlap;
                // one vote per batch for "all negligible" and one for "some ratio is near 1".
                // |t| <= max_c |t| <= y, so a ratio is near 1 exactly when it is >= 0.875 and the
                // largest ratio of the batch answers both questions.
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    float u[4][4], lg[4][4], big = 0.f;
#pragma unroll
                    for (int ii = 0; ii < 4; ii++) {
                        const float ry = yp[4 * h + ii];
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            u[ii][k] = (xv[4 * h + ii][k] - wv[k]) * ry;
                            lg[ii][k] = lg2_approx(fabsf(u[ii][k]));
                        }
                        if (FINE) {
#pragma unroll
                            for (int k = 0; k < 4; k += 2) big = max3abs(big, u[ii][k], u[ii][k + 1]);
                        }
                    }
                    if (FINE && use_skip && __all_sync(0xffffffffu, big < skip_below)) continue;
                    if (FINE && __any_sync(0xffffffffu, big >= 0.875f)) {
#pragma unroll
                        for (int ii = 0; ii < 4; ii++)
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                const float a = fabsf(u[ii][k]);
                                if (near_one(a)) {
                                    // the product t * ry was rounded: its exact remainder (one fma),
                                    // relative to the ratio (1 / a = 2 - a near 1), corrects the logarithm,
                                    // which the exponent would otherwise amplify by p - 1
                                    const float ry = yp[4 * h + ii];
                                    const float rem = fmaf(xv[4 * h + ii][k] - wv[k], ry, -u[ii][k]);
                                    const float corr = copysignf(rem, rem * u[ii][k]) * (2.0f - a);
                                    lg[ii][k] = fmaf(corr, 1.4426950408889634f, log2_series(a));
                                }
                            }
                    }
#pragma unroll
                    for (int ii = 0; ii < 4; ii++) {
                        const float gv = gp[4 * h + ii];
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const float ps = copysignf(ex2_approx(p.pm1 * lg[ii][k]), u[ii][k]);
                            gx[4 * h + ii][k] = fmaf(gv, ps, gx[4 * h + ii][k]);
                            gwp[k] = fmaf(gv, ps, gwp[k]);
                        }
                    }
                }
            }
            if (p.gw) {
                // Sum over the four lanes (tb = 0..3) that hold the same four columns, ending with
                // column tb on lane tb: each lane passes on the half it does not keep (3 shuffles
                // instead of 8).  The warp then issues ONE reduction instruction per output row
                // covering 32 neighbouring kept columns (4-5 sectors).
                {
                    const bool hi2 = tb & 2, hi1 = tb & 1;
                    const float a0 = (hi2 ? gwp[2] : gwp[0]) + __shfl_xor_sync(0xffffffffu, hi2 ? gwp[0] : gwp[2], 2);
                    const float a1 = (hi2 ? gwp[3] : gwp[1]) + __shfl_xor_sync(0xffffffffu, hi2 ? gwp[1] : gwp[3], 2);
                    const float v = (hi1 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, hi1 ? a0 : a1, 1);
                    const int row = co_s ? co_s[j0 + jj] : j0 + jj;
                    if (mycol >= 0) atomicAdd(p.gw + (size_t)row * p.W_CI + mycol, -v);
                }
            }
        }
    }
    const bool whole = t_begin == 0 && t_end == ntiles;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int b = b0 + tb * 8 + i;
        if (b >= p.B) continue;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            if (col[k] < 0) continue;
            float* dst = p.gx + (size_t)b * p.CI + c0 + k;
            if (whole) *dst = gx[i][k];
            else atomicAdd(dst, gx[i][k]);
        }
    }
    u += t_end - t_begin;
  }
}

// One CTA per resident slot (SMs x CTAs per SM by the occupancy calculator), each with an equal
// share of the work units; grad_x is zero-filled first because partial ranges add into it.
template <int IP, bool FINE = true>
static cudaError_t launch_lp_bwd(const LpBwdParams& q, cudaStream_t st) {
    constexpr int NT = 128;
    constexpr int SMEM = (2 * LPB_JT * (NT + 4) + 2 * 2 * LPB_JT * LPB_GLD) * (int)sizeof(float);
    static std::atomic<int> cached[64];
    int dev = 0;
    cudaGetDevice(&dev);
    std::atomic<int>& slot = cached[dev & 63];
    int cps = slot.load(std::memory_order_acquire);
    auto kern = lp_bwd_kernel<IP, NT, FINE>;
    if (cps == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        int occ = 0;
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, NT, SMEM);
        if (e != cudaSuccess) return e;
        cps = occ > 0 ? occ : 1;
        slot.store(cps, std::memory_order_release);
    }
    const long long total = (long long)((q.B + 31) / 32) * ((q.CI + NT - 1) / NT) * ((q.CO + LPB_JT - 1) / LPB_JT);
    const long long slots = (long long)sm_count() * cps;
    cudaError_t e = cudaMemsetAsync(q.gx, 0, sizeof(float) * (size_t)q.B * q.CI, st);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(total < slots ? total : slots), NT, SMEM, st>>>(q);
    return cudaGetLastError();
}

// p.m == nullptr with NORM: the maxima are in y and no scratch is available -> one CTA per tile,
// finished in the kernel.  Otherwise equal (tile, k-tile) ranges over all resident CTA slots.
template <int WN, int MODE, int IP, bool NORM>
static cudaError_t launch_lp_fwd(LpFwdParams p, cudaStream_t st) {
    constexpr int BN = 64 * WN;
    constexpr int SMEM = 2 * (32 + BN) * LDS * (int)sizeof(float);
    auto kern = lp_fwd_kernel<WN, MODE, IP, NORM>;
    static std::atomic<int> cached[64];
    int dev = 0;
    cudaGetDevice(&dev);
    std::atomic<int>& slot = cached[dev & 63];
    int cps = slot.load(std::memory_order_acquire);
    if (cps == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        int occ = 0;
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, WN * 32, SMEM);
        if (e != cudaSuccess) return e;
        cps = occ > 0 ? occ : 1;
        slot.store(cps, std::memory_order_release);
    }
    const long long tiles = (long long)((p.B + 31) / 32) * ((p.CO + BN - 1) / BN);
    const long long slots = (long long)sm_count() * cps;
    const bool no_scratch = NORM && p.m == nullptr;
    // whole tiles per CTA when they fill the slots evenly anyway, or when there is nowhere to keep M
    p.direct = (no_scratch || tiles % slots == 0) ? 1 : 0;
    if (NORM && p.m == nullptr) p.m = p.y;
    if (p.direct) {
        kern<<<(unsigned)tiles, WN * 32, SMEM, st>>>(p);
        return cudaGetLastError();
    }
    const size_t n = (size_t)p.B * p.CO;
    cudaError_t e = cudaMemsetAsync(p.y, 0, sizeof(float) * n, st);
    if (e != cudaSuccess) return e;
    const long long units = tiles * ((p.CI + BK - 1) / BK);
    kern<<<(unsigned)(units < slots ? units : slots), WN * 32, SMEM, st>>>(p);
    lp_finish_kernel<<<sm_count() * 4, 256, 0, st>>>(p.y, NORM ? p.m : nullptr, (long long)n, 1.0f / p.p);
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

static int lp_forward_impl(const float* x, const float* w, int B, int CO, int CI, int G, int HW, float* y,
                           float p, const int* w_index_ci, const int* w_index_co, int W_CO, int W_CI,
                           float* scratch, cudaStream_t st) {
    if (!(p > 0) || isinf(p)) return SNB_ERR_UNSUPPORTED;
    if (G != 1 || HW != 1)
        return general_lp_forward(x, w, B, CO, CI, G, HW, y, p, w_index_ci, w_index_co, W_CO, W_CI, st);
    if (!x || !w || !y) return SNB_ERR_NULL_POINTER;
    if (B <= 0 || CO <= 0 || CI <= 0 || W_CO <= 0 || W_CI <= 0) return SNB_ERR_BAD_SHAPE;
    if ((!w_index_ci && W_CI != CI) || (!w_index_co && W_CO != CO) || CI > W_CI || CO > W_CO)
        return SNB_ERR_BAD_SHAPE;
    if ((long long)W_CO * W_CI >= (1ll << 31) || (long long)B * CO >= (1ll << 31) || (long long)B * CI >= (1ll << 31))
        return SNB_ERR_TOO_LARGE;
    LpFwdParams q{x, w, y, nullptr, w_index_ci, w_index_co, B, CO, CI, W_CI, p, 0};
    if (p > 10.0f) {
        // the maxima go to the scratch array when there is one (y is then free to collect partial
        // sums from CTAs that share a tile), else into y itself
        float* maxima = scratch ? scratch : y;
        SNB_CUDA(inf_forward_values(x, w, maxima, w_index_ci, w_index_co, B, CO, CI, W_CI, st));
        q.m = scratch;
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

extern "C" int snb_norm_dist_forward(const float* x, const float* w, int B, int CO, int CI, int G,
                                     int HW, float* y, float p, const int* w_index_ci,
                                     const int* w_index_co, int W_CO, int W_CI, void* stream) {
    return lp_forward_impl(x, w, B, CO, CI, G, HW, y, p, w_index_ci, w_index_co, W_CO, W_CI, nullptr,
                           (cudaStream_t)stream);
}

extern "C" size_t snb_norm_dist_forward_workspace_bytes(int B, int CO, float p) {
    return (B > 0 && CO > 0 && p > 10.0f) ? sizeof(float) * (size_t)B * (size_t)CO : 0;
}

extern "C" int snb_norm_dist_forward_ws(const float* x, const float* w, int B, int CO, int CI, int G,
                                        int HW, float* y, float p, const int* w_index_ci,
                                        const int* w_index_co, int W_CO, int W_CI, void* workspace,
                                        size_t workspace_bytes, void* stream) {
    float* scratch = nullptr;
    if (workspace && p > 10.0f) {
        if (reinterpret_cast<uintptr_t>(workspace) & 15u) return SNB_ERR_ALIGNMENT;
        if (workspace_bytes >= snb_norm_dist_forward_workspace_bytes(B, CO, p)) scratch = (float*)workspace;
    }
    return lp_forward_impl(x, w, B, CO, CI, G, HW, y, p, w_index_ci, w_index_co, W_CO, W_CI, scratch,
                           (cudaStream_t)stream);
}

static int lp_backward(const float* g, const float* x, const float* w, const float* y, int B, int CO,
                       int CI, int G, int HW, float* gx, float* gw, float p, const int* ci,
                       const int* co, int W_CO, int W_CI, cudaStream_t st) {
    if (!(p > 0) || isinf(p)) return SNB_ERR_UNSUPPORTED;
    if (G != 1 || HW != 1)
        return general_lp_backward(g, x, w, y, B, CO, CI, G, HW, gx, gw, p, ci, co, W_CO, W_CI, st);
    if (!g || !x || !w || !y || !gx) return SNB_ERR_NULL_POINTER;
    if (B <= 0 || CO <= 0 || CI <= 0 || W_CO <= 0 || W_CI <= 0) return SNB_ERR_BAD_SHAPE;
    if ((!ci && W_CI != CI) || (!co && W_CO != CO) || CI > W_CI || CO > W_CO) return SNB_ERR_BAD_SHAPE;
    if ((long long)W_CO * W_CI >= (1ll << 31) || (long long)B * CO >= (1ll << 31) || (long long)B * CI >= (1ll << 31))
        return SNB_ERR_TOO_LARGE;
    if (gw) SNB_CUDA(cudaMemsetAsync(gw, 0, sizeof(float) * (size_t)W_CO * W_CI, st));
    LpBwdParams q{g, x, w, y, gx, gw, ci, co, B, CO, CI, W_CI, p - 1.0f};
    switch (integer_power(p - 1.0f)) {
        case 0: SNB_CUDA(launch_lp_bwd<0>(q, st)); break;
        case 1: SNB_CUDA(launch_lp_bwd<1>(q, st)); break;
        case 2: SNB_CUDA(launch_lp_bwd<2>(q, st)); break;
        case 3: SNB_CUDA(launch_lp_bwd<3>(q, st)); break;
        case 4: SNB_CUDA(launch_lp_bwd<4>(q, st)); break;
        case 5: SNB_CUDA(launch_lp_bwd<5>(q, st)); break;
        case 6: SNB_CUDA(launch_lp_bwd<6>(q, st)); break;
        case 7: SNB_CUDA(launch_lp_bwd<7>(q, st)); break;
        default:
            if (p - 1.0f >= 40.0f) SNB_CUDA((launch_lp_bwd<-1, true>(q, st)));
            else SNB_CUDA((launch_lp_bwd<-1, false>(q, st)));
            break;
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
