// Interval-bound (IBP) propagation through an l-infinity distance layer.
//
// Replaces zbh2047/SortNet core/cuda/bound_inf_dist_cuda.cu (kernels :15-118, :121-238,
// :240-299; launchers :314-383).  For x in the box [xL, xU] (xL > xU is repaired to the
// midpoint, :63):
//     t1 = w - xL, t2 = xU - w
//     yL = -min(-1e-10, min_c min(t1, t2)),   yU = max(1e-10, max_c max(t1, t2))
// bit for bit.  The word variant records the first c (strict comparisons, ascending c) that
// set each bound, bit 31 = (t1 > t2); posL = 0xffffffff when the lower bound never left
// its floor.
#include <stdlib.h>
#include "tile.cuh"
#include "launch.h"
#include "general_shapes.h"

namespace snb {

// bound_tma.cu: TMA-staged kernel for large aligned problems; cudaErrorNotSupported = not applicable
cudaError_t bound_forward_tma(const float* xl, const float* xu, const float* w, float* yl, float* yu, int B, int CO,
                              int CI, cudaStream_t st);

struct BoundParams {
    const float* xl;
    const float* xu;
    const float* w;
    float* yl;
    float* yu;
    int* posl;
    int* posu;
    int B, CO, CI;
    int tiles_m, tiles_n;
    int split;  // 1: some tiles are shared between CTAs -> merge with atomics into zeroed outputs
};

// ---- bounds only: 8x8 outputs x 2 accumulators per thread, stream-K over (tile, k) -------
template <int WM, int WN, bool VEC>
__global__ void __launch_bounds__(WM* WN * 32) bound_fwd_kernel(const BoundParams p) {
    constexpr int BM = 32 * WM, BN = 64 * WN, NT = WM * WN * 32;
    extern __shared__ __align__(16) float smem[];
    float* ls = smem;                      // [2][BM][LDS]
    float* us = ls + 2 * BM * LDS;         // [2][BM][LDS]
    float* ws = us + 2 * BM * LDS;         // [2][BN][LDS]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp / WN, wn = warp % WN, tb = lane >> 3, tj = lane & 7;

    StreamK sk{p.tiles_m, p.tiles_n, (p.CI + BK - 1) / BK};
    long long u0, u1;
    sk.range(u0, u1);

    while (u0 < u1) {
        const int tile = (int)(u0 / sk.nk);
        const int ka = (int)(u0 % sk.nk);
        const int kb = (int)min((long long)sk.nk, ka + (u1 - u0));
        const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;

        auto stage = [&](int kt, int st) {
            float* ld = ls + st * BM * LDS;
            float* ud = us + st * BM * LDS;
            float* wd = ws + st * BN * LDS;
            if (VEC) {
                stage_dense_vec<BM, NT>(ld, p.xl, m0, p.B, p.CI, kt * BK, p.CI, tid);
                stage_dense_vec<BM, NT>(ud, p.xu, m0, p.B, p.CI, kt * BK, p.CI, tid);
                stage_dense_vec<BN, NT>(wd, p.w, n0, p.CO, p.CI, kt * BK, p.CI, tid);
            } else {
                stage_dense_scalar<BM, NT>(ld, p.xl, m0, p.B, p.CI, kt * BK, p.CI, tid);
                stage_dense_scalar<BM, NT>(ud, p.xu, m0, p.B, p.CI, kt * BK, p.CI, tid);
                stage_dense_scalar<BN, NT>(wd, p.w, n0, p.CO, p.CI, kt * BK, p.CI, tid);
            }
        };

        float accl[8][8], accu[8][8];
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) {
                accl[i][j] = -SNB_EPS;
                accu[i][j] = SNB_EPS;
            }

        __syncthreads();  // previous tile's readers are done with both stages
        stage(ka, ka & 1);
        cp_async_commit();
        for (int kt = ka; kt < kb; kt++) {
            cp_async_wait<0>();
            __syncthreads();
            if (kt + 1 < kb) stage(kt + 1, (kt + 1) & 1);
            cp_async_commit();
            // midpoint repair of inverted intervals, in place, before anyone reads the tile
            {
                float* ld = ls + (kt & 1) * BM * LDS;
                float* ud = us + (kt & 1) * BM * LDS;
#pragma unroll
                for (int r = 0; r < BM * BK / NT; r++) {
                    const int e = tid + r * NT;
                    const int o = (e >> 5) * LDS + (e & 31);
                    const float a = ld[o], b = ud[o];
                    if (a > b) {
                        const float m = (a + b) * 0.5f;
                        ld[o] = m;
                        ud[o] = m;
                    }
                }
            }
            __syncthreads();
            const float* lr = ls + (kt & 1) * BM * LDS + (wm * 32 + tb) * LDS;
            const float* ur = us + (kt & 1) * BM * LDS + (wm * 32 + tb) * LDS;
            const float* wr = ws + (kt & 1) * BN * LDS + (wn * 64 + tj) * LDS;
#pragma unroll 4
            for (int kk = 0; kk < BK / 2; kk++) {
                float2 lf[8], uf[8], wf[8];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    lf[i] = *reinterpret_cast<const float2*>(lr + i * 4 * LDS + kk * 2);
                    uf[i] = *reinterpret_cast<const float2*>(ur + i * 4 * LDS + kk * 2);
                }
#pragma unroll
                for (int j = 0; j < 8; j++) wf[j] = *reinterpret_cast<const float2*>(wr + j * 8 * LDS + kk * 2);
#pragma unroll
                for (int i = 0; i < 8; i++) {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        float t1 = wf[j].x - lf[i].x, t2 = uf[i].x - wf[j].x;
                        accl[i][j] = min3(accl[i][j], t1, t2);
                        accu[i][j] = max3(accu[i][j], t1, t2);
                        t1 = wf[j].y - lf[i].y;
                        t2 = uf[i].y - wf[j].y;
                        accl[i][j] = min3(accl[i][j], t1, t2);
                        accu[i][j] = max3(accu[i][j], t1, t2);
                    }
                }
            }
        }
        const bool whole = (ka == 0 && kb == sk.nk);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int m = m0 + wm * 32 + tb + 4 * i;
            if (m >= p.B) continue;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int n = n0 + wn * 64 + tj + 8 * j;
                if (n >= p.CO) continue;
                const size_t o = (size_t)m * p.CO + n;
                if (whole) {
                    p.yl[o] = -accl[i][j];
                    p.yu[o] = accu[i][j];
                } else {
                    atomic_max_nonneg(p.yl + o, -accl[i][j]);
                    atomic_max_nonneg(p.yu + o, accu[i][j]);
                }
            }
        }
        u0 += kb - ka;
    }
}

// ---- bounds + argmin/argmax words: 4x4 outputs per thread, per-element strict updates ----
template <bool VEC>
__global__ void __launch_bounds__(256) bound_fwd_pos_kernel(const BoundParams p) {
    constexpr int BM = 64, BN = 64, NT = 256;
    extern __shared__ __align__(16) float smem[];
    float(*ls)[BM * LDS] = reinterpret_cast<float(*)[BM * LDS]>(smem);
    float(*us)[BM * LDS] = reinterpret_cast<float(*)[BM * LDS]>(smem + 2 * BM * LDS);
    float(*ws)[BN * LDS] = reinterpret_cast<float(*)[BN * LDS]>(smem + 4 * BM * LDS);
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int nk = (p.CI + BK - 1) / BK;

    auto stage = [&](int kt, int st) {
        if (VEC) {
            stage_dense_vec<BM, NT>(ls[st], p.xl, m0, p.B, p.CI, kt * BK, p.CI, tid);
            stage_dense_vec<BM, NT>(us[st], p.xu, m0, p.B, p.CI, kt * BK, p.CI, tid);
            stage_dense_vec<BN, NT>(ws[st], p.w, n0, p.CO, p.CI, kt * BK, p.CI, tid);
        } else {
            stage_dense_scalar<BM, NT>(ls[st], p.xl, m0, p.B, p.CI, kt * BK, p.CI, tid);
            stage_dense_scalar<BM, NT>(us[st], p.xu, m0, p.B, p.CI, kt * BK, p.CI, tid);
            stage_dense_scalar<BN, NT>(ws[st], p.w, n0, p.CO, p.CI, kt * BK, p.CI, tid);
        }
    };

    float accl[4][4], accu[4][4];
    uint32_t pl[4][4], pu[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            accl[i][j] = -SNB_EPS;
            accu[i][j] = SNB_EPS;
            pl[i][j] = SNB_NO_GRAD_ID;
            pu[i][j] = 0;
        }

    stage(0, 0);
    cp_async_commit();
    for (int kt = 0; kt < nk; kt++) {
        cp_async_wait<0>();
        __syncthreads();
        if (kt + 1 < nk) stage(kt + 1, (kt + 1) & 1);
        cp_async_commit();
        {
            float* ld = ls[kt & 1];
            float* ud = us[kt & 1];
#pragma unroll
            for (int r = 0; r < BM * BK / NT; r++) {
                const int e = tid + r * NT;
                const int o = (e >> 5) * LDS + (e & 31);
                const float a = ld[o], b = ud[o];
                if (a > b) {
                    const float m = (a + b) * 0.5f;
                    ld[o] = m;
                    ud[o] = m;
                }
            }
        }
        __syncthreads();
        const float* lr = ls[kt & 1] + ty * LDS;
        const float* ur = us[kt & 1] + ty * LDS;
        const float* wr = ws[kt & 1] + tx * LDS;
#pragma unroll 4
        for (int k = 0; k < BK; k++) {
            float lf[4], uf[4], wf[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                lf[i] = lr[i * 16 * LDS + k];
                uf[i] = ur[i * 16 * LDS + k];
                wf[i] = wr[i * 16 * LDS + k];
            }
            const uint32_t c = (uint32_t)(kt * BK + k);
#pragma unroll
            for (int i = 0; i < 4; i++) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float t1 = wf[j] - lf[i], t2 = uf[i] - wf[j];
                    const float lo = fminf(t1, t2), hi = fmaxf(t1, t2);
                    const uint32_t word = c | (t1 <= t2 ? 0u : SNB_SIGN_BIT);
                    if (lo < accl[i][j]) {
                        accl[i][j] = lo;
                        pl[i][j] = word;
                    }
                    if (hi > accu[i][j]) {
                        accu[i][j] = hi;
                        pu[i][j] = word;
                    }
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty + 16 * i;
        if (m >= p.B) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx + 16 * j;
            if (n >= p.CO) continue;
            const size_t o = (size_t)m * p.CO + n;
            p.yl[o] = -accl[i][j];
            p.yu[o] = accu[i][j];
            p.posl[o] = (int)pl[i][j];
            p.posu[o] = (int)pu[i][j];
        }
    }
}

// Sparse backward: one CTA per batch row, both grad_x rows accumulated in shared memory.
__global__ void __launch_bounds__(256) bound_bwd_kernel(const float* __restrict__ gl,
                                                        const float* __restrict__ gu,
                                                        const int* __restrict__ posl,
                                                        const int* __restrict__ posu, int CO, int CI,
                                                        float* __restrict__ gxl, float* __restrict__ gxu,
                                                        float* __restrict__ gw, int use_smem) {
    extern __shared__ float rows[];  // [2][CI] when use_smem
    const int b = blockIdx.x;
    float* rl = use_smem ? rows : gxl + (size_t)b * CI;
    float* ru = use_smem ? rows + CI : gxu + (size_t)b * CI;
    if (use_smem) {
        for (int c = threadIdx.x; c < 2 * CI; c += blockDim.x) rows[c] = 0.f;
        __syncthreads();
    }
    for (int j = threadIdx.x; j < CO; j += blockDim.x) {
        const size_t o = (size_t)b * CO + j;
        const uint32_t wl = (uint32_t)posl[o], wu = (uint32_t)posu[o];
        const float vl = (wl & SNB_SIGN_BIT) ? -gl[o] : gl[o];
        const float vu = (wu & SNB_SIGN_BIT) ? -gu[o] : gu[o];
        const int il = (int)(wl & ~SNB_SIGN_BIT), iu = (int)(wu & ~SNB_SIGN_BIT);
        if (wl != SNB_NO_GRAD_ID) {
            atomicAdd(((wl & SNB_SIGN_BIT) ? ru : rl) + il, vl);
            if (gw) atomicAdd(gw + (size_t)j * CI + il, -vl);
        }
        atomicAdd(((wu & SNB_SIGN_BIT) ? rl : ru) + iu, vu);
        if (gw) atomicAdd(gw + (size_t)j * CI + iu, -vu);
    }
    if (use_smem) {
        __syncthreads();
        for (int c = threadIdx.x; c < CI; c += blockDim.x) {
            gxl[(size_t)b * CI + c] = rows[c];
            gxu[(size_t)b * CI + c] = rows[CI + c];
        }
    }
}

template <int WM, int WN, bool VEC>
static cudaError_t launch_bound(BoundParams p, cudaStream_t st) {
    constexpr int BM = 32 * WM, BN = 64 * WN, NT = WM * WN * 32;
    constexpr int SMEM = 2 * (2 * BM + BN) * LDS * (int)sizeof(float);
    auto kern = bound_fwd_kernel<WM, WN, VEC>;
    static std::atomic<int> ctas_per_sm[64];
    int dev = 0;
    cudaGetDevice(&dev);
    std::atomic<int>& slot = ctas_per_sm[dev & 63];
    int cps = slot.load(std::memory_order_acquire);
    if (cps == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        int occ = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, NT, SMEM);
        if (e != cudaSuccess) return e;
        cps = occ > 0 ? occ : 1;
        slot.store(cps, std::memory_order_release);
    }
    p.tiles_m = (p.B + BM - 1) / BM;
    p.tiles_n = (p.CO + BN - 1) / BN;
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    const long long units = tiles * ((p.CI + BK - 1) / BK);
    long long grid = (long long)sm_count() * cps;
    // whole tiles when they balance anyway; a problem with fewer (tile, k-tile) pairs than resident
    // CTAs (few tiles, e.g. a narrow head layer) still spreads over one CTA per pair
    if (tiles % grid == 0) grid = tiles;
    else if (units < grid) grid = units;
    p.split = (grid != tiles);
    if (p.split) {
        cudaError_t e = cudaMemsetAsync(p.yl, 0, sizeof(float) * (size_t)p.B * p.CO, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(p.yu, 0, sizeof(float) * (size_t)p.B * p.CO, st);
        if (e != cudaSuccess) return e;
    }
    kern<<<(unsigned)grid, NT, SMEM, st>>>(p);
    return cudaGetLastError();
}

}  // namespace snb

using namespace snb;

// SNB_DISABLE_TMA=1 in the environment keeps the cp.async staging everywhere.
static bool tma_enabled() {
    static const bool enabled = [] {
        const char* e = getenv("SNB_DISABLE_TMA");
        return !(e && e[0] == '1');
    }();
    return enabled;
}

static int check_bound(const void* xl, const void* xu, const void* w, const void* yl, const void* yu,
                       int B, int CO, int CI, int G, int HW) {
    if (!xl || !xu || !w || !yl || !yu) return SNB_ERR_NULL_POINTER;
    if (G != 1 || HW != 1) return SNB_ERR_UNSUPPORTED;
    if (B <= 0 || CO <= 0 || CI <= 0) return SNB_ERR_BAD_SHAPE;
    if ((long long)CO * CI >= (1ll << 31) || (long long)B * CO >= (1ll << 31) || (long long)B * CI >= (1ll << 31))
        return SNB_ERR_TOO_LARGE;
    return SNB_OK;
}

extern "C" int snb_bound_inf_dist_forward_nograd(const float* xl, const float* xu, const float* w,
                                                 int B, int CO, int CI, int G, int HW, float* yl,
                                                 float* yu, void* stream) {
    if (G != 1 || HW != 1)
        return general_bound_forward(xl, xu, w, B, CO, CI, G, HW, yl, yu, nullptr, nullptr, (cudaStream_t)stream);
    int rc = check_bound(xl, xu, w, yl, yu, B, CO, CI, G, HW);
    if (rc) return rc;
    BoundParams p{xl, xu, w, yl, yu, nullptr, nullptr, B, CO, CI, 0, 0, 0};
    const bool vec = (CI % 4 == 0) && aligned16(xl) && aligned16(xu) && aligned16(w);
    cudaStream_t st = (cudaStream_t)stream;
    // Tile shape by measurement on B200 (5120 x 5120 layers, 32..1024 rows): 64 x 256 output tiles are
    // the fastest from 64 rows up (0.33 / 0.62 / 0.92 / 1.22 / 2.40 ms at 64 / 128 / 192 / 256 / 512 rows;
    // 128-row tiles waste the padding rows below 256 and are 1 % slower above), 32 x 256 for a single
    // sub-batch.  Narrow layers (a head with few outputs) keep tall tiles: the TMA-staged 128 x 128
    // kernel when the rows fill it, else 32 x 128.
    if (CO > 128) {
        if (B > 32) SNB_CUDA(vec ? launch_bound<2, 4, true>(p, st) : launch_bound<2, 4, false>(p, st));
        else SNB_CUDA(vec ? launch_bound<1, 4, true>(p, st) : launch_bound<1, 4, false>(p, st));
        return SNB_OK;
    }
    if (B >= 128 && tma_enabled()) {
        cudaError_t e = bound_forward_tma(xl, xu, w, yl, yu, B, CO, CI, st);
        if (e == cudaSuccess) return SNB_OK;
        if (e != cudaErrorNotSupported) SNB_CUDA(e);
    }
    if (B >= 128) {
        SNB_CUDA(vec ? launch_bound<4, 2, true>(p, st) : launch_bound<4, 2, false>(p, st));
    } else {
        SNB_CUDA(vec ? launch_bound<1, 2, true>(p, st) : launch_bound<1, 2, false>(p, st));
    }
    return SNB_OK;
}

extern "C" int snb_bound_inf_dist_forward(const float* xl, const float* xu, const float* w, int B,
                                          int CO, int CI, int G, int HW, float* yl, float* yu,
                                          int* posl, int* posu, void* stream) {
    if (G != 1 || HW != 1) {
        if (!posl || !posu) return SNB_ERR_NULL_POINTER;
        return general_bound_forward(xl, xu, w, B, CO, CI, G, HW, yl, yu, posl, posu, (cudaStream_t)stream);
    }
    int rc = check_bound(xl, xu, w, yl, yu, B, CO, CI, G, HW);
    if (rc) return rc;
    if (!posl || !posu) return SNB_ERR_NULL_POINTER;
    BoundParams p{xl, xu, w, yl, yu, posl, posu, B, CO, CI, 0, 0, 0};
    const bool vec = (CI % 4 == 0) && aligned16(xl) && aligned16(xu) && aligned16(w);
    dim3 grid((B + 63) / 64, (CO + 63) / 64);
    constexpr int SMEM = 2 * 3 * 64 * LDS * (int)sizeof(float);
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        SNB_CUDA(cudaFuncSetAttribute(bound_fwd_pos_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        SNB_CUDA(cudaFuncSetAttribute(bound_fwd_pos_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        configured[dev & 63].store(true, std::memory_order_release);
    }
    if (vec) bound_fwd_pos_kernel<true><<<grid, 256, SMEM, (cudaStream_t)stream>>>(p);
    else bound_fwd_pos_kernel<false><<<grid, 256, SMEM, (cudaStream_t)stream>>>(p);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

static int bound_backward(const float* gl, const float* gu, const int* posl, const int* posu, int B,
                          int CO, int CI, int G, int HW, float* gxl, float* gxu, float* gw,
                          cudaStream_t st) {
    if (G != 1 || HW != 1)
        return general_bound_backward(gl, gu, posl, posu, B, CO, CI, G, HW, gxl, gxu, gw, st);
    if (!gl || !gu || !posl || !posu || !gxl || !gxu) return SNB_ERR_NULL_POINTER;
    if (B <= 0 || CO <= 0 || CI <= 0) return SNB_ERR_BAD_SHAPE;
    if ((long long)CO * CI >= (1ll << 31)) return SNB_ERR_TOO_LARGE;
    if (gw) SNB_CUDA(cudaMemsetAsync(gw, 0, sizeof(float) * (size_t)CO * CI, st));
    const int use_smem = (size_t)2 * CI * sizeof(float) <= 48 * 1024;
    if (!use_smem) {
        SNB_CUDA(cudaMemsetAsync(gxl, 0, sizeof(float) * (size_t)B * CI, st));
        SNB_CUDA(cudaMemsetAsync(gxu, 0, sizeof(float) * (size_t)B * CI, st));
    }
    bound_bwd_kernel<<<B, 256, use_smem ? 2 * CI * sizeof(float) : 0, st>>>(gl, gu, posl, posu, CO, CI,
                                                                         gxl, gxu, gw, use_smem);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

extern "C" int snb_bound_inf_dist_backward_input(const float* grad_yl, const float* grad_yu,
                                                 const int* posl, const int* posu, int B, int CO,
                                                 int CI, int G, int HW, float* grad_xl,
                                                 float* grad_xu, void* stream) {
    return bound_backward(grad_yl, grad_yu, posl, posu, B, CO, CI, G, HW, grad_xl, grad_xu, nullptr,
                          (cudaStream_t)stream);
}

extern "C" int snb_bound_inf_dist_backward_input_weight(const float* grad_yl, const float* grad_yu,
                                                        const int* posl, const int* posu, int B,
                                                        int CO, int CI, int G, int HW, float* grad_xl,
                                                        float* grad_xu, float* grad_w, void* stream) {
    if (!grad_w) return SNB_ERR_NULL_POINTER;
    return bound_backward(grad_yl, grad_yu, posl, posu, B, CO, CI, G, HW, grad_xl, grad_xu, grad_w,
                          (cudaStream_t)stream);
}
