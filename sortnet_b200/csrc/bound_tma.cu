// Interval-bound forward, TMA-staged variant for large 16-byte-aligned problems.
//
// Same arithmetic and the same stream-K work split as bound_fwd_kernel (bound_inf_dist.cu), which
// replaces zbh2047/SortNet core/cuda/bound_inf_dist_cuda.cu:15-118,314-328.  What differs is the
// staging: one elected thread per CTA issues three cp.async.bulk.tensor.2d copies per k-tile
// (the x_L, x_U and W tiles, 128 rows x 32 fp32 = 16 KiB each) that complete on an mbarrier; the
// tiles land in the 128-byte-swizzled layout, so rows are 128 bytes apart (no padding) and the
// 16-byte fragment reads of a quarter-warp still hit distinct banks; four stages are in flight.
// Rows or columns past the end of a tensor are zero-filled by the copy unit, which is what the
// arithmetic expects (t1 = t2 = 0 never moves an accumulator off its floor).
//
// Every wait on an mbarrier is bounded: if a phase has not completed after SNB_TMA_WAIT_CYCLES SM
// clocks (about 0.2 s) the thread raises a device-side error flag and the whole CTA leaves the
// kernel at its next barrier (the output is then meaningless, but the kernel ends and the
// context stays usable); snb_device_wait_failed() reports the flag to the host.
#include <cuda.h>
#include "tile.cuh"
#include "launch.h"

#define SNB_TMA_WAIT_CYCLES 400000000ll

namespace snb {

static __device__ int snb_tma_wait_failed = 0;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; returns false (and raises the error flag) if the phase never completed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (clock64() - t0 < SNB_TMA_WAIT_CYCLES)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(&snb_tma_wait_failed, 1);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

constexpr int TMA_TN = 8;                                         // output columns per thread
constexpr int TMA_BM = 128, TMA_BN = 128, TMA_NT = 256 * 8 / TMA_TN, TMA_STAGES = 4;
constexpr int TMA_TILE_FLOATS = 128 * BK;                         // 16 KiB
constexpr int TMA_STAGE_FLOATS = 3 * TMA_TILE_FLOATS;             // x_L, x_U, W
constexpr int TMA_SMEM = TMA_STAGES * TMA_STAGE_FLOATS * 4 + 1024 /*alignment slack*/ + 64 /*barriers*/;

struct BoundTmaParams {
    float* yl;
    float* yu;
    int B, CO, CI;
    int tiles_m, tiles_n;
};

// Offset (in floats) of the 16-byte chunk `chunk` (0..7) of row r inside a 128-byte-swizzled tile.
__device__ __forceinline__ int swz(int r, int chunk) { return r * BK + ((chunk ^ (r & 7)) << 2); }

__global__ void __launch_bounds__(TMA_NT) bound_fwd_tma_kernel(const __grid_constant__ CUtensorMap map_l,
                                                               const __grid_constant__ CUtensorMap map_u,
                                                               const __grid_constant__ CUtensorMap map_w,
                                                               const BoundTmaParams p) {
    extern __shared__ uint8_t raw[];
    // 1024-byte aligned tile storage (the swizzle pattern is a function of the address bits)
    float* tiles = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + TMA_STAGES * TMA_STAGE_FLOATS);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int WN = TMA_BN / (8 * TMA_TN);   // warps along the columns
    const int wm = warp / WN, wn = warp % WN, tb = lane >> 3, tj = lane & 7;

    __shared__ int abort_flag;
    if (tid == 0) {
        abort_flag = 0;
#pragma unroll
        for (int s = 0; s < TMA_STAGES; s++) mbar_init(smem_u32(bars + s), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    StreamK sk{p.tiles_m, p.tiles_n, (p.CI + BK - 1) / BK};
    long long u0, u1;
    sk.range(u0, u1);
    uint32_t it = 0;       // k-tiles consumed so far by this CTA: stage = it % STAGES, parity = (it / STAGES) & 1
    uint32_t issued = 0;   // k-tiles whose copies have been issued (thread 0)

    while (u0 < u1) {
        const int tile = (int)(u0 / sk.nk);
        const int ka = (int)(u0 % sk.nk);
        const int kb = (int)min((long long)sk.nk, ka + (u1 - u0));
        const int m0 = (tile % p.tiles_m) * TMA_BM, n0 = (tile / p.tiles_m) * TMA_BN;

        auto issue = [&](int kt) {   // thread 0 only
            const uint32_t st = issued % TMA_STAGES;
            const uint32_t bar = smem_u32(bars + st);
            float* base = tiles + st * TMA_STAGE_FLOATS;
            mbar_expect_tx(bar, 3u * TMA_TILE_FLOATS * 4u);
            tma_load_2d(smem_u32(base), &map_l, kt * BK, m0, bar);
            tma_load_2d(smem_u32(base + TMA_TILE_FLOATS), &map_u, kt * BK, m0, bar);
            tma_load_2d(smem_u32(base + 2 * TMA_TILE_FLOATS), &map_w, kt * BK, n0, bar);
            issued++;
        };

        float accl[8][TMA_TN], accu[8][TMA_TN];
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < TMA_TN; j++) {
                accl[i][j] = -SNB_EPS;
                accu[i][j] = SNB_EPS;
            }

        __syncthreads();  // every thread has finished reading the previous segment's stages
        if (tid == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            for (int kt = ka; kt < kb && kt < ka + TMA_STAGES - 1; kt++) issue(kt);
        }

        for (int kt = ka; kt < kb; kt++, it++) {
            const uint32_t st = it % TMA_STAGES;
            if (!mbar_wait(smem_u32(bars + st), (it / TMA_STAGES) & 1)) abort_flag = 1;
            float* lt = tiles + st * TMA_STAGE_FLOATS;
            float* ut = lt + TMA_TILE_FLOATS;
            const float* wt = ut + TMA_TILE_FLOATS;
            // midpoint repair of inverted intervals, in place; x_L and x_U tiles share the layout,
            // so equal offsets are the same (row, column)
#pragma unroll
            for (int r = 0; r < TMA_TILE_FLOATS / 4 / TMA_NT; r++) {
                const int o = (tid + r * TMA_NT) * 4;
                float4 a = *reinterpret_cast<float4*>(lt + o), b = *reinterpret_cast<float4*>(ut + o);
                if (a.x > b.x || a.y > b.y || a.z > b.z || a.w > b.w) {
                    if (a.x > b.x) a.x = b.x = (a.x + b.x) * 0.5f;
                    if (a.y > b.y) a.y = b.y = (a.y + b.y) * 0.5f;
                    if (a.z > b.z) a.z = b.z = (a.z + b.z) * 0.5f;
                    if (a.w > b.w) a.w = b.w = (a.w + b.w) * 0.5f;
                    *reinterpret_cast<float4*>(lt + o) = a;
                    *reinterpret_cast<float4*>(ut + o) = b;
                }
            }
            __syncthreads();  // repairs visible; everyone is past the previous k-tile's reads
            if (abort_flag) return;  // a wait timed out somewhere in the CTA: leave together
            if (tid == 0 && kt + TMA_STAGES - 1 < kb) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue(kt + TMA_STAGES - 1);   // refills the stage consumed in the previous iteration
            }
#pragma unroll 4
            for (int kk = 0; kk < BK / 2; kk++) {
                float2 lf[8], uf[8], wf[TMA_TN];
                const int chunk = kk >> 1, within = (kk & 1) * 2;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int o = swz(wm * 32 + tb + 4 * i, chunk) + within;
                    lf[i] = *reinterpret_cast<const float2*>(lt + o);
                    uf[i] = *reinterpret_cast<const float2*>(ut + o);
                }
#pragma unroll
                for (int j = 0; j < TMA_TN; j++)
                    wf[j] = *reinterpret_cast<const float2*>(wt + swz(wn * 8 * TMA_TN + tj + 8 * j, chunk) + within);
#pragma unroll
                for (int i = 0; i < 8; i++) {
#pragma unroll
                    for (int j = 0; j < TMA_TN; j++) {
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
            for (int j = 0; j < TMA_TN; j++) {
                const int n = n0 + wn * 8 * TMA_TN + tj + 8 * j;
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// Row-major [rows][cols] fp32 tensor, boxes of 128 rows x 32 columns, 128-byte swizzle.
static bool make_map(CUtensorMap* map, const float* base, int rows, int cols) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)BK, 128u};
    const cuuint32_t elem[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Returns cudaErrorNotSupported when the TMA path does not apply (caller falls back to cp.async).
cudaError_t bound_forward_tma(const float* xl, const float* xu, const float* w, float* yl, float* yu, int B, int CO,
                              int CI, cudaStream_t st) {
    if (CI % 4 != 0 || !aligned16(xl) || !aligned16(xu) || !aligned16(w)) return cudaErrorNotSupported;
    CUtensorMap ml, mu, mw;
    if (!make_map(&ml, xl, B, CI) || !make_map(&mu, xu, B, CI) || !make_map(&mw, w, CO, CI)) return cudaErrorNotSupported;
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(bound_fwd_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TMA_SMEM);
        if (e != cudaSuccess) return e;
        configured[dev & 63].store(true, std::memory_order_release);
    }
    BoundTmaParams p{yl, yu, B, CO, CI, (B + TMA_BM - 1) / TMA_BM, (CO + TMA_BN - 1) / TMA_BN};
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    const long long units = tiles * ((CI + BK - 1) / BK);
    long long grid = sm_count();   // one CTA per SM (192 KiB of tiles each)
    if (tiles % grid == 0) grid = tiles;
    else if (units < grid) grid = units;
    if (grid != tiles) {
        cudaError_t e = cudaMemsetAsync(yl, 0, sizeof(float) * (size_t)B * CO, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(yu, 0, sizeof(float) * (size_t)B * CO, st);
        if (e != cudaSuccess) return e;
    }
    bound_fwd_tma_kernel<<<(unsigned)grid, TMA_NT, TMA_SMEM, st>>>(ml, mu, mw, p);
    return cudaGetLastError();
}

}  // namespace snb

// 1 if a bounded device-side wait ever gave up on the current device (synchronises the device).
extern "C" int snb_device_wait_failed(void) {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, snb::snb_tma_wait_failed, sizeof(int)) != cudaSuccess) return -1;
    return flag;
}
