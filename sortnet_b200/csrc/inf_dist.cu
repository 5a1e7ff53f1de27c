// l-infinity distance neuron: forward (with / without argmax word, dense or index-masked)
// and the sparse backward.
//
// Replaces zbh2047/SortNet core/cuda/inf_dist_cuda.cu (kernels :17-107, :110-212, :214-271;
// launchers :277-354).  Results are identical to that file's: y = max(1e-10, max_c |x - w|)
// bit for bit, pos = lowest c attaining the maximum | sign bit of (x - w), 0 when nothing
// exceeds 1e-10.
//
// Forward = max-plus "GEMM": 8x8 outputs per thread, two reduction steps per instruction pair
// (packed fp32 subtract on a register pair + three-input |.|-max into the accumulator).
// The argmax is not tracked per element: the main loop only records, per output, the first
// 32-wide chunk of the reduction axis in which the accumulator grew to its final value
// (one compare per output per chunk); a second small kernel rescans that one chunk and
// writes the exact word.  Strict '>' on chunk level followed by "first equal element"
// inside the chunk is the same total order as the reference's strict '>' element scan.
#include "tile.cuh"
#include "launch.h"
#include "general_shapes.h"

namespace snb {

struct InfFwdParams {
    const float* x;
    const float* w;
    float* y;
    int* pos;       // TRACK: receives the chunk id (or -1), rewritten by the resolve kernel
    const int* ci;  // [S][CI] kept columns of W per sub-batch, or null
    const int* co;  // [S][CO] kept rows of W per sub-batch, or null
    int B, CO, CI;  // compact sizes seen by x / y
    int W_CI;       // leading dimension of w
    const int* inv; // [S][CI] full column -> compact position (full-width form, see expand_rows_kernel) or null
};

constexpr int CHUNK_TILES = 1;  // argmax chunk = one k-tile = 32 reduction steps

enum { MODE_VEC = 0, MODE_SCALAR = 1, MODE_GATHER = 2, MODE_ROWVEC = 3 };

// Four reduction steps of one output: acc = max(acc, |x_k - w_k|), k = 0..3, operands given as
// two 64-bit register pairs each: packed subtracts + three-input |.|-max.  All instruction forms of
// subtract + max cost two issue cycles per element on sm_100a (scalar subtract + two-input max and
// the mixed forms were measured); this one needs the fewest auxiliary instructions.
__device__ __forceinline__ void linf_step(float& acc, const ulonglong2& x, const ulonglong2& w) {
    float a, b;
    unpack2(sub2(x.x, w.x), a, b);
    acc = max3abs(acc, a, b);
    unpack2(sub2(x.y, w.y), a, b);
    acc = max3abs(acc, a, b);
}

// Turns the chunk id left by the tracking kernel into the reference's argmax word.  Four lanes
// share one output: each rescans eight consecutive elements of the output's 32-element chunk
// (32 contiguous bytes of the x row and of the W row, two 16-byte loads each), keeps the
// lowest element that equals y, and two shuffles pick the lowest of the four.  Every lane reads its
// output's (chunk, y, row) itself - the four loads of a group coalesce into one - so nothing is
// broadcast by shuffles and a thread's sixteen operand loads are all independent.
// FROM_WS: the tracking kernel ran split over k and left (value bits << 32 | ~chunk) keys in the
// 64-bit workspace instead of y / pos; y is written here too.
// Needs dense columns (no ci list), CI and W_CI multiples of 4 and 16-byte aligned x and w.
template <bool FROM_WS>
__global__ void __launch_bounds__(256) inf_resolve_kernel(const InfFwdParams p, const unsigned long long* __restrict__ keys) {
    static_assert(CHUNK_TILES * BK == 32, "four lanes x eight elements per chunk");
    const int q4 = threadIdx.x & 3;
    const int m = blockIdx.x, n = blockIdx.y * 64 + (threadIdx.x >> 2);   // grid: B x ceil(CO / 64)
    const bool have = n < p.CO;
    const size_t o = have ? (size_t)m * p.CO + n : 0;
    const int s = m / SNB_SUB_BATCH;
    int chunk = -1;
    float yv = 0.f;
    if (have) {
        if (FROM_WS) {
            const unsigned long long key = keys[o];
            yv = __uint_as_float((uint32_t)(key >> 32));
            chunk = (int)(0xffffffffu - (uint32_t)key);      // 0xffffffff - 0 = -1: no chunk
        } else {
            chunk = p.pos[o];
            yv = p.y[o];
        }
    }
    constexpr uint32_t NONE = 0xffffu;
    uint32_t mine = NONE;                                    // (element of the chunk << 1) | (x - w < 0)
    if (chunk >= 0) {
        const int row = p.co ? p.co[(size_t)s * p.CO + n] : n;
        const int c0 = chunk * 32 + q4 * 8;
        const float* xr = p.x + (size_t)m * p.CI;
        const float* wr = p.w + (size_t)row * p.W_CI;
        float xv[8], wv[8];
        bool ok[8];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const bool in = c0 + 4 * h < p.CI;               // CI % 4 == 0: a quad is inside or outside
            const float4 a = in ? *reinterpret_cast<const float4*>(xr + c0 + 4 * h) : make_float4(0, 0, 0, 0);
            const float4 b = in ? *reinterpret_cast<const float4*>(wr + c0 + 4 * h) : make_float4(0, 0, 0, 0);
            xv[4 * h] = a.x; xv[4 * h + 1] = a.y; xv[4 * h + 2] = a.z; xv[4 * h + 3] = a.w;
            wv[4 * h] = b.x; wv[4 * h + 1] = b.y; wv[4 * h + 2] = b.z; wv[4 * h + 3] = b.w;
            ok[4 * h] = ok[4 * h + 1] = ok[4 * h + 2] = ok[4 * h + 3] = in;
        }
#pragma unroll
        for (int e = 7; e >= 0; e--) {                       // descending: the lowest match stays
            const float t = xv[e] - wv[e];
            if (ok[e] && fabsf(t) == yv) mine = (uint32_t)((q4 * 8 + e) << 1) | (t < 0.f ? 1u : 0u);
        }
    }
    mine = min(mine, __shfl_xor_sync(0xffffffffu, mine, 1));
    mine = min(mine, __shfl_xor_sync(0xffffffffu, mine, 2));
    if (!have || q4 != 0) return;
    uint32_t word = 0;
    if (mine != NONE) {
        int idx = chunk * 32 + (int)(mine >> 1);
        if (p.inv) idx = p.inv[(size_t)s * p.CI + idx];      // full-width column -> position in the kept list
        word = (uint32_t)idx | ((mine & 1u) ? SNB_SIGN_BIT : 0u);
    }
    if (FROM_WS) p.y[o] = yv;
    p.pos[o] = (int)word;
}

// The same for operands that cannot be read with aligned 16-byte loads (a kept-column list, odd
// row lengths):
// One warp owns 32 consecutive outputs of one row; for each of them the 32 lanes load the 32
// elements of its chunk (coalesced in x, one row segment of W), compare with y and the lowest
// matching lane gives the index.  RESOLVE_BATCH outputs are in flight per warp to overlap the
// index -> weight load chains (the kernel is bound by their latency).
constexpr int RESOLVE_BATCH = 8;

template <bool FROM_WS>
__global__ void __launch_bounds__(256) inf_resolve_lists_kernel(const InfFwdParams p, const unsigned long long* __restrict__ keys) {
    static_assert(CHUNK_TILES * BK == 32, "one lane per chunk element");
    const int lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * 32;
    const int m = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (m >= p.B) return;
    const int s = m / SNB_SUB_BATCH;
    const int n = n0 + lane;
    const bool have = n < p.CO;
    const size_t o = (size_t)m * p.CO + n;
    int my_chunk = -1;
    float my_y = 0.f;
    if (have) {
        if (FROM_WS) {
            const unsigned long long key = keys[o];
            my_y = __uint_as_float((uint32_t)(key >> 32));
            my_chunk = (int)(0xffffffffu - (uint32_t)key);      // 0xffffffff - 0 = -1: no chunk
            p.y[o] = my_y;
        } else {
            my_chunk = p.pos[o];
            my_y = p.y[o];
        }
    }
    const int my_row = have ? (p.co ? p.co[(size_t)s * p.CO + n] : n) : 0;
    const float* xr = p.x + (size_t)m * p.CI;
    const int* ci_s = p.ci ? p.ci + (size_t)s * p.CI : nullptr;
    uint32_t my_word = 0;
#pragma unroll 1
    for (int base = 0; base < 32; base += RESOLVE_BATCH) {
        int col[RESOLVE_BATCH];
        float xv[RESOLVE_BATCH], yv[RESOLVE_BATCH], wv[RESOLVE_BATCH];
        int rowv[RESOLVE_BATCH];
#pragma unroll
        for (int u = 0; u < RESOLVE_BATCH; u++) {
            const int chunk = __shfl_sync(0xffffffffu, my_chunk, base + u);
            yv[u] = __shfl_sync(0xffffffffu, my_y, base + u);
            rowv[u] = __shfl_sync(0xffffffffu, my_row, base + u);
            const int c = chunk * 32 + lane;
            const bool ok = chunk >= 0 && c < p.CI;
            col[u] = ok ? (ci_s ? ci_s[c] : c) : -1;
            xv[u] = ok ? xr[c] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < RESOLVE_BATCH; u++) wv[u] = col[u] >= 0 ? p.w[(size_t)rowv[u] * p.W_CI + col[u]] : 0.f;
#pragma unroll
        for (int u = 0; u < RESOLVE_BATCH; u++) {
            const float t = xv[u] - wv[u];
            const uint32_t hits = __ballot_sync(0xffffffffu, col[u] >= 0 && fabsf(t) == yv[u]);
            const int first = hits ? __ffs(hits) - 1 : 0;
            const float tf = __shfl_sync(0xffffffffu, t, first);
            const int chunk = __shfl_sync(0xffffffffu, my_chunk, base + u);
            const uint32_t word = hits ? ((uint32_t)(chunk * 32 + first) | (tf >= 0 ? 0u : SNB_SIGN_BIT)) : 0u;
            if (lane == base + u) my_word = word;
        }
    }
    if (have) p.pos[o] = (int)my_word;
}

static cudaError_t launch_resolve(const InfFwdParams& p, const unsigned long long* keys, bool from_ws, cudaStream_t st) {
    const dim3 grid(p.B, (p.CO + 63) / 64);
    const bool vec = !p.ci && (p.CI % 4 == 0) && (p.W_CI % 4 == 0) && aligned16(p.x) && aligned16(p.w) &&
                     (p.CO + 63) / 64 <= 65535;
    const dim3 lists_grid((p.CO + 31) / 32, (p.B + 7) / 8);
    if (from_ws) {
        if (vec) inf_resolve_kernel<true><<<grid, 256, 0, st>>>(p, keys);
        else inf_resolve_lists_kernel<true><<<lists_grid, 256, 0, st>>>(p, keys);
    } else {
        if (vec) inf_resolve_kernel<false><<<grid, 256, 0, st>>>(p, nullptr);
        else inf_resolve_lists_kernel<false><<<lists_grid, 256, 0, st>>>(p, nullptr);
    }
    return cudaGetLastError();
}

// Sparse backward: one CTA per batch row.  grad_x of the row is accumulated in shared
// memory (many outputs of a row share an argmax column) and written once, so grad_x needs
// neither a memset nor global atomics; grad_w gets one global reduction per output.
__global__ void __launch_bounds__(256) inf_bwd_kernel(const float* __restrict__ g,
                                                      const int* __restrict__ pos, int B, int CO,
                                                      int CI, float* __restrict__ gx,
                                                      float* __restrict__ gw,
                                                      const int* __restrict__ ci,
                                                      const int* __restrict__ co, int W_CI) {
    extern __shared__ float row[];  // [CI]
    const int b = blockIdx.x, s = b / SNB_SUB_BATCH;
    for (int c = threadIdx.x; c < CI; c += blockDim.x) row[c] = 0.f;
    __syncthreads();
    const int* ci_s = ci ? ci + (size_t)s * CI : nullptr;
    const int* co_s = co ? co + (size_t)s * CO : nullptr;
    for (int j = threadIdx.x; j < CO; j += blockDim.x) {
        const uint32_t pw = (uint32_t)pos[(size_t)b * CO + j];
        const float gv = g[(size_t)b * CO + j];
        const int idx = (int)(pw & ~SNB_SIGN_BIT);
        const float v = (pw & SNB_SIGN_BIT) ? -gv : gv;
        atomicAdd(&row[idx], v);
        if (gw) {
            const int r = co_s ? co_s[j] : j;
            const int c = ci_s ? ci_s[idx] : idx;
            atomicAdd(&gw[(size_t)r * W_CI + c], -v);
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < CI; c += blockDim.x) gx[(size_t)b * CI + c] = row[c];
}

// Same as above for rows too wide for shared memory: global atomics into a zeroed grad_x.
__global__ void __launch_bounds__(256) inf_bwd_wide_kernel(const float* __restrict__ g,
                                                           const int* __restrict__ pos, int B,
                                                           int CO, int CI, float* __restrict__ gx,
                                                           float* __restrict__ gw,
                                                           const int* __restrict__ ci,
                                                           const int* __restrict__ co, int W_CI) {
    const int b = blockIdx.y, s = b / SNB_SUB_BATCH;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= CO) return;
    const uint32_t pw = (uint32_t)pos[(size_t)b * CO + j];
    const float gv = g[(size_t)b * CO + j];
    const int idx = (int)(pw & ~SNB_SIGN_BIT);
    const float v = (pw & SNB_SIGN_BIT) ? -gv : gv;
    atomicAdd(&gx[(size_t)b * CI + idx], v);
    if (gw) {
        const int r = co ? co[(size_t)s * CO + j] : j;
        const int c = ci ? ci[(size_t)s * CI + idx] : idx;
        atomicAdd(&gw[(size_t)r * W_CI + c], -v);
    }
}

// Full-width form of a column-masked input: xw[b][k] = x[b][c] where k = ci[s][c], NaN in every
// dropped column, and inv[s][k] = c (or -1).  max.f32 returns the other operand when one is NaN, so a
// NaN difference never reaches the accumulator and the distance over all W_CI columns of xw equals
// the distance over the kept columns, bit for bit; in exchange W is read along whole rows with
// 16-byte copies instead of one 4-byte copy per kept element.  With ascending lists (the
// sampler's and the reference's, core/models/norm_dist.py:14-17) full-column order is compact order,
// so "first chunk that reached the maximum, first equal element in it" picks the same position.
// One CTA per batch row; the first row of every sub-batch also writes the inverse list.
__global__ void __launch_bounds__(256) expand_rows_kernel(const float* __restrict__ x, const int* __restrict__ ci, int B,
                                                          int CI, int W_CI, float* __restrict__ xw,
                                                          int* __restrict__ inv) {
    const int b = blockIdx.x, s = b / SNB_SUB_BATCH;
    const bool first = (b % SNB_SUB_BATCH) == 0;
    float* row = xw + (size_t)b * W_CI;
    int* inv_s = inv + (size_t)s * W_CI;
    const float nan = __int_as_float(0x7fc00000);
    for (int k = threadIdx.x; k < W_CI; k += blockDim.x) {
        row[k] = nan;
        if (first) inv_s[k] = -1;
    }
    __syncthreads();   // this CTA's own global writes are ordered for its threads
    const int* ci_s = ci + (size_t)s * CI;
    const float* xr = x + (size_t)b * CI;
    for (int c = threadIdx.x; c < CI; c += blockDim.x) {
        const int k = ci_s[c];
        row[k] = xr[c];
        if (first) inv_s[k] = c;
    }
}

// Forward kernel (dense or index-masked operands, with or without argmax tracking), stream-K over
// (tile, k-tile) pairs: every CTA of a persistent grid does the same number of k-tiles, so the
// run time does not depend on how the tile count divides the SMs (with 32-row masked tiles and
// Binomial mask sizes that count changes from step to step).  Partial tiles merge exactly:
// plain values by atomicMax on the non-negative float patterns, (value, chunk) pairs by 64-bit
// atomicMax on keys in caller-provided scratch; without scratch, tracking runs whole tiles only.
struct InfSkParams {
    const float* x;
    const float* w;
    float* y;
    int* pos;                   // TRACK without workspace: receives chunk ids
    unsigned long long* keys;   // TRACK split over k: (value bits << 32 | 0xffffffff - chunk), zeroed
    const int* ci;              // GATHER: kept columns / rows of W per 32-row sub-batch (or null)
    const int* co;
    int B, CO, CI, W_CI;
    int tiles_m, tiles_n;
};

__device__ __forceinline__ unsigned long long pack_key(float v, uint32_t chunk16) {
    const uint32_t lo = chunk16 == 0xffffu ? 0u : 0xffffffffu - chunk16;
    return ((unsigned long long)__float_as_uint(v) << 32) | lo;
}

template <int WM, int WN, int MODE, bool TRACK>
__global__ void __launch_bounds__(WM* WN * 32) inf_fwd_sk_kernel(const InfSkParams p) {
    constexpr int BM = 32 * WM, BN = 64 * WN, NT = WM * WN * 32;
    static_assert((MODE != MODE_GATHER && MODE != MODE_ROWVEC) || WM == 1, "masked tiles are one 32-row sub-batch");
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;
    float* ws = smem + 2 * BM * LDS;
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
        GatherW<BN, NT> gw;
        RowVecW<BN, NT> rw;
        const int* ci_s = nullptr;
        if (MODE == MODE_GATHER) {
            const int s = m0 / SNB_SUB_BATCH;
            ci_s = p.ci ? p.ci + (size_t)s * p.CI : nullptr;
            gw.init_rows(p.co ? p.co + (size_t)s * p.CO : nullptr, n0, p.CO, p.W_CI, tid);
            gw.fetch_cols(ci_s, ka * BK, p.CI, tid);
        }
        if (MODE == MODE_ROWVEC)
            rw.init_rows(p.co ? p.co + (size_t)(m0 / SNB_SUB_BATCH) * p.CO : nullptr, n0, p.CO, p.W_CI, tid);
        auto stage = [&](int kt, int st) {
            float* xd = xs + st * BM * LDS;
            float* wd = ws + st * BN * LDS;
            if (MODE == MODE_ROWVEC) {
                // full-width form: x holds all W_CI columns (NaN where a column was dropped, which
                // the three-input max ignores), W rows come through the kept-row list
                stage_dense_vec<BM, NT>(xd, p.x, m0, p.B, p.CI, kt * BK, p.CI, tid);
                rw.stage(wd, p.w, kt * BK, p.CI, tid);
            } else if (MODE == MODE_VEC) {
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
        float acc[8][8];
        float prev[TRACK ? 8 : 1][TRACK ? 8 : 1];
        uint32_t q[TRACK ? 8 : 1][TRACK ? 4 : 1];  // two 16-bit chunk ids per word, 0xffff = none
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[i][j] = SNB_EPS;
        if (TRACK) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
#pragma unroll
                for (int j = 0; j < 8; j++) prev[i][j] = SNB_EPS;
#pragma unroll
                for (int j = 0; j < 4; j++) q[i][j] = 0xffffffffu;
            }
        }
        __syncthreads();  // the previous tile's readers are done with both stages
        stage(ka, ka & 1);
        cp_async_commit();
        if (MODE == MODE_GATHER && ka + 1 < kb) gw.fetch_cols(ci_s, (ka + 1) * BK, p.CI, tid);
        for (int kt = ka; kt < kb; kt++) {
            cp_async_wait<0>();
            __syncthreads();
            if (kt + 1 < kb) {
                stage(kt + 1, (kt + 1) & 1);
                // kept-column indices of the tile after next: their load latency hides behind
                // this tile's arithmetic
                if (MODE == MODE_GATHER && kt + 2 < kb) gw.fetch_cols(ci_s, (kt + 2) * BK, p.CI, tid);
            }
            cp_async_commit();
            const float* xr = xs + (kt & 1) * BM * LDS + (wm * 32 + tb) * LDS;
            const float* wr = ws + (kt & 1) * BN * LDS + (wn * 64 + tj) * LDS;
#pragma unroll 2
            for (int kk = 0; kk < BK / 4; kk++) {
                ulonglong2 xf[8], wf[8];
#pragma unroll
                for (int i = 0; i < 8; i++)
                    xf[i] = *reinterpret_cast<const ulonglong2*>(xr + i * 4 * LDS + kk * 4);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    wf[j] = *reinterpret_cast<const ulonglong2*>(wr + j * 8 * LDS + kk * 4);
#pragma unroll
                for (int i = 0; i < 8; i++) {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        linf_step(acc[i][j], xf[i], wf[j]);
                    }
                }
            }
            if (TRACK) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        if (acc[i][j] > prev[i][j])
                            q[i][j >> 1] = (j & 1) ? __byte_perm(q[i][j >> 1], (uint32_t)kt, 0x5410)
                                                   : __byte_perm(q[i][j >> 1], (uint32_t)kt, 0x3254);
                        prev[i][j] = acc[i][j];
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
                if (TRACK) {
                    const uint32_t c = (j & 1) ? (q[i][j >> 1] >> 16) : (q[i][j >> 1] & 0xffffu);
                    if (p.keys) {
                        const unsigned long long key = pack_key(acc[i][j], c);
                        if (whole) p.keys[o] = key;
                        else atomicMax(p.keys + o, key);
                    } else {
                        p.y[o] = acc[i][j];
                        p.pos[o] = c == 0xffffu ? -1 : (int)c;
                    }
                } else {
                    if (whole) p.y[o] = acc[i][j];
                    else atomic_max_nonneg(p.y + o, acc[i][j]);
                }
            }
        }
        u0 += kb - ka;
    }
}

// keys: 8 * B * CO bytes of scratch or null.  Without it a TRACK launch uses whole tiles only.
template <int WM, int WN, int MODE, bool TRACK>
static cudaError_t launch_sk(InfSkParams p, bool* split, cudaStream_t st) {
    constexpr int BM = 32 * WM, BN = 64 * WN, NT = WM * WN * 32;
    constexpr int SMEM = 2 * (BM + BN) * LDS * (int)sizeof(float);
    auto kern = inf_fwd_sk_kernel<WM, WN, MODE, TRACK>;
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
    // whole tiles when they balance anyway or when there is nowhere to merge (value, chunk) pairs; a
    // problem with fewer (tile, k-tile) pairs than resident CTAs (few tiles, e.g. a narrow head
    // layer) still spreads over one CTA per pair
    if (tiles % grid == 0 || (TRACK && !p.keys)) grid = tiles;
    else if (units < grid) grid = units;
    *split = (grid != tiles);
    if (!*split) {
        p.keys = nullptr;
    } else {
        cudaError_t e = TRACK ? cudaMemsetAsync(p.keys, 0, sizeof(unsigned long long) * (size_t)p.B * p.CO, st)
                              : cudaMemsetAsync(p.y, 0, sizeof(float) * (size_t)p.B * p.CO, st);
        if (e != cudaSuccess) return e;
    }
    kern<<<(unsigned)grid, NT, SMEM, st>>>(p);
    return cudaGetLastError();
}

// *split tells whether tiles were shared between CTAs; for TRACK that means the result is in
// `keys` (workspace) and still has to be turned into y / pos by the resolve kernel.
template <bool TRACK>
static cudaError_t dispatch_fwd(const InfFwdParams& q, unsigned long long* keys, bool* split, cudaStream_t st,
                                bool full_width = false) {
    InfSkParams p{q.x, q.w, q.y, q.pos, keys, q.ci, q.co, q.B, q.CO, q.CI, q.W_CI, 0, 0};
    const int sms = sm_count();
    if (full_width) return launch_sk<1, 4, MODE_ROWVEC, TRACK>(p, split, st);
    if (q.ci || q.co) {
        const long wide = (long)((q.B + 31) / 32) * ((q.CO + 255) / 256);
        return wide >= sms / 2 ? launch_sk<1, 4, MODE_GATHER, TRACK>(p, split, st)
                               : launch_sk<1, 2, MODE_GATHER, TRACK>(p, split, st);
    }
    const bool vec = (q.CI % 4 == 0) && (q.W_CI % 4 == 0) && aligned16(q.x) && aligned16(q.w);
    // 64-row tiles from two sub-batches up (measured: never slower than 32-row tiles, 1-2 % faster at
    // 64..256 rows); the stream-K split keeps every SM busy whatever the tile count
    if (q.B > 32)
        return vec ? launch_sk<2, 2, MODE_VEC, TRACK>(p, split, st) : launch_sk<2, 2, MODE_SCALAR, TRACK>(p, split, st);
    return vec ? launch_sk<1, 2, MODE_VEC, TRACK>(p, split, st) : launch_sk<1, 2, MODE_SCALAR, TRACK>(p, split, st);
}

cudaError_t inf_forward_values(const float* x, const float* w, float* y, const int* ci, const int* co,
                               int B, int CO, int CI, int W_CI, cudaStream_t st) {
    InfFwdParams p{x, w, y, nullptr, ci, co, B, CO, CI, W_CI};
    bool split = false;
    return dispatch_fwd<false>(p, nullptr, &split, st);
}

}  // namespace snb

using namespace snb;

static int check_fwd(const void* x, const void* w, const void* y, int B, int CO, int CI, int G,
                     int HW, int W_CO, int W_CI, const int* ci, const int* co) {
    if (!x || !w || !y) return SNB_ERR_NULL_POINTER;
    if (G != 1 || HW != 1) return SNB_ERR_UNSUPPORTED;
    if (B <= 0 || CO <= 0 || CI <= 0 || W_CO <= 0 || W_CI <= 0) return SNB_ERR_BAD_SHAPE;
    if (!ci && W_CI != CI) return SNB_ERR_BAD_SHAPE;
    if (!co && W_CO != CO) return SNB_ERR_BAD_SHAPE;
    if (CI > W_CI || CO > W_CO) return SNB_ERR_BAD_SHAPE;
    if ((long long)W_CO * W_CI >= (1ll << 31) || (long long)B * CO >= (1ll << 31) ||
        (long long)B * CI >= (1ll << 31))
        return SNB_ERR_TOO_LARGE;
    return SNB_OK;
}

static int inf_forward_impl(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                            float* y, int* pos, const int* ci, const int* co, int W_CO, int W_CI,
                            unsigned long long* keys, cudaStream_t st) {
    if (G != 1 || HW != 1)
        return general_inf_forward(x, w, B, CO, CI, G, HW, y, pos, ci, co, W_CO, W_CI, st);
    int rc = check_fwd(x, w, y, B, CO, CI, G, HW, W_CO, W_CI, ci, co);
    if (rc) return rc;
    if (!pos) return SNB_ERR_NULL_POINTER;
    if ((CI + CHUNK_TILES * BK - 1) / (CHUNK_TILES * BK) >= 0xffff) return SNB_ERR_TOO_LARGE;
    InfFwdParams p{x, w, y, pos, ci, co, B, CO, CI, W_CI};
    bool split = false;
    SNB_CUDA(dispatch_fwd<true>(p, keys, &split, st));
    SNB_CUDA(launch_resolve(p, keys, split, st));
    return SNB_OK;
}

extern "C" int snb_inf_dist_forward(const float* x, const float* w, int B, int CO, int CI, int G,
                                    int HW, float* y, int* pos, const int* w_index_ci,
                                    const int* w_index_co, int W_CO, int W_CI, void* stream) {
    return inf_forward_impl(x, w, B, CO, CI, G, HW, y, pos, w_index_ci, w_index_co, W_CO, W_CI, nullptr,
                            (cudaStream_t)stream);
}

extern "C" size_t snb_inf_dist_forward_workspace_bytes(int B, int CO) {
    return (B > 0 && CO > 0) ? sizeof(unsigned long long) * (size_t)B * (size_t)CO : 0;
}

extern "C" int snb_inf_dist_forward_ws(const float* x, const float* w, int B, int CO, int CI, int G,
                                       int HW, float* y, int* pos, const int* w_index_ci,
                                       const int* w_index_co, int W_CO, int W_CI, void* workspace,
                                       size_t workspace_bytes, void* stream) {
    unsigned long long* keys = nullptr;
    if (workspace) {
        if (reinterpret_cast<uintptr_t>(workspace) & 7u) return SNB_ERR_ALIGNMENT;
        if (workspace_bytes >= snb_inf_dist_forward_workspace_bytes(B, CO)) keys = (unsigned long long*)workspace;
    }
    return inf_forward_impl(x, w, B, CO, CI, G, HW, y, pos, w_index_ci, w_index_co, W_CO, W_CI, keys,
                            (cudaStream_t)stream);
}

// Workspace of the ascending-list form: merge keys [B * CO] u64, then the full-width input
// [B * W_CI] f32 (16-byte aligned), then the inverse lists [S * W_CI] i32.
static size_t sorted_ws_input_offset(int B, int CO) {
    return (sizeof(unsigned long long) * (size_t)B * (size_t)CO + 15) & ~(size_t)15;
}
extern "C" size_t snb_inf_dist_forward_sorted_workspace_bytes(int B, int CO, int W_CI) {
    if (B <= 0 || CO <= 0 || W_CI <= 0) return 0;
    const size_t S = (size_t)(B + SNB_SUB_BATCH - 1) / SNB_SUB_BATCH;
    return sorted_ws_input_offset(B, CO) + sizeof(float) * (size_t)B * W_CI + sizeof(int) * S * W_CI;
}

// Masked forward whose index lists are in ascending order (every list strictly increasing), as
// the sampler and the reference's sample_mask produce them.  Same results as
// snb_inf_dist_forward_ws; with enough workspace and 16-byte aligned rows of W it runs in the
// full-width form (expand_rows_kernel), otherwise through the general masked path.  Lists in
// another order still give exact distances, but ties for the maximum between different columns
// may then resolve to another of the tied positions than the reference's scan order would.
extern "C" int snb_inf_dist_forward_sorted_ws(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                                              float* y, int* pos, const int* w_index_ci, const int* w_index_co,
                                              int W_CO, int W_CI, void* workspace, size_t workspace_bytes,
                                              void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    const bool masked = w_index_ci || w_index_co;
    bool fast = masked && G == 1 && HW == 1 && workspace && pos && (W_CI % 4 == 0) && aligned16(w) &&
                !(reinterpret_cast<uintptr_t>(workspace) & 15u) &&
                workspace_bytes >= snb_inf_dist_forward_sorted_workspace_bytes(B, CO, W_CI) &&
                (long long)B * W_CI < (1ll << 31);
    // computing the dropped columns too must cost less than the vector copies save
    if (fast && w_index_ci && (long long)CI * 4 < (long long)W_CI * 3) fast = false;
    if (fast && !w_index_ci && !aligned16(x)) fast = false;
    if (!fast)
        return snb_inf_dist_forward_ws(x, w, B, CO, CI, G, HW, y, pos, w_index_ci, w_index_co, W_CO, W_CI, workspace,
                                       workspace_bytes, stream);
    int rc = check_fwd(x, w, y, B, CO, CI, G, HW, W_CO, W_CI, w_index_ci, w_index_co);
    if (rc) return rc;
    if ((W_CI + CHUNK_TILES * BK - 1) / (CHUNK_TILES * BK) >= 0xffff) return SNB_ERR_TOO_LARGE;
    unsigned long long* keys = (unsigned long long*)workspace;
    const float* xin = x;
    const int* inv = nullptr;
    if (w_index_ci) {
        float* xw = reinterpret_cast<float*>(static_cast<char*>(workspace) + sorted_ws_input_offset(B, CO));
        int* inv_w = reinterpret_cast<int*>(xw + (size_t)B * W_CI);
        expand_rows_kernel<<<B, 256, 0, st>>>(x, w_index_ci, B, CI, W_CI, xw, inv_w);
        SNB_CUDA(cudaGetLastError());
        xin = xw;
        inv = inv_w;
    }
    // the kernels see a dense input of W_CI columns and a row-masked W
    InfFwdParams p{xin, w, y, pos, nullptr, w_index_co, B, CO, W_CI, W_CI, inv};
    bool split = false;
    SNB_CUDA(dispatch_fwd<true>(p, keys, &split, st, true));
    SNB_CUDA(launch_resolve(p, keys, split, st));
    return SNB_OK;
}

extern "C" int snb_inf_dist_forward_nograd(const float* x, const float* w, int B, int CO, int CI,
                                           int G, int HW, float* y, void* stream) {
    if (G != 1 || HW != 1)
        return general_inf_forward(x, w, B, CO, CI, G, HW, y, nullptr, nullptr, nullptr, CO, CI,
                                   (cudaStream_t)stream);
    int rc = check_fwd(x, w, y, B, CO, CI, G, HW, CO, CI, nullptr, nullptr);
    if (rc) return rc;
    InfFwdParams p{x, w, y, nullptr, nullptr, nullptr, B, CO, CI, CI};
    bool split = false;
    SNB_CUDA(dispatch_fwd<false>(p, nullptr, &split, (cudaStream_t)stream));
    return SNB_OK;
}

// ---- entry point that allocates nothing ----------------------------------------------------
// Scratch for snb_inf_dist_forward_noalloc: one 64-bit merge key per output, held by every GPU
// that loads this library until the process exits (8 MiB).
#define SNB_NOALLOC_MAX_OUTPUTS (1 << 20)
static __device__ __align__(256) unsigned long long snb_noalloc_keys[SNB_NOALLOC_MAX_OUTPUTS];

// Device address of snb_noalloc_keys on the current device.  In host code the array's name is
// only a handle for the runtime, not a pointer a kernel could use, so the address is looked up
// once per device with that device current and cached.
static cudaError_t noalloc_keys_address(unsigned long long** out) {
    static std::atomic<unsigned long long*> cached[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    unsigned long long* keys = cached[dev].load(std::memory_order_acquire);
    if (!keys) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, snb_noalloc_keys);
        if (e != cudaSuccess) return e;
        keys = static_cast<unsigned long long*>(ptr);
        cached[dev].store(keys, std::memory_order_release);     // every thread looks up the same address
    }
    *out = keys;
    return cudaSuccess;
}

extern "C" int snb_inf_dist_forward_noalloc(const float* x, const float* w, int B, int CO, int CI,
                                            int G, int HW, float* y, int* pos, void* stream) {
    if (G != 1 || HW != 1) return SNB_ERR_UNSUPPORTED;  // the general shapes take scratch from an allocator
    if (B > 0 && CO > 0 && (long long)B * CO > SNB_NOALLOC_MAX_OUTPUTS) return SNB_ERR_STATIC_CAPACITY;
    unsigned long long* keys = nullptr;
    SNB_CUDA(noalloc_keys_address(&keys));
    // The launcher zero-fills the keys it is going to merge into (cudaMemsetAsync on `stream`)
    // before the kernel runs, so what an earlier call left in the array does not matter.
    return inf_forward_impl(x, w, B, CO, CI, G, HW, y, pos, nullptr, nullptr, CO, CI, keys,
                            (cudaStream_t)stream);
}

extern "C" int snb_inf_dist_forward_noalloc_max_outputs(void) { return SNB_NOALLOC_MAX_OUTPUTS; }

static int inf_backward(const float* g, const int* pos, int B, int CO, int CI, int G, int HW,
                        float* gx, float* gw, const int* ci, const int* co, int W_CO, int W_CI,
                        cudaStream_t st) {
    if (G != 1 || HW != 1)
        return general_inf_backward(g, pos, B, CO, CI, G, HW, gx, gw, ci, co, W_CO, W_CI, st);
    if (!g || !pos || !gx) return SNB_ERR_NULL_POINTER;
    if (B <= 0 || CO <= 0 || CI <= 0) return SNB_ERR_BAD_SHAPE;
    if (gw) {
        if (W_CO <= 0 || W_CI <= 0 || (!ci && W_CI != CI) || (!co && W_CO != CO)) return SNB_ERR_BAD_SHAPE;
        if ((long long)W_CO * W_CI >= (1ll << 31)) return SNB_ERR_TOO_LARGE;
        SNB_CUDA(cudaMemsetAsync(gw, 0, sizeof(float) * (size_t)W_CO * W_CI, st));
    }
    if ((size_t)CI * sizeof(float) <= 48 * 1024) {
        inf_bwd_kernel<<<B, 256, CI * sizeof(float), st>>>(g, pos, B, CO, CI, gx, gw, ci, co, W_CI);
    } else {
        SNB_CUDA(cudaMemsetAsync(gx, 0, sizeof(float) * (size_t)B * CI, st));
        dim3 grid((CO + 255) / 256, B);
        inf_bwd_wide_kernel<<<grid, 256, 0, st>>>(g, pos, B, CO, CI, gx, gw, ci, co, W_CI);
    }
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

extern "C" int snb_inf_dist_backward_input(const float* grad_output, const int* pos, int B, int CO,
                                           int CI, int G, int HW, float* grad_input, void* stream) {
    return inf_backward(grad_output, pos, B, CO, CI, G, HW, grad_input, nullptr, nullptr, nullptr,
                        CO, CI, (cudaStream_t)stream);
}

extern "C" int snb_inf_dist_backward_input_weight(const float* grad_output, const int* pos, int B,
                                                  int CO, int CI, int G, int HW, float* grad_input,
                                                  float* grad_weight, const int* w_index_ci,
                                                  const int* w_index_co, int W_CO, int W_CI,
                                                  void* stream) {
    if (!grad_weight) return SNB_ERR_NULL_POINTER;
    return inf_backward(grad_output, pos, B, CO, CI, G, HW, grad_input, grad_weight, w_index_ci,
                        w_index_co, W_CO, W_CI, (cudaStream_t)stream);
}
