// Sort neuron: the deterministic, evaluation-time form of the masked l-infinity neuron.
//   y[b,j] = (1e-10 + sum_{r<K} q (1-q)^r * (r-th largest |x[b,c] - w[j,c]|)) / (1 - (1-q)^K)
// and its interval bounds, positions of the K largest elements, and the sparse backward.
//
// Replaces zbh2047/SortNet core/cuda/sort_neuron.cu (kernels :16-102, :115-214, :216-314, :316-375;
// launchers :403-562).  K = min(CI, truncate) is 10 in every reference recipe; 2 <= K <= 25 is
// accepted like there.  The values-only kernels keep a sorted K-slot list per output in
// registers and insert with the min/max chain of the reference; they always carry 10 (or 25)
// slots and use the top K of them, which is the same set.  The weighted sum is evaluated in
// the reference's operation order; results agree with its kernels to fp32 rounding (the
// reference binary may contract multiply-adds differently), positions agree exactly.
#include "tile.cuh"
#include "launch.h"
#include "general_shapes.h"

namespace snb {

struct SortParams {
    const float* x;   // point value, or lower end of the box
    const float* xu;  // upper end of the box (bounds only)
    const float* w;
    float* y;         // value, or lower bound
    float* yu;        // upper bound (bounds only)
    int* pos;         // [K][B][CO] or null
    int B, CO, CI, K;
    float q;
};

// ans = eps0 + sum over ranks, then / (1 - (1-q)^K); res ascending with res[KMAX-1] the largest.
template <int KMAX>
__device__ __forceinline__ float combine(const float (&res)[KMAX], int K, float q, float eps0) {
    float ans = eps0, c = 1.0f;
#pragma unroll
    for (int r = 0; r < KMAX; r++) {
        if (r < K) {
            ans += res[KMAX - 1 - r] * c * q;
            c *= 1 - q;
        }
    }
    return ans / (1 - c);
}

// CTA of 256 threads, TM x TN outputs per thread (rows ty + 16 i, columns tx + 16 j): 2 x 2 for up to
// 10 slots (64 registers for values, 128 for bounds: 4 resp. 2 CTAs per SM - the kernel lives on
// hiding the subtract -> compare -> vote -> branch latency of every element, so resident warps
// matter more than operand reuse), 2 x 4 resp. 2 x 2 for up to 25 slots; BOUND carries two chains
// per output (bottom-K of min(t1,t2), top-K of max(t1,t2)).
template <int KMAX, bool BOUND>
__global__ void __launch_bounds__(256, KMAX > 10 ? 1 : (BOUND ? 2 : 4)) sort_fwd_kernel(const SortParams p) {
    constexpr int TM = 2, TN = (BOUND || KMAX <= 10) ? 2 : 4, BM = 16 * TM, BN = 16 * TN, NT = 256;
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;                              // [2][BM][LDS]
    float* us = xs + 2 * BM * LDS;                 // [2][BM][LDS] (BOUND)
    float* ws = BOUND ? us + 2 * BM * LDS : us;    // [2][BN][LDS]
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int nk = (p.CI + BK - 1) / BK;
    const bool vec = (p.CI % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.w) |
                                          reinterpret_cast<uintptr_t>(p.xu)) & 15u) == 0;

    auto stage = [&](int kt, int st) {
        if (vec) {
            stage_dense_vec<BM, NT>(xs + st * BM * LDS, p.x, m0, p.B, p.CI, kt * BK, p.CI, tid);
            if (BOUND) stage_dense_vec<BM, NT>(us + st * BM * LDS, p.xu, m0, p.B, p.CI, kt * BK, p.CI, tid);
            stage_dense_vec<BN, NT>(ws + st * BN * LDS, p.w, n0, p.CO, p.CI, kt * BK, p.CI, tid);
        } else {
            stage_dense_scalar<BM, NT>(xs + st * BM * LDS, p.x, m0, p.B, p.CI, kt * BK, p.CI, tid);
            if (BOUND) stage_dense_scalar<BM, NT>(us + st * BM * LDS, p.xu, m0, p.B, p.CI, kt * BK, p.CI, tid);
            stage_dense_scalar<BN, NT>(ws + st * BN * LDS, p.w, n0, p.CO, p.CI, kt * BK, p.CI, tid);
        }
    };

    float ru[TM][TN][KMAX];                      // top list (value kernel: the only list)
    float rl[BOUND ? TM : 1][BOUND ? TN : 1][BOUND ? KMAX : 1];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++)
#pragma unroll
            for (int k = 0; k < KMAX; k++) {
                ru[i][j][k] = 0.f;
                if (BOUND) rl[i][j][k] = 0.f;
            }

    stage(0, 0);
    cp_async_commit();
    for (int kt = 0; kt < nk; kt++) {
        cp_async_wait<0>();
        __syncthreads();
        if (kt + 1 < nk) stage(kt + 1, (kt + 1) & 1);
        cp_async_commit();
        if (BOUND) {  // midpoint repair of inverted intervals, in place
            float* ld = xs + (kt & 1) * BM * LDS;
            float* ud = us + (kt & 1) * BM * LDS;
#pragma unroll
            for (int r = 0; r < BM * BK / NT; r++) {
                const int e = tid + r * NT, o = (e >> 5) * LDS + (e & 31);
                const float a = ld[o], b = ud[o];
                if (a > b) {
                    const float m = (a + b) * 0.5f;
                    ld[o] = m;
                    ud[o] = m;
                }
            }
            __syncthreads();
        }
        const float* xr = xs + (kt & 1) * BM * LDS + ty * LDS;
        const float* ur = us + (kt & 1) * BM * LDS + ty * LDS;
        const float* wr = ws + (kt & 1) * BN * LDS + tx * LDS;
        // zero padding past CI or past the last row contributes |0 - 0| = 0 (resp. t1 = t2 = 0),
        // which never changes a list that starts from zeros
#pragma unroll 1
        for (int k = 0; k < BK; k++) {
            float xv[TM], uv[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; i++) {
                xv[i] = xr[i * 16 * LDS + k];
                if (BOUND) uv[i] = ur[i * 16 * LDS + k];
            }
#pragma unroll
            for (int j = 0; j < TN; j++) wv[j] = wr[j * 16 * LDS + k];
#pragma unroll
            for (int i = 0; i < TM; i++) {
#pragma unroll
                for (int j = 0; j < TN; j++) {
                    if constexpr (BOUND) {
                        const float t1 = wv[j] - xv[i], t2 = uv[i] - wv[j];
                        const float vl = fminf(t1, t2), vu = fmaxf(t1, t2);
                        // A value that does not beat the weakest slot leaves the whole list
                        // unchanged, so the chain is only walked when some lane of the warp needs it
                        // (a warp vote keeps the branch uniform; after the first few hundred columns
                        // that is a minority of the steps).
                        if (__any_sync(0xffffffffu, vl < rl[i][j][0])) {
#pragma unroll
                            for (int s = 0; s < KMAX - 1; s++)
                                rl[i][j][s] = fminf(rl[i][j][s], fmaxf(rl[i][j][s + 1], vl));
                            rl[i][j][KMAX - 1] = fminf(rl[i][j][KMAX - 1], vl);
                        }
                        if (__any_sync(0xffffffffu, vu > ru[i][j][0])) {
#pragma unroll
                            for (int s = 0; s < KMAX - 1; s++)
                                ru[i][j][s] = fmaxf(ru[i][j][s], fminf(ru[i][j][s + 1], vu));
                            ru[i][j][KMAX - 1] = fmaxf(ru[i][j][KMAX - 1], vu);
                        }
                    } else {
                        const float v = fabsf(xv[i] - wv[j]);
                        if (__any_sync(0xffffffffu, v > ru[i][j][0])) {
#pragma unroll
                            for (int s = 0; s < KMAX - 1; s++)
                                ru[i][j][s] = fmaxf(ru[i][j][s], fminf(ru[i][j][s + 1], v));
                            ru[i][j][KMAX - 1] = fmaxf(ru[i][j][KMAX - 1], v);
                        }
                    }
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int m = m0 + ty + 16 * i;
        if (m >= p.B) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int n = n0 + tx + 16 * j;
            if (n >= p.CO) continue;
            const size_t o = (size_t)m * p.CO + n;
            if constexpr (BOUND) {
                p.y[o] = -combine<KMAX>(rl[i][j], p.K, p.q, -SNB_EPS);
                p.yu[o] = combine<KMAX>(ru[i][j], p.K, p.q, SNB_EPS);
            } else {
                p.y[o] = combine<KMAX>(ru[i][j], p.K, p.q, SNB_EPS);
            }
        }
    }
}

// Values and positions of the K largest elements: one WARP per output.  The 32 lanes look at 32
// consecutive columns of the output per step; the sorted list (ascending, K <= 25 entries of
// (value, position word)) lives one entry per lane, and its weakest value - the entry threshold -
// is a warp-uniform register.  A step is subtract, compare, one ballot; only when some lane holds a
// value above the threshold does the warp insert, hit by hit in column order: broadcast the
// candidate, count the entries it is >= to (ballot + popc), shift those down by one lane (shuffle)
// and drop it into the freed lane.  A value enters only when it beats the weakest entry and moves
// up past every entry it is >= to, so among equal values the later column ranks higher, exactly
// the reference's bubble rule (sort_neuron.cu:178-187).  Insertions happen about K (1 + ln(CI / K))
// times per output, i.e. a few dozen shuffle sequences against thousands of columns.
//
// CTA = 8 warps on a tile of 16 rows x 8 columns of outputs (warp w: rows 2w, 2w+1, all 8
// columns = 16 outputs whose list entries sit in 16 register pairs per lane); the operands of 64
// columns are staged in shared memory with cp.async, double buffered.
constexpr int SP_ROWS = 16, SP_COLS = 8, SP_KT = 64, SP_THREADS = 256, SP_OUT = 2 * SP_COLS;

// Operands of one k-tile -> shared memory: 16 rows of x and 8 rows of w, 64 columns each, zero-filled
// past the edges; 16-byte copies when the rows are 16-byte aligned, else 4-byte copies.
__device__ __forceinline__ void sp_stage(const SortParams& p, float (*xs)[SP_KT], float (*ws)[SP_KT], int kt,
                                         int m0, int n0, int tid, bool vec) {
    const int k0 = kt * SP_KT;
    if (vec) {
#pragma unroll
        for (int r = 0; r < ((SP_ROWS + SP_COLS) * SP_KT / 4 + SP_THREADS - 1) / SP_THREADS; r++) {
            const int e = tid + r * SP_THREADS, row = e / (SP_KT / 4), kq = (e % (SP_KT / 4)) * 4, k = k0 + kq;
            if (row < SP_ROWS) {
                const bool ok = m0 + row < p.B && k < p.CI;
                cp_async16(smem_u32(&xs[row][kq]), ok ? p.x + (size_t)(m0 + row) * p.CI + k : p.x, ok ? 16 : 0);
            } else if (row < SP_ROWS + SP_COLS) {
                const int c = row - SP_ROWS;
                const bool ok = n0 + c < p.CO && k < p.CI;
                cp_async16(smem_u32(&ws[c][kq]), ok ? p.w + (size_t)(n0 + c) * p.CI + k : p.w, ok ? 16 : 0);
            }
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < (SP_ROWS + SP_COLS) * SP_KT / SP_THREADS; r++) {
        const int e = tid + r * SP_THREADS, row = e / SP_KT, k = k0 + e % SP_KT;
        if (row < SP_ROWS) {
            const bool ok = m0 + row < p.B && k < p.CI;
            cp_async4(smem_u32(&xs[row][e % SP_KT]), ok ? p.x + (size_t)(m0 + row) * p.CI + k : p.x, ok ? 4 : 0);
        } else {
            const int c = row - SP_ROWS;
            const bool ok = n0 + c < p.CO && k < p.CI;
            cp_async4(smem_u32(&ws[c][e % SP_KT]), ok ? p.w + (size_t)(n0 + c) * p.CI + k : p.w, ok ? 4 : 0);
        }
    }
}

__global__ void __launch_bounds__(SP_THREADS, 4) sort_fwd_pos_kernel(const SortParams p) {
    __shared__ __align__(16) float xs[2][SP_ROWS][SP_KT];
    __shared__ __align__(16) float ws[2][SP_COLS][SP_KT];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int m0 = blockIdx.x * SP_ROWS, n0 = blockIdx.y * SP_COLS;
    const int K = p.K;
    const int nk = (p.CI + SP_KT - 1) / SP_KT;

    const bool vec = (p.CI % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.w)) & 15u) == 0;
    auto stage = [&](int kt, int st) { sp_stage(p, xs[st], ws[st], kt, m0, n0, tid, vec); };

    float val[SP_OUT], thr[SP_OUT];
    uint32_t word[SP_OUT];
#pragma unroll
    for (int o = 0; o < SP_OUT; o++) {
        val[o] = 0.f;
        thr[o] = 0.f;
        word[o] = 0u;
    }

    stage(0, 0);
    cp_async_commit();
    for (int kt = 0; kt < nk; kt++) {
        const int cur = kt & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (kt + 1 < nk) stage(kt + 1, cur ^ 1);
        cp_async_commit();
        // zero-filled padding gives |0 - 0| = 0, which never beats a threshold (>= 0)
#pragma unroll
        for (int h = 0; h < SP_KT / 32; h++) {
            const int c0 = kt * SP_KT + h * 32;
            float xv[2], wv[SP_COLS];
#pragma unroll
            for (int i = 0; i < 2; i++) xv[i] = xs[cur][2 * warp + i][h * 32 + lane];
#pragma unroll
            for (int j = 0; j < SP_COLS; j++) wv[j] = ws[cur][j][h * 32 + lane];
#pragma unroll
            for (int o = 0; o < SP_OUT; o++) {
                const float d = xv[o / SP_COLS] - wv[o % SP_COLS];
                const float v = fabsf(d);
                uint32_t hits = __ballot_sync(0xffffffffu, v > thr[o]);
                while (hits) {                                     // rare, warp-uniform
                    const int src = __ffs(hits) - 1;
                    hits &= hits - 1;
                    const float bv = __shfl_sync(0xffffffffu, v, src);
                    const float bd = __shfl_sync(0xffffffffu, d, src);
                    if (bv > thr[o]) {                             // an earlier hit may have raised it
                        const uint32_t bw = (uint32_t)(c0 + src) | (bd >= 0 ? 0u : SNB_SIGN_BIT);
                        const int cnt = __popc(__ballot_sync(0xffffffffu, lane < K && bv >= val[o]));
                        const float up_v = __shfl_down_sync(0xffffffffu, val[o], 1);
                        const uint32_t up_w = __shfl_down_sync(0xffffffffu, word[o], 1);
                        if (lane < cnt - 1) {
                            val[o] = up_v;
                            word[o] = up_w;
                        } else if (lane == cnt - 1) {
                            val[o] = bv;
                            word[o] = bw;
                        }
                        thr[o] = __shfl_sync(0xffffffffu, val[o], 0);
                    }
                }
            }
        }
    }
    const size_t plane = (size_t)p.B * p.CO;
#pragma unroll
    for (int o = 0; o < SP_OUT; o++) {
        const int m = m0 + 2 * warp + o / SP_COLS, n = n0 + o % SP_COLS;
        // the weighted sum in rank order (rank 0 = largest = lane K-1), every lane redundantly
        float ans = SNB_EPS, c = 1.0f;
        for (int r = 0; r < K; r++) {
            const float vr = __shfl_sync(0xffffffffu, val[o], K - 1 - r);
            ans += vr * c * p.q;
            c *= 1 - p.q;
        }
        if (m >= p.B || n >= p.CO) continue;
        const size_t off = (size_t)m * p.CO + n;
        if (lane == 0) p.y[off] = ans / (1 - c);
        if (lane < K) p.pos[(size_t)(K - 1 - lane) * plane + off] = (int)word[o];
    }
}

// The same algorithm for K <= 16 with one HALF-warp per output: lanes 0-15 work on row 2w, lanes
// 16-31 on row 2w+1 of the same output column, 16 columns per step each, all shuffles 16 wide.  The
// two outputs of a warp insert side by side (a round of the insertion loop serves one candidate of
// each half).
//
// Insertions are what this kernel pays for, and an online top-K makes about K (1 + ln(CI / K)) of
// them per output because its threshold starts at zero.  So the columns are swept twice.  Sweep 1
// only takes, per lane, the maximum over the lane's columns (c = hl mod 16): 16 maxima of disjoint
// column sets, i.e. 16 distinct elements, of which the K-th largest (K <= 16) is a value T0 that at
// least K elements reach - a lower bound of the final threshold.  Sweep 2 is the algorithm above
// with the entry threshold floored just below T0, so the elements that would have entered the
// list only to be pushed out again are never inserted.  Elements >= T0 meet exactly the
// comparisons they meet in the unseeded scan (anything below T0 in the list loses to them either
// way), so values, positions and the tie rules are unchanged.
__global__ void __launch_bounds__(SP_THREADS, 4) sort_fwd_pos_half_kernel(const SortParams p) {
    __shared__ __align__(16) float xs[2][SP_ROWS][SP_KT];
    __shared__ __align__(16) float ws[2][SP_COLS][SP_KT];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, half = lane >> 4, hl = lane & 15;
    const int m0 = blockIdx.x * SP_ROWS, n0 = blockIdx.y * SP_COLS;
    const int K = p.K;
    const int nk = (p.CI + SP_KT - 1) / SP_KT;

    const bool vec = (p.CI % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.w)) & 15u) == 0;
    auto stage = [&](int kt, int st) { sp_stage(p, xs[st], ws[st], kt, m0, n0, tid, vec); };

    float val[SP_COLS], thr[SP_COLS];   // entry hl of the list of output (row 2w + half, column j)
    uint32_t word[SP_COLS];
#pragma unroll
    for (int j = 0; j < SP_COLS; j++) {
        val[j] = 0.f;
        thr[j] = 0.f;
        word[j] = 0u;
    }
    const uint32_t my_half = 0xffffu << (16 * half);

    // ---- sweep 1: lane maxima -> T0 -> threshold floor ---------------------------------------
    float seed[SP_COLS];
#pragma unroll
    for (int j = 0; j < SP_COLS; j++) seed[j] = 0.f;
    stage(0, 0);
    cp_async_commit();
    for (int kt = 0; kt < nk; kt++) {
        const int cur = kt & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (kt + 1 < nk) stage(kt + 1, cur ^ 1);
        cp_async_commit();
#pragma unroll
        for (int t = 0; t < SP_KT / 16; t++) {
            const float xv = xs[cur][2 * warp + half][t * 16 + hl];
#pragma unroll
            for (int j = 0; j < SP_COLS; j++) seed[j] = fmaxf(seed[j], fabsf(xv - ws[cur][j][t * 16 + hl]));
        }
    }
#pragma unroll
    for (int j = 0; j < SP_COLS; j++) {
        // rank of this lane's maximum among the 16 of its half (ties: lower lane first)
        int rank = 0;
#pragma unroll
        for (int t = 0; t < 16; t++) {
            const float other = __shfl_sync(0xffffffffu, seed[j], t, 16);
            rank += (other > seed[j]) || (other == seed[j] && t < hl);
        }
        const uint32_t pick = __ballot_sync(0xffffffffu, rank == K - 1) & my_half;
        const float t0 = __shfl_sync(0xffffffffu, seed[j], __ffs(pick) - 1);
        // largest float below T0 (0 stays 0: nothing enters on a zero difference anyway)
        seed[j] = t0 > 0.f ? __int_as_float(__float_as_int(t0) - 1) : 0.f;
        thr[j] = seed[j];
    }
    __syncthreads();                           // everyone is done with the last tile of sweep 1

    // ---- sweep 2: the insertion scan ----------------------------------------------------------
    stage(0, 0);
    cp_async_commit();
    for (int kt = 0; kt < nk; kt++) {
        const int cur = kt & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (kt + 1 < nk) stage(kt + 1, cur ^ 1);
        cp_async_commit();
#pragma unroll 1                               // one copy of the insertion loops (instruction cache)
        for (int t = 0; t < SP_KT / 32; t++) {
            // a lane looks at two columns per step (c and c + 16); one vote on the larger magnitude
            // tells whether this output has a candidate at all
            const int c0 = kt * SP_KT + t * 32;
            const float xa = xs[cur][2 * warp + half][t * 32 + hl], xb = xs[cur][2 * warp + half][t * 32 + 16 + hl];
#pragma unroll
            for (int j = 0; j < SP_COLS; j++) {
                const float da = xa - ws[cur][j][t * 32 + hl], db = xb - ws[cur][j][t * 32 + 16 + hl];
                if (!__any_sync(0xffffffffu, fmaxf(fabsf(da), fabsf(db)) > thr[j])) continue;
                // rare, warp-uniform: the candidates of the first 16 columns in order, then the next 16
#pragma unroll 1
                for (int sub = 0; sub < 2; sub++) {
                    const float d = sub ? db : da;
                    const float v = fabsf(d);
                    uint32_t hits = __ballot_sync(0xffffffffu, v > thr[j]);
                    while (hits) {
                        const uint32_t mine = hits & my_half;
                        const int src = mine ? __ffs(mine) - 1 : lane;  // absolute lane of this half's next candidate
                        // drop the lowest candidate of each half
                        const uint32_t lo = hits & 0xffffu, hi = hits & 0xffff0000u;
                        hits = (lo & (lo - 1)) | (hi & (hi - 1));
                        const float bv = __shfl_sync(0xffffffffu, v, src);
                        const float bd = __shfl_sync(0xffffffffu, d, src);
                        const bool enter = mine != 0u && bv > thr[j];   // uniform within the half
                        const uint32_t bal = __ballot_sync(0xffffffffu, enter && hl < K && bv >= val[j]);
                        const int cnt = __popc(bal & my_half);
                        const float up_v = __shfl_down_sync(0xffffffffu, val[j], 1, 16);
                        const uint32_t up_w = __shfl_down_sync(0xffffffffu, word[j], 1, 16);
                        if (enter) {
                            if (hl < cnt - 1) {
                                val[j] = up_v;
                                word[j] = up_w;
                            } else if (hl == cnt - 1) {
                                val[j] = bv;
                                word[j] = (uint32_t)(c0 + sub * 16 + (src & 15)) | (bd >= 0 ? 0u : SNB_SIGN_BIT);
                            }
                        }
                        thr[j] = fmaxf(seed[j], __shfl_sync(0xffffffffu, val[j], 0, 16));
                    }
                }
            }
        }
    }
    const size_t plane = (size_t)p.B * p.CO;
#pragma unroll
    for (int j = 0; j < SP_COLS; j++) {
        const int m = m0 + 2 * warp + half, n = n0 + j;
        float ans = SNB_EPS, c = 1.0f;
        for (int r = 0; r < K; r++) {
            const float vr = __shfl_sync(0xffffffffu, val[j], K - 1 - r, 16);
            ans += vr * c * p.q;
            c *= 1 - p.q;
        }
        if (m >= p.B || n >= p.CO) continue;
        const size_t off = (size_t)m * p.CO + n;
        if (hl == 0) p.y[off] = ans / (1 - c);
        if (hl < K) p.pos[(size_t)(K - 1 - hl) * plane + off] = (int)word[j];
    }
}

// Sparse backward: one CTA per batch row, grad_x of the row accumulated in shared memory.
__global__ void __launch_bounds__(256) sort_bwd_kernel(const float* __restrict__ g, const int* __restrict__ pos,
                                                       int B, int CO, int CI, int K, float q, float c0,
                                                       float* __restrict__ gx, float* __restrict__ gw,
                                                       int use_smem) {
    extern __shared__ float row[];
    const int b = blockIdx.x;
    float* acc = use_smem ? row : gx + (size_t)b * CI;
    if (use_smem) {
        for (int c = threadIdx.x; c < CI; c += blockDim.x) row[c] = 0.f;
        __syncthreads();
    }
    const size_t plane = (size_t)B * CO;
    for (int j = threadIdx.x; j < CO; j += blockDim.x) {
        const size_t o = (size_t)b * CO + j;
        const float grad = g[o];
        float c = c0;
        for (int k = 0; k < K; k++) {
            const uint32_t pw = (uint32_t)pos[(size_t)k * plane + o];
            const int i = (int)(pw & ~SNB_SIGN_BIT);
            const float v = ((pw & SNB_SIGN_BIT) ? -grad : grad) * c * q;
            atomicAdd(acc + i, v);
            if (gw) atomicAdd(gw + (size_t)j * CI + i, -v);
            c *= 1 - q;
        }
    }
    if (use_smem) {
        __syncthreads();
        for (int c = threadIdx.x; c < CI; c += blockDim.x) gx[(size_t)b * CI + c] = row[c];
    }
}

template <int KMAX, bool BOUND>
static cudaError_t launch_sort_fwd(const SortParams& p, cudaStream_t st) {
    constexpr int BM = 32, BN = (BOUND || KMAX <= 10) ? 32 : 64;
    constexpr int SMEM = 2 * ((BOUND ? 2 : 1) * BM + BN) * LDS * (int)sizeof(float);
    auto kern = sort_fwd_kernel<KMAX, BOUND>;
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        configured[dev & 63].store(true, std::memory_order_release);
    }
    dim3 grid((p.B + BM - 1) / BM, (p.CO + BN - 1) / BN);
    kern<<<grid, 256, SMEM, st>>>(p);
    return cudaGetLastError();
}

}  // namespace snb

using namespace snb;

static int check_sort(const void* x, const void* w, const void* y, int B, int CO, int CI, int G, int HW,
                      float q, int K) {
    if (!x || !w || !y) return SNB_ERR_NULL_POINTER;
    if (G != 1 || HW != 1 || K < 2 || K > 25 || !(q > 0.f) || !(q < 1.f)) return SNB_ERR_UNSUPPORTED;
    if (B <= 0 || CO <= 0 || CI <= 0 || K > CI) return SNB_ERR_BAD_SHAPE;
    if ((long long)CO * CI >= (1ll << 31) || (long long)B * CO * K >= (1ll << 31) || (long long)B * CI >= (1ll << 31))
        return SNB_ERR_TOO_LARGE;
    return SNB_OK;
}

extern "C" int snb_sort_neuron_forward_nograd(const float* x, const float* w, int B, int CO, int CI, int G,
                                              int HW, float* y, float q, int K, void* stream) {
    if ((G != 1 || HW != 1) && q > 0.f && q < 1.f)
        return general_sort_forward(x, w, B, CO, CI, G, HW, y, nullptr, q, K, (cudaStream_t)stream);
    int rc = check_sort(x, w, y, B, CO, CI, G, HW, q, K);
    if (rc) return rc;
    SortParams p{x, x, w, y, nullptr, nullptr, B, CO, CI, K, q};
    SNB_CUDA(K <= 10 ? launch_sort_fwd<10, false>(p, (cudaStream_t)stream)
                     : launch_sort_fwd<25, false>(p, (cudaStream_t)stream));
    return SNB_OK;
}

extern "C" int snb_sort_neuron_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                                       float* y, int* pos, float q, int K, void* stream) {
    if ((G != 1 || HW != 1) && q > 0.f && q < 1.f) {
        if (!pos) return SNB_ERR_NULL_POINTER;
        return general_sort_forward(x, w, B, CO, CI, G, HW, y, pos, q, K, (cudaStream_t)stream);
    }
    int rc = check_sort(x, w, y, B, CO, CI, G, HW, q, K);
    if (rc) return rc;
    if (!pos) return SNB_ERR_NULL_POINTER;
    SortParams p{x, x, w, y, nullptr, pos, B, CO, CI, K, q};
    dim3 grid((B + SP_ROWS - 1) / SP_ROWS, (CO + SP_COLS - 1) / SP_COLS);
    if (K <= 16) sort_fwd_pos_half_kernel<<<grid, SP_THREADS, 0, (cudaStream_t)stream>>>(p);
    else sort_fwd_pos_kernel<<<grid, SP_THREADS, 0, (cudaStream_t)stream>>>(p);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

extern "C" int snb_bound_sort_neuron_forward(const float* xl, const float* xu, const float* w, int B, int CO,
                                             int CI, int G, int HW, float* yl, float* yu, float q, int K,
                                             void* stream) {
    if ((G != 1 || HW != 1) && q > 0.f && q < 1.f)
        return general_sort_bound_forward(xl, xu, w, B, CO, CI, G, HW, yl, yu, q, K, (cudaStream_t)stream);
    int rc = check_sort(xl, w, yl, B, CO, CI, G, HW, q, K);
    if (rc) return rc;
    if (!xu || !yu) return SNB_ERR_NULL_POINTER;
    SortParams p{xl, xu, w, yl, yu, nullptr, B, CO, CI, K, q};
    SNB_CUDA(K <= 10 ? launch_sort_fwd<10, true>(p, (cudaStream_t)stream)
                     : launch_sort_fwd<25, true>(p, (cudaStream_t)stream));
    return SNB_OK;
}

static int sort_backward(const float* g, const int* pos, int B, int CO, int CI, int G, int HW, float* gx,
                         float* gw, float q, int K, cudaStream_t st) {
    if ((G != 1 || HW != 1) && q > 0.f && q < 1.f)
        return general_sort_backward(g, pos, B, CO, CI, G, HW, gx, gw, q, K, st);
    if (!g || !pos || !gx) return SNB_ERR_NULL_POINTER;
    if (G != 1 || HW != 1 || K < 2 || K > 25 || !(q > 0.f) || !(q < 1.f)) return SNB_ERR_UNSUPPORTED;
    if (B <= 0 || CO <= 0 || CI <= 0) return SNB_ERR_BAD_SHAPE;
    if ((long long)CO * CI >= (1ll << 31) || (long long)B * CO * K >= (1ll << 31)) return SNB_ERR_TOO_LARGE;
    if (gw) SNB_CUDA(cudaMemsetAsync(gw, 0, sizeof(float) * (size_t)CO * CI, st));
    const int use_smem = (size_t)CI * sizeof(float) <= 48 * 1024;
    if (!use_smem) SNB_CUDA(cudaMemsetAsync(gx, 0, sizeof(float) * (size_t)B * CI, st));
    float n = powf(1 - q, (float)K);
    n = 1.0f + n / (1.0f - n);
    sort_bwd_kernel<<<B, 256, use_smem ? CI * sizeof(float) : 0, st>>>(g, pos, B, CO, CI, K, q, n, gx, gw, use_smem);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

extern "C" int snb_sort_neuron_backward_input(const float* grad_output, const int* pos, int B, int CO, int CI,
                                              int G, int HW, float* grad_input, float q, int K, void* stream) {
    return sort_backward(grad_output, pos, B, CO, CI, G, HW, grad_input, nullptr, q, K, (cudaStream_t)stream);
}

extern "C" int snb_sort_neuron_backward_input_weight(const float* grad_output, const int* pos, int B, int CO,
                                                     int CI, int G, int HW, float* grad_input,
                                                     float* grad_weight, float q, int K, void* stream) {
    if (!grad_weight) return SNB_ERR_NULL_POINTER;
    return sort_backward(grad_output, pos, B, CO, CI, G, HW, grad_input, grad_weight, q, K, (cudaStream_t)stream);
}
