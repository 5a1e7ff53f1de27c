// Tile geometry and global->shared staging shared by the max-plus "GEMM-shaped" kernels.
//
// A CTA of WM x WN warps owns a (32*WM) x (64*WN) tile of outputs.  Each warp owns 32 x 64,
// each thread 8 x 8 (rows tb + 4*i, columns tj + 8*j with tb = lane / 8, tj = lane % 8), and
// walks the reduction axis in k-tiles of 32 staged in shared memory as [row][36] floats:
// the 4-float pad makes the eight 16-byte fragments a quarter-warp reads fall in distinct
// banks.  Two stages, filled with cp.async one k-tile ahead.
#pragma once
#include "common.cuh"

namespace snb {

constexpr int BK = 32;
constexpr int LDS = 36;  // shared-memory row stride in floats

// Dense rows, 16-byte copies.  Requires ld % 4 == 0 and a 16-byte aligned base.
template <int ROWS, int NT>
__device__ __forceinline__ void stage_dense_vec(float* s, const float* __restrict__ g, int row0,
                                                int nrows, int ld, int k0, int K, int tid) {
    constexpr int CHUNKS = ROWS * (BK / 4);
    static_assert(CHUNKS % NT == 0, "tile/threads mismatch");
#pragma unroll
    for (int r = 0; r < CHUNKS / NT; r++) {
        int c = tid + r * NT;
        int row = c >> 3, kc = (c & 7) * 4;
        bool ok = (row0 + row < nrows) && (k0 + kc < K);
        const float* src = ok ? g + (size_t)(row0 + row) * ld + k0 + kc : g;
        cp_async16(smem_u32(s + row * LDS + kc), src, ok ? 16 : 0);
    }
}

// Dense rows, 4-byte copies (any alignment, any K).
template <int ROWS, int NT>
__device__ __forceinline__ void stage_dense_scalar(float* s, const float* __restrict__ g, int row0,
                                                   int nrows, int ld, int k0, int K, int tid) {
    constexpr int PASSES = ROWS * BK / NT;
    const int lane = tid & 31, w = tid >> 5;
    const bool kok = k0 + lane < K;
#pragma unroll
    for (int r = 0; r < PASSES; r++) {
        int row = w + r * (NT / 32);
        bool ok = kok && (row0 + row < nrows);
        const float* src = ok ? g + (size_t)(row0 + row) * ld + k0 + lane : g;
        cp_async4(smem_u32(s + row * LDS + lane), src, ok ? 4 : 0);
    }
}

// Rows and columns of W picked through per-sub-batch index lists.  Eight lanes walk eight
// consecutive kept columns of one row (one 32-byte sector when the kept columns are
// adjacent); every thread keeps the element offsets of its ROWS / (NT / 8) rows in registers.
template <int ROWS, int NT>
struct GatherW {
    static_assert(NT == 64 || NT == 128 || NT == 256, "group_row assumes 2, 4 or 8 warps");
    static constexpr int RPT = ROWS / (NT / 8);
    int rowoff[RPT];  // element offset of the row start in W, or -1 past the last row
    int col[4];       // W column of this thread's four k positions in the next k-tile, or -1

    // Row of the tile handled by 8-lane group `grp` in pass 0.  The four groups of a warp take
    // rows two apart (bank offset 8 words with the 36-float stride), so the 32 four-byte
    // shared-memory writes of one warp instruction hit 32 distinct banks.
    __device__ __forceinline__ static int group_row(int tid) {
        const int w = tid >> 5, g = (tid >> 3) & 3;
        return 2 * g + (w & 1) + 8 * (w >> 1);
    }
    __device__ __forceinline__ void init_rows(const int* __restrict__ co_s, int n0, int CO,
                                              int W_CI, int tid) {
        const int r0 = group_row(tid);
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            int n = n0 + r0 + (NT / 8) * i;
            rowoff[i] = n < CO ? (co_s ? co_s[n] : n) * W_CI : -1;
        }
    }
    __device__ __forceinline__ void fetch_cols(const int* __restrict__ ci_s, int k0, int K, int tid) {
        const int l8 = tid & 7;
#pragma unroll
        for (int m = 0; m < 4; m++) {
            int k = k0 + l8 + 8 * m;
            col[m] = k < K ? (ci_s ? ci_s[k] : k) : -1;
        }
    }
    __device__ __forceinline__ void stage(float* s, const float* __restrict__ w, int tid) const {
        const int r0 = group_row(tid), l8 = tid & 7;
#pragma unroll
        for (int i = 0; i < RPT; i++) {
#pragma unroll
            for (int m = 0; m < 4; m++) {
                bool ok = (rowoff[i] >= 0) && (col[m] >= 0);
                const float* src = ok ? w + rowoff[i] + col[m] : w;
                cp_async4(smem_u32(s + (r0 + (NT / 8) * i) * LDS + l8 + 8 * m), src, ok ? 4 : 0);
            }
        }
    }
};

// Rows of W picked through a per-sub-batch index list, all columns of each row: 16-byte copies
// along the row like stage_dense_vec (requires W_CI % 4 == 0 and a 16-byte aligned base).  Every
// thread keeps the element offsets of the ROWS / (NT / 8) rows it copies from in registers.
template <int ROWS, int NT>
struct RowVecW {
    static constexpr int RPT = ROWS / (NT / 8);
    int rowoff[RPT];  // element offset of the row start in W, or -1 past the last row

    __device__ __forceinline__ void init_rows(const int* __restrict__ co_s, int n0, int CO, int W_CI, int tid) {
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            const int n = n0 + (tid >> 3) + (NT / 8) * i;
            rowoff[i] = n < CO ? (co_s ? co_s[n] : n) * W_CI : -1;
        }
    }
    __device__ __forceinline__ void stage(float* s, const float* __restrict__ w, int k0, int K, int tid) const {
        const int kc = (tid & 7) * 4;
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            const bool ok = rowoff[i] >= 0 && k0 + kc < K;
            const float* src = ok ? w + rowoff[i] + k0 + kc : w;
            cp_async16(smem_u32(s + ((tid >> 3) + (NT / 8) * i) * LDS + kc), src, ok ? 16 : 0);
        }
    }
};

}  // namespace snb

namespace snb {

// Stream-K style work split for kernels whose partial results merge exactly (max / min):
// the (tile, k-tile) pairs of the whole problem are laid out as one sequence and cut into
// gridDim.x equal ranges, so every CTA does the same amount of work whatever the tile count.
// A CTA's range may start and end in the middle of a tile; such partial tiles are merged
// into the output with integer atomicMax on the (non-negative) float bit patterns.
struct StreamK {
    int tiles_m, tiles_n, nk;  // tile grid and k-tiles per tile
    __device__ __forceinline__ long long total() const { return (long long)tiles_m * tiles_n * nk; }
    __device__ __forceinline__ void range(long long& u0, long long& u1) const {
        const long long t = total();
        u0 = t * blockIdx.x / gridDim.x;
        u1 = t * (blockIdx.x + 1) / gridDim.x;
    }
};

// atomicMax for non-negative floats through their integer ordering.
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
    atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

}  // namespace snb
