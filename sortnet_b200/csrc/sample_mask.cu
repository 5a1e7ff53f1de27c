// Kept-channel lists for the masked training step: `lists` independent uniformly random subsets of
// {0 .. channels-1}, each of exactly `count` elements, written in ascending order as int32.
//
// Replaces the mask sampler of zbh2047/SortNet core/models/norm_dist.py:14-17 (uniform scores,
// top-k, cast: a segmented radix sort plus several element-wise launches per layer in PyTorch; no
// native counterpart there).  Same distribution: every channel of a list draws an independent
// 32-bit key and the `count` smallest keys are kept, which is a uniformly random subset.  One CTA
// per list does everything in shared memory:
//   1. keys from the Philox-4x32-10 counter-based generator (Salmon et al., SC'11), counter =
//      (channel / 4, list), key = (seed lo, seed hi) - reproducible for a given seed whatever the grid;
//   2. radix select of the count-th smallest key (four 8-bit passes over a 256-bin histogram);
//   3. stream compaction in channel order (CTA-wide prefix sum), which leaves the list sorted;
//      keys equal to the threshold are taken in channel order until the count is reached.
#include "common.cuh"
#include "launch.h"

namespace snb {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint32_t lo0 = 0xD2511F53u * c[0], hi0 = __umulhi(0xD2511F53u, c[0]);
    const uint32_t lo1 = 0xCD9E8D57u * c[2], hi1 = __umulhi(0xCD9E8D57u, c[2]);
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0;
    c[1] = lo1;
    c[2] = n2;
    c[3] = lo0;
}

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; r++) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

constexpr int SM_THREADS = 512;

// Exclusive prefix sum of one value per thread over the CTA; *total gets the sum.
__device__ __forceinline__ int cta_exclusive_scan(int v, int* warp_sums, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = lane < SM_THREADS / 32 ? warp_sums[lane] : 0;
        int wi = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, wi, d);
            if (lane >= d) wi += n;
        }
        if (lane < SM_THREADS / 32) warp_sums[lane] = wi - w;
        if (lane == 31) *total = wi;
    }
    __syncthreads();
    const int r = warp_sums[warp] + incl - v;
    __syncthreads();
    return r;
}

// One list by one CTA (see the file header); `list` is the list's number within its call, which
// enters the random counter.
__device__ __forceinline__ void sample_one_list(int* __restrict__ out, int channels, int count, uint32_t seed_lo,
                                                uint32_t seed_hi, int list) {
    extern __shared__ uint32_t keys[];  // [channels rounded up to 4]
    __shared__ int hist[256];
    __shared__ int warp_sums[SM_THREADS / 32];
    __shared__ int s_total;
    __shared__ uint32_t s_prefix;
    __shared__ int s_need;
    const int tid = threadIdx.x;
    for (int q = tid; q * 4 < channels; q += SM_THREADS) {
        uint32_t c[4] = {(uint32_t)q, (uint32_t)list, 0u, 0u};
        philox4x32_10(c, seed_lo, seed_hi);
#pragma unroll
        for (int k = 0; k < 4; k++) keys[q * 4 + k] = c[k];
    }
    if (tid == 0) {
        s_prefix = 0u;
        s_need = count;  // rank (1-based) of the threshold key among the keys that match the prefix
    }
    __syncthreads();
    // radix select, most significant byte first
    for (int pass = 0; pass < 4; pass++) {
        const int shift = 24 - 8 * pass;
        const uint32_t mask_hi = pass == 0 ? 0u : 0xffffffffu << (shift + 8);
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (int c = tid; c < channels; c += SM_THREADS) {
            const uint32_t k = keys[c];
            if ((k & mask_hi) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int need = s_need, bin = 0;
            while (bin < 255 && need > hist[bin]) {
                need -= hist[bin];
                bin++;
            }
            s_need = need;
            s_prefix = prefix | ((uint32_t)bin << shift);
        }
        __syncthreads();
    }
    const uint32_t threshold = s_prefix;  // the count-th smallest key
    const int ties_wanted = s_need;       // how many keys equal to it belong to the subset
    // compaction in channel order: thread t owns the contiguous channel range [t*per, (t+1)*per)
    const int per = (channels + SM_THREADS - 1) / SM_THREADS;
    const int c0 = tid * per, c1 = min(channels, c0 + per);
    int n_less = 0, n_equal = 0;
    for (int c = c0; c < c1; c++) {
        const uint32_t k = keys[c];
        n_less += k < threshold;
        n_equal += k == threshold;
    }
    const int equal_before = cta_exclusive_scan(n_equal, warp_sums, &s_total);
    int take_equal = min(max(ties_wanted - equal_before, 0), n_equal);
    int pos = cta_exclusive_scan(n_less + take_equal, warp_sums, &s_total);
    int* dst = out + (size_t)list * count;
    for (int c = c0; c < c1; c++) {
        const uint32_t k = keys[c];
        bool keep = k < threshold;
        if (k == threshold && take_equal > 0) {
            keep = true;
            take_equal--;
        }
        if (keep && pos < count) dst[pos++] = c;
    }
}

__global__ void __launch_bounds__(SM_THREADS) sample_mask_kernel(int* __restrict__ out, int channels, int count,
                                                                 uint32_t seed_lo, uint32_t seed_hi) {
    sample_one_list(out, channels, count, seed_lo, seed_hi, blockIdx.x);
}

// Several independent calls of the kernel above in one launch (the masks of all layers of a model
// for one step): CTA b makes list b % lists of job b / lists, with that job's seed, so every job's
// lists are the ones its own snb_sample_mask call would have produced.
constexpr int SAMPLE_MAX_JOBS = 16;
struct SampleJobs {
    int* out[SAMPLE_MAX_JOBS];
    int channels[SAMPLE_MAX_JOBS];
    int count[SAMPLE_MAX_JOBS];
    uint32_t seed_lo[SAMPLE_MAX_JOBS];
    uint32_t seed_hi[SAMPLE_MAX_JOBS];
};

__global__ void __launch_bounds__(SM_THREADS) sample_mask_batch_kernel(const SampleJobs jobs, int lists) {
    const int job = blockIdx.x / lists, list = blockIdx.x % lists;
    // compile-time indices keep the job table in the parameter bank
    int* out = nullptr;
    int channels = 0, count = 0;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < SAMPLE_MAX_JOBS; j++)
        if (j == job) {
            out = jobs.out[j];
            channels = jobs.channels[j];
            count = jobs.count[j];
            lo = jobs.seed_lo[j];
            hi = jobs.seed_hi[j];
        }
    sample_one_list(out, channels, count, lo, hi, list);
}

// Validation of caller-made index lists (debug aid): bit 0 = an entry outside [0, channels),
// bit 1 = a list that is not strictly ascending.
__device__ int snb_index_check_bits;

__global__ void check_index_kernel(const int* __restrict__ idx, long long n, int count, int channels) {
    int bits = 0;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int v = idx[i];
        if (v < 0 || v >= channels) bits |= 1;
        if (i % count != 0 && idx[i - 1] >= v) bits |= 2;
    }
    if (bits) atomicOr(&snb_index_check_bits, bits);
}

}  // namespace snb

using namespace snb;

// index [lists, count] int32 (the [S, G, count] lists of one operand flattened): checks that every
// entry lies in [0, channels) and whether every list is strictly ascending.  Copies the result
// back and synchronises `stream`, so it is meant for debugging, not for the training loop.
// *flags (host, optional) receives bit 0 = out of range, bit 1 = not ascending.
extern "C" int snb_check_index_lists(const int* index, int lists, int count, int channels, int* flags, void* stream) {
    if (!index) return SNB_ERR_NULL_POINTER;
    if (lists <= 0 || count <= 0 || channels <= 0) return SNB_ERR_BAD_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    int bits = 0;
    SNB_CUDA(cudaMemcpyToSymbolAsync(snb_index_check_bits, &bits, sizeof(int), 0, cudaMemcpyHostToDevice, st));
    const long long n = (long long)lists * count;
    const int blocks = (int)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
    check_index_kernel<<<blocks, 256, 0, st>>>(index, n, count, channels);
    SNB_CUDA(cudaGetLastError());
    SNB_CUDA(cudaMemcpyFromSymbolAsync(&bits, snb_index_check_bits, sizeof(int), 0, cudaMemcpyDeviceToHost, st));
    SNB_CUDA(cudaStreamSynchronize(st));
    if (flags) *flags = bits;
    return (bits & 1) ? SNB_ERR_INDEX_RANGE : SNB_OK;
}

static int configure_sampler() {
    static std::atomic<bool> configured[64];
    int dev = 0;
    SNB_CUDA(cudaGetDevice(&dev));
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        SNB_CUDA(cudaFuncSetAttribute(sample_mask_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        SNB_CUDA(cudaFuncSetAttribute(sample_mask_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured[dev & 63].store(true, std::memory_order_release);
    }
    return SNB_OK;
}

// `jobs` calls of snb_sample_mask in one launch: outs[j] receives `lists` lists of counts[j] kept
// channels out of channels[j], drawn with seeds[j] (host arrays).  Same lists as the separate calls.
extern "C" int snb_sample_mask_batch(int jobs, int* const* outs, const int* channels, const int* counts,
                                     const unsigned long long* seeds, int lists, void* stream) {
    if (!outs || !channels || !counts || !seeds) return SNB_ERR_NULL_POINTER;
    if (jobs <= 0 || lists <= 0) return SNB_ERR_BAD_SHAPE;
    if (jobs > SAMPLE_MAX_JOBS) return SNB_ERR_UNSUPPORTED;
    SampleJobs table{};
    size_t smem = 0;
    for (int j = 0; j < jobs; j++) {
        if (!outs[j]) return SNB_ERR_NULL_POINTER;
        if (channels[j] <= 0 || counts[j] <= 0 || counts[j] > channels[j]) return SNB_ERR_BAD_SHAPE;
        const size_t need = sizeof(uint32_t) * (size_t)((channels[j] + 3) / 4 * 4);
        if (need > 200 * 1024) return SNB_ERR_TOO_LARGE;
        smem = need > smem ? need : smem;
        table.out[j] = outs[j];
        table.channels[j] = channels[j];
        table.count[j] = counts[j];
        table.seed_lo[j] = (uint32_t)seeds[j];
        table.seed_hi[j] = (uint32_t)(seeds[j] >> 32);
    }
    int rc = configure_sampler();
    if (rc) return rc;
    sample_mask_batch_kernel<<<jobs * lists, SM_THREADS, smem, (cudaStream_t)stream>>>(table, lists);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

extern "C" int snb_sample_mask(int* out, int lists, int channels, int count, unsigned long long seed,
                               void* stream) {
    if (!out) return SNB_ERR_NULL_POINTER;
    if (lists <= 0 || channels <= 0 || count <= 0 || count > channels) return SNB_ERR_BAD_SHAPE;
    const size_t smem = sizeof(uint32_t) * (size_t)((channels + 3) / 4 * 4);
    if (smem > 200 * 1024) return SNB_ERR_TOO_LARGE;  // 51200 channels
    int rc = configure_sampler();
    if (rc) return rc;
    sample_mask_kernel<<<lists, SM_THREADS, smem, (cudaStream_t)stream>>>(out, channels, count, (uint32_t)seed,
                                                                         (uint32_t)(seed >> 32));
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}
