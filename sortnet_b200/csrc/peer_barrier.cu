// Stream-ordered barrier between the ranks of one NVLink node, with a bounded wait.
//
// The data-parallel step exchanges gradients and parameters through peer memory (dp_step.cu,
// adamw.cu) and needs two orderings per step: "every rank's backward has written its gradients"
// before anyone reads them, and "every rank's new parameter shard has landed" before the next
// forward.  The reference gets both from DistributedDataParallel / NCCL (main.py:402).  Here one
// tiny kernel per rank does it on the caller's stream: thread r stores this barrier's epoch into
// rank r's flag word for this rank (a release store at system scope, through the peer mapping)
// and then polls this rank's own flag word for rank r (relaxed loads of local memory every 2 us,
// one acquire fence at the end) until it holds that epoch or a later one.
//
// The wait is bounded: after `timeout_ns` of the GPU's nanosecond timer the thread writes
// 1 + r into *status (a word the host can read, e.g. pinned host memory) and the kernel returns
// normally, so a rank that never arrives costs its peers one time-out, not a hung or trapped
// GPU; the context stays usable and the host decides what to do.  One process per GPU: the
// kernels that wait on one another always run on different devices.
#include "common.cuh"
#include "launch.h"

#define SNB_MAX_PEERS 16

namespace snb {

struct FlagPtrs {
    unsigned int* f[SNB_MAX_PEERS];   // f[r] = rank r's flag array [world], mapped into this process
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

enum { PEER_SIGNAL = 1, PEER_WAIT = 2 };

__global__ void __launch_bounds__(32) peer_barrier_kernel(const FlagPtrs fp, int rank, int world, unsigned int epoch,
                                                          unsigned long long timeout_ns, int* status, int what) {
    const int r = threadIdx.x;
    if (r >= world || r == rank) return;
    if (what & PEER_SIGNAL) {
        // everything this GPU wrote before this kernel (earlier kernels and copies of the stream) is
        // ordered before the signal
        __threadfence_system();
        unsigned int* remote = fp.f[r] + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    }
    if (!(what & PEER_WAIT)) return;
    const unsigned int* mine = fp.f[rank] + r;
    const unsigned long long t0 = global_timer_ns();
    unsigned int spins = 0;
    // The poll is a relaxed load every 2 us; the acquire fence comes once, after the flag has been
    // seen.  Waiting is still not free for the kernels of other streams: measured on B200, the
    // persistent distance kernels running beside a waiting barrier kernel lose about half of the
    // time it waits (3 ms of waiting cost the interval-bound pass 1.7 ms, whatever the polling
    // rate).  Hence the split entry points below: signal early, wait late, when the peers have
    // long signalled and the wait returns at once.
    for (;;) {
        unsigned int seen;
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if ((int)(seen - epoch) >= 0) {                              // wrap-safe "seen >= epoch"
            __threadfence_system();                                  // acquire: later reads see the peer's writes
            return;
        }
        if ((++spins & 15u) == 0 && global_timer_ns() - t0 > timeout_ns) break;
        __nanosleep(2000);
    }
    atomicExch(status, 1 + r);                                       // gave up on rank r
}

}  // namespace snb

using namespace snb;

static int launch_peer(void* const* flag_ptrs, int rank, int world, unsigned int epoch, unsigned long long timeout_ns,
                       int* status, int what, void* stream) {
    if (!flag_ptrs || ((what & PEER_WAIT) && !status)) return SNB_ERR_NULL_POINTER;
    if (world < 1 || world > SNB_MAX_PEERS || rank < 0 || rank >= world) return SNB_ERR_UNSUPPORTED;
    FlagPtrs fp;
    for (int r = 0; r < SNB_MAX_PEERS; r++) fp.f[r] = nullptr;
    for (int r = 0; r < world; r++) {
        if (!flag_ptrs[r]) return SNB_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(flag_ptrs[r]) & 3u) return SNB_ERR_ALIGNMENT;
        fp.f[r] = static_cast<unsigned int*>(flag_ptrs[r]);
    }
    if (world == 1) return SNB_OK;
    peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(fp, rank, world, epoch, timeout_ns, status, what);
    SNB_CUDA(cudaGetLastError());
    return SNB_OK;
}

// flag_ptrs: `world` pointers (host array) to the ranks' flag arrays of `world` 32-bit words each,
// zero-initialised, entry `rank` this GPU's own (symmetric memory or any peer mapping).  `epoch`
// must grow by one with every barrier on these flags (all ranks pass the same value).  `status`:
// device-accessible int, 0 while all waits have succeeded.
extern "C" int snb_peer_barrier(void* const* flag_ptrs, int rank, int world, unsigned int epoch,
                                unsigned long long timeout_ns, int* status, void* stream) {
    return launch_peer(flag_ptrs, rank, world, epoch, timeout_ns, status, PEER_SIGNAL | PEER_WAIT, stream);
}

// The two halves of snb_peer_barrier as separate stream-ordered operations: "this rank has reached
// epoch" and "wait until every rank has".  A barrier is signal + wait with the same epoch.
extern "C" int snb_peer_signal(void* const* flag_ptrs, int rank, int world, unsigned int epoch, void* stream) {
    return launch_peer(flag_ptrs, rank, world, epoch, 0, nullptr, PEER_SIGNAL, stream);
}

extern "C" int snb_peer_wait(void* const* flag_ptrs, int rank, int world, unsigned int epoch,
                             unsigned long long timeout_ns, int* status, void* stream) {
    return launch_peer(flag_ptrs, rank, world, epoch, timeout_ns, status, PEER_WAIT, stream);
}
