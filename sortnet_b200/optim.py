"""Flat-buffer training state: parameters, gradients and AdamW moments in four flat fp32 buffers.

Why: (1) the data-parallel gradient exchange becomes ONE all-reduce of one buffer instead of one
per parameter; (2) the optimiser is one fused kernel (`snb_adamw_step`, 28 bytes of HBM traffic
per parameter); (3) the backward kernels write `grad_weight` straight into their slice of the
flat gradient buffer, so no gradient is copied or accumulated by autograd.

The reference uses torch.optim.AdamW on ordinary parameters behind DistributedDataParallel
(main.py:402,429-432); parameter names, shapes and values are unchanged here (each parameter
becomes a view into the flat buffer), so state_dicts stay interchangeable.
"""
import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib
from . import norm_dist_cuda as _C

# Only plain peer loads, stores and copies are used here: keep symmetric memory off the NVLink
# multicast objects (a rank that dies while bound to one disturbs its peers' GPUs).
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


def _pad4(n):
    return (n + 3) // 4 * 4


def shard_bounds(numel, world, rank):
    """[lo, hi) of rank's shard of a flat buffer of `numel` (multiple of 4) elements; every bound
    is a multiple of 4 and the shards tile the buffer."""
    quads = numel // 4
    per = (quads + world - 1) // world
    lo = min(rank * per, quads)
    hi = min(lo + per, quads)
    return lo * 4, hi * 4


class FlatAdamW:
    """AdamW over all parameters of `module` held in flat buffers.

    After construction every parameter's `.data` is a view into `self.flat_param` and every
    parameter carries `grad_sink`, a view into `self.flat_grad`: the operators of
    `sortnet_b200.ops` write the weight gradient there during backward and hand `None` to autograd
    (see ops._dist_backward); parameters of other modules get ordinary `.grad` tensors, which
    `gather_grads()` copies into the flat buffer.  One weight-decay value for all parameters
    (the reference uses 0 for every norm-distance weight).
    """

    def __init__(self, module, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=0.0, process_group=None,
                 peer_memory=False, overlap=False, barrier_timeout_s=10.0):
        """peer_memory=True (ranks of one NVLink node): the flat gradient and parameter buffers are
        allocated as symmetric memory and `step()` runs the fused reduce-scatter + AdamW +
        all-gather kernel over peer pointers instead of an NCCL all-reduce plus a local update;
        each rank then keeps AdamW moments for its 1/world shard only.

        overlap=True (with peer_memory): the exchange runs beside other work of the step.
        `begin_exchange()` queues, on a side stream, device-to-device copies of this rank's shard of
        every peer's gradients (copy engines over NVLink, no SM time); `apply_update()` runs the
        local sum + AdamW kernel on the caller's stream between two of its kernels and lets the side
        stream copy the updated shard into every peer's *second* parameter buffer;
        `end_exchange()` makes the main stream wait for that and switches the parameters to the
        second buffer.  Kernels launched in between (the interval-bound pass) keep reading the old
        values.

        Ranks are ordered by `snb_peer_barrier` kernels on the exchange's stream.  Their wait is
        bounded by `barrier_timeout_s`: a rank that does not arrive makes its peers' barrier give up
        and record which rank was missing; `check()` (called by `end_exchange()` / `step()` and by
        whoever reads results back) turns that record into an exception.  Nothing traps or hangs."""
        self.params = [p for p in module.parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters")
        dev = self.params[0].device
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.step_count = 0
        offsets, total = [], 0
        for p in self.params:
            offsets.append(total)
            total += _pad4(p.numel())          # every slice starts 16-byte aligned
        self.numel = total
        self.peer = bool(peer_memory) and self.world > 1
        if self.peer:
            import torch.distributed._symmetric_memory as symm_mem
            group = process_group if process_group is not None else dist.group.WORLD
            self.flat_param = symm_mem.empty(total, dtype=torch.float32, device=dev)
            self.flat_grad = symm_mem.empty(total, dtype=torch.float32, device=dev)
            self.flat_param.zero_()
            self.flat_grad.zero_()
            self._hdl_param = symm_mem.rendezvous(self.flat_param, group)
            self._hdl_grad = symm_mem.rendezvous(self.flat_grad, group)
            self.rank = self._hdl_grad.rank
            assert self._hdl_grad.world_size == self.world
            arr = ctypes.c_void_p * self.world
            self._grad_ptrs = arr(*[int(q) for q in self._hdl_grad.buffer_ptrs])
            self._param_ptrs = arr(*[int(q) for q in self._hdl_param.buffer_ptrs])
            self.lo, self.hi = shard_bounds(total, self.world, self.rank)
            moments = max(self.hi - self.lo, 4)
            self.overlap = bool(overlap)
            # barrier state: one 32-bit flag per peer in symmetric memory, an epoch counter that all
            # ranks advance in step, and a status word in pinned host memory that the barrier kernel
            # writes when it gives up (read by check() without synchronising)
            self._flags = symm_mem.empty(max(self.world, 4), dtype=torch.int32, device=dev)
            self._flags.zero_()
            self._hdl_flags = symm_mem.rendezvous(self._flags, group)
            self._flag_ptrs = arr(*[int(q) for q in self._hdl_flags.buffer_ptrs])
            self._epoch = 0
            self._timeout_ns = int(barrier_timeout_s * 1e9)
            self._status = torch.zeros(1, dtype=torch.int32).pin_memory()
            torch.cuda.synchronize(dev)
            dist.barrier(group)                       # every rank's flags are zero before anyone signals
            for ptr in list(self._grad_ptrs) + list(self._param_ptrs):
                if not ptr or ptr % 16:
                    raise ValueError("peer buffers must be non-null and 16-byte aligned")
            if self.overlap:
                self._setup_overlap(symm_mem, group, total, dev)
        else:
            self.flat_param = torch.zeros(total, device=dev, dtype=torch.float32)
            self.flat_grad = torch.zeros(total, device=dev, dtype=torch.float32)
            moments = total
            self.overlap = False
        self.exp_avg = torch.zeros(moments, device=dev, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(moments, device=dev, dtype=torch.float32)
        self._slices = []
        self._views = [[], []]          # parameter views into the two parameter buffers (overlap)
        self._failed = None
        self._grads_prepared = False
        for p, off in zip(self.params, offsets):
            view = self.flat_param[off:off + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view
            sink = self.flat_grad[off:off + p.numel()].view_as(p)
            p.grad_sink = sink
            p.grad_sink_written = False
            self._slices.append((p, sink))
            if self.overlap:
                self._views[0].append(view)
                self._views[1].append(self._param_bufs[1][off:off + p.numel()].view_as(p))

    def _setup_overlap(self, symm_mem, group, total, dev):
        second = symm_mem.empty(total, dtype=torch.float32, device=dev)
        second.zero_()
        hdl_second = symm_mem.rendezvous(second, group)
        self._param_bufs = [self.flat_param, second]
        self._param_hdls = [self._hdl_param, hdl_second]
        self._cur = 0
        n = self.hi - self.lo
        shape = (max(n, 0),)
        # ring order (rank + 1, rank + 2, ...): at any moment of the pull or push phase every rank is
        # read by one peer and written by one peer, instead of all ranks converging on rank 0 first
        peers = [(self.rank + k) % self.world for k in range(1, self.world)]
        # this rank's shard of every peer's gradient buffer / of every peer's parameter buffers
        self._peer_grad = {r: self._hdl_grad.get_buffer(r, shape, torch.float32, self.lo) for r in peers}
        self._peer_param = [{r: h.get_buffer(r, shape, torch.float32, self.lo) for r in peers}
                            for h in self._param_hdls]
        self._recv = {r: torch.empty(shape, device=dev, dtype=torch.float32) for r in peers}
        self._side = torch.cuda.Stream(device=dev)
        self._ready = torch.cuda.Event()
        self._pulled = torch.cuda.Event()
        self._updated = torch.cuda.Event()
        self._done = torch.cuda.Event()
        self._in_flight, self._stage = False, 0

    def _barrier(self, stream):
        """Enqueues the bounded inter-rank barrier on `stream`; raises at once if it cannot be launched."""
        self._epoch += 1
        rc = _lib.load().snb_peer_barrier(self._flag_ptrs, self.rank, self.world, self._epoch, self._timeout_ns,
                                          self._status.data_ptr(), stream.cuda_stream)
        if rc != 0:
            self._failed = "peer barrier could not be launched"
        _lib.check(rc, "peer_barrier")
        _C.launch_count += 1

    def check(self):
        """Raises if a barrier of an earlier step gave up on a peer (reads a pinned host word, no
        synchronisation) or if this rank failed to enqueue part of an exchange.  The parameters of a
        step whose barrier failed were built from incomplete data and must be discarded."""
        if self._failed:
            raise RuntimeError("data-parallel step failed on this rank: %s" % self._failed)
        if self.peer and int(self._status[0]) != 0:
            raise RuntimeError("rank %d did not reach the gradient-exchange barrier within %.1f s"
                               % (int(self._status[0]) - 1, self._timeout_ns * 1e-9))

    def _signal(self, stream):
        self._epoch += 1
        rc = _lib.load().snb_peer_signal(self._flag_ptrs, self.rank, self.world, self._epoch, stream.cuda_stream)
        if rc != 0:
            self._failed = "peer signal could not be launched"
        _lib.check(rc, "peer_signal")
        _C.launch_count += 1
        return self._epoch

    def _wait(self, epoch, stream):
        rc = _lib.load().snb_peer_wait(self._flag_ptrs, self.rank, self.world, epoch, self._timeout_ns,
                                       self._status.data_ptr(), stream.cuda_stream)
        if rc != 0:
            self._failed = "peer wait could not be launched"
        _lib.check(rc, "peer_wait")
        _C.launch_count += 1

    def begin_exchange(self):
        """Opens the gradient exchange behind everything that is on the current stream now (the
        backward) and returns at once: the side stream tells every peer that this rank's gradients
        are complete.  Nothing waits yet.

        The exchange then proceeds in three more stream-ordered stages, each of which the caller may
        place between two kernels of the work it overlaps with the exchange (the interval-bound pass),
        and each of which the next stage runs itself if the caller did not:
          start_pulls()   side stream: wait for the peers' signals, copy this rank's shard of every
                          peer's gradient buffer (copy engines over NVLink, no SM time);
          apply_update()  caller's stream: sum + AdamW for the shard into the second parameter
                          buffer; side stream: copy the shard into every peer's second buffer, signal;
          end_exchange()  wait for the peers' signals, switch the parameters to the second buffer.
        Signals are sent as early and waited for as late as the data flow allows: a kernel that
        waits on the GPU costs the kernels running beside it about half of the time it waits, and
        by the time of the wait the peers have normally long signalled.

        Every launch status is examined before the next operation is queued: a rank that cannot
        launch stops there (pushing nothing, signalling nothing) and raises, and its peers' next
        wait runs into its time limit and reports this rank through check()."""
        if not self.overlap:
            raise RuntimeError("begin_exchange() needs FlatAdamW(peer_memory=True, overlap=True)")
        self.check()
        self._prepare_grads()
        self.step_count += 1
        dev = self.flat_grad.device
        with torch.cuda.device(dev):
            self._ready.record(torch.cuda.current_stream(dev))
            self._side.wait_event(self._ready)
            self._grads_epoch = self._signal(self._side)
        self._grads_consumed()
        self._in_flight, self._stage = True, 1

    def start_pulls(self):
        """Second stage (side stream): every rank's backward has written its gradients -> pull this
        rank's shard of each peer's gradient buffer."""
        if not self._in_flight or self._stage != 1:
            return
        dev = self.flat_grad.device
        with torch.cuda.device(dev), torch.cuda.stream(self._side):
            self._wait(self._grads_epoch, self._side)
            if self.hi > self.lo:
                for r, src in self._peer_grad.items():
                    self._recv[r].copy_(src, non_blocking=True)
            self._pulled.record(self._side)
        self._stage = 2

    def apply_update(self):
        """Third stage, on the *current* stream: waits for the pulled gradient shards, runs the sum +
        AdamW kernel for this rank's shard into the second parameter buffer, and hands over to the
        side stream, which pushes the shard into every peer's second buffer and signals.

        Why not on the side stream as well: the distance kernels are persistent, one CTA per SM with
        the whole register file and an equal share of the work each, so a kernel that arrives from
        another stream can only start at a kernel boundary, holds back some CTAs of the next
        persistent kernel there, and that kernel then ends as late as its last CTA started.  On the
        caller's own stream, between two of its kernels, the update costs its own duration (0.2 ms
        for a quarter of 120 M parameters) and nothing else.  Call it where the pulls have surely
        landed and enough work follows to cover the pushes."""
        if not self._in_flight or self._stage > 2:
            return
        self.start_pulls()
        dev = self.flat_grad.device
        lo, hi, n = self.lo, self.hi, self.hi - self.lo
        cur, nxt = self._param_bufs[self._cur], self._param_bufs[self._cur ^ 1]
        with torch.cuda.device(dev):
            main = torch.cuda.current_stream(dev)
            main.wait_event(self._pulled)
            if n > 0:
                parts = [self.flat_grad[lo:hi] if r == self.rank else self._recv[r] for r in range(self.world)]
                ptrs = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in parts])
                rc = _lib.load().snb_adamw_reduce_step(
                    cur[lo:hi].data_ptr(), nxt[lo:hi].data_ptr(), ptrs, self.world, self.exp_avg.data_ptr(),
                    self.exp_avg_sq.data_ptr(), n, float(self.lr), float(self.betas[0]), float(self.betas[1]),
                    float(self.eps), float(self.weight_decay), self.step_count, 1.0 / self.world, main.cuda_stream)
                if rc != 0:
                    self._failed = "the shard update could not be launched"
                _lib.check(rc, "adamw_reduce_step")
                _C.launch_count += 1
            self._updated.record(main)
            self._side.wait_event(self._updated)
            with torch.cuda.stream(self._side):
                if n > 0:
                    for r, dst in self._peer_param[self._cur ^ 1].items():
                        dst.copy_(nxt[lo:hi], non_blocking=True)
                self._params_epoch = self._signal(self._side)
        self._stage = 3

    def end_exchange(self):
        """The current stream waits for the exchange (running the update first if `apply_update()`
        was not called); parameters switch to the updated buffer."""
        if not self._in_flight:
            raise RuntimeError("end_exchange() without begin_exchange()")
        self.apply_update()
        dev = self.flat_grad.device
        with torch.cuda.device(dev), torch.cuda.stream(self._side):
            # every rank's shard of the new values has landed in this rank's second buffer
            self._wait(self._params_epoch, self._side)
            self._done.record(self._side)
        torch.cuda.current_stream(dev).wait_event(self._done)
        self.check()
        self._cur ^= 1
        self.flat_param = self._param_bufs[self._cur]
        for p, view in zip(self.params, self._views[self._cur]):
            p.data = view
        self._in_flight = False

    def zero_grad(self):
        """Autograd-owned gradients are dropped; the sinks are marked unwritten (the first backward
        of the step overwrites them, further ones add, see ops._dist_backward)."""
        for p in self.params:
            p.grad = None
            p.grad_sink_written = False
        self._grads_prepared = False

    def gather_grads(self):
        """Moves gradients that autograd produced itself (parameters whose operator does not
        write into the sink) into the flat buffer, adding to what the step already wrote there."""
        for p, sink in self._slices:
            if p.grad is not None:
                if p.grad_sink_written:
                    sink.add_(p.grad)
                else:
                    sink.copy_(p.grad)
                    p.grad_sink_written = True
                p.grad = None

    def set_flat_grad(self, flat=None):
        """Declares the flat gradient buffer to hold this step's gradients of all parameters (after
        copying `flat` into it when given): for callers that fill the buffer themselves instead of
        running a backward, e.g. to replay recorded gradients."""
        if flat is not None:
            self.flat_grad.copy_(flat)
        for p in self.params:
            p.grad_sink_written = True

    def _prepare_grads(self):
        """Before the gradients are consumed: a parameter that no backward reached since the last
        step (or zero_grad()) has a zero gradient, not the previous step's.  Idempotent within a step."""
        if self._grads_prepared:
            return
        for p, sink in self._slices:
            if not p.grad_sink_written:
                sink.zero_()
        self._grads_prepared = True

    def _grads_consumed(self):
        """After the update has been queued: the next backward overwrites the sinks again."""
        for p in self.params:
            p.grad_sink_written = False
        self._grads_prepared = False

    def all_reduce(self, async_op=False):
        """Sums the flat gradient over ranks (one collective); the mean is taken inside step()."""
        if self.world == 1 or self.peer:
            return None            # with peer memory the exchange is part of step()
        self._prepare_grads()
        return dist.all_reduce(self.flat_grad, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)

    def step(self):
        if self.overlap:
            self.begin_exchange()
            self.end_exchange()
            return
        self.check()
        self._prepare_grads()
        self.step_count += 1
        dev = self.flat_param.device
        if self.peer:
            with torch.cuda.device(dev):
                stream = torch.cuda.current_stream(dev)
                # every rank's backward has finished writing its gradients ...
                self._barrier(stream)
                rc = _lib.load().snb_dp_adamw_step(
                    self._grad_ptrs, self._param_ptrs, self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                    self.rank, self.world, self.lo, self.hi, float(self.lr), float(self.betas[0]),
                    float(self.betas[1]), float(self.eps), float(self.weight_decay), self.step_count,
                    stream.cuda_stream)
                if rc != 0:
                    self._failed = "the fused exchange kernel could not be launched"
                _lib.check(rc, "dp_adamw_step")
                _C.launch_count += 1
                # ... and every rank's new parameters have landed here before the next forward
                self._barrier(stream)
            self._grads_consumed()
            return
        with torch.cuda.device(dev):
            rc = _lib.load().snb_adamw_step(
                self.flat_param.data_ptr(), self.flat_grad.data_ptr(), self.exp_avg.data_ptr(),
                self.exp_avg_sq.data_ptr(), self.numel, float(self.lr), float(self.betas[0]),
                float(self.betas[1]), float(self.eps), float(self.weight_decay), self.step_count,
                1.0 / self.world, torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(rc, "adamw_step")
        _C.launch_count += 1
        self._grads_consumed()
