#!/usr/bin/env python
"""Benchmark of the norm-distance hot path on B200: one SortNet-MLP training step plus the
interval-bound (certification) forward, batch 512 per GPU.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                      (the CPU arm, see below)

A step = masked l-inf forward of the 6-layer SortNet-MLP (fresh sub-batch masks), mixture
loss, sparse backward, the gradient exchange between ranks (N > 1), fused AdamW, and the l-inf
interval-bound forward through all layers under no_grad.  Inputs are seeded synthetic tensors
with the CIFAR-10 shapes ([512, 3, 32, 32] uniform in [0, 1), labels uniform in [0, 10)),
weights N(0, 1); the per-GPU batch is fixed as N grows (weak scaling).

Prints one JSON line (rank 0).  `value` is samples/s with inputs resident in HBM; `e2e` is the
same step fed from pinned host memory with the loss read back every step; `roofline` is the
dominant kernel's FP32 fraction, its time taken from CUDA events around its launches in a short
separate pass (the headline regions run without those events); `cpu_baseline` is the
reference's PyTorch way of computing the same step timed on this host's cores.  Secondary
blocks (never the headline): `gpu_comparator` (the same step through the reference's own model
code and CUDA kernels compiled for sm_100a, when oracle/_ref holds them), `configs[0]`,
`configs[2]`, `configs[3]` (the other single-GPU configurations), `lp_training_step` (finite p),
and at N > 1 `dp_check` (replica identity + one step against all-reduce + AdamW),
`strong_scaling` (global batch 512 split over the ranks) and at N = 8 `configs[4]`.
"""
import argparse
import copy
import ctypes
import gc
import json
import math
import os
import statistics
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

INF = float("inf")

# The configurations of this project, numbered as in its configuration list (0 = single layer).
CONFIGS = {
    1: dict(label="configs[1]: SortNet-MLP (5 x 5120 + head 10), CIFAR-shaped input [512, 3072] per GPU, "
                  "keep 0.9 sub-batch masks, p = inf, train eps 8/255, IBP eps 8/255",
            input_dim=(3, 32, 32), depth=6, width=5120, classes=10, keep=0.9, batch=512, eps=8 / 255),
    2: dict(label="configs[2]: pure l-inf net, 6 x 5120 with mean shift + head 10, no masks, input [512, 3072], eps 2/255",
            input_dim=(3, 32, 32), depth=7, width=5120, classes=10, keep=1.0, batch=512, eps=2 / 255),
    3: dict(label="configs[3]: SortNet-MLP (5 x 5120 + head 200), input [512, 12288], keep 0.9, eps 1/255",
            input_dim=(3, 64, 64), depth=6, width=5120, classes=200, keep=0.9, batch=512, eps=1 / 255),
    4: dict(label="configs[4]: SortNet-MLP-2x (5 x 10240 + head 1000), input [1024, 12288] sharded 128 per GPU over 8, "
                  "keep 0.9, eps 1/255",
            input_dim=(3, 64, 64), depth=6, width=10240, classes=1000, keep=0.9, batch=128, eps=1 / 255),
}
HEADLINE = CONFIGS[1]
ADAM = dict(lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=0.0)
# limit of a GPU-side wait for a peer: generous, because the ranks reach their first step (module
# loading, first-launch set-up) seconds apart on a busy host; a rank that is really gone still ends
# the run with an error instead of a hang
PEER_WAIT_S = 30.0

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/ (bound_fwd_kernel_64x256_512x5120x5120.md; inf_fwd_sk_kernel_masked_512x4619x4596.md,
# all kernels of the entry point), at the shapes of the widest layers of the headline workload.
NCU_DRAM_BYTES_PER_LAUNCH = {
    "snb_bound_inf_dist_forward_nograd": 302.8e6,
    "snb_inf_dist_forward_ws": 262.2e6,
    "snb_inf_dist_forward_sorted_ws": 266.2e6,
    "snb_inf_dist_forward_nograd": 203.9e6,       # inf_fwd_sk_kernel_dense_512x5120x5120.md
}


# adamw_kernel: 480.0 MB read + 302.2-304.4 MB written per launch on 30 M parameters (ncu, the capture
# of profiles/adamw_kernel_30m_parameters.md; the last writes are still in L2 when the kernel ends);
# traffic grows in proportion to the parameter count
NCU_ADAMW_BYTES_PER_PARAMETER = 26.1


def layer_dims(cfg):
    pixels = cfg["input_dim"][0] * cfg["input_dim"][1] * cfg["input_dim"][2]
    w = cfg["width"]
    return [(pixels, w)] + [(w, w)] * (cfg["depth"] - 2) + [(w, cfg["classes"])]


# ------------------------------------------------------------------------------------------
# CPU arm: the reference's own PyTorch branches (or their restatement) on a bounded slice
# ------------------------------------------------------------------------------------------

def cpu_functions():
    """(functions, kind): the reference's own operator functions when its Python is staged under
    oracle/_ref/py, else the restatement in oracle/torch_fallback.py."""
    from oracle import torch_fallback
    try:
        fns = torch_fallback.reference_functions()
    except Exception:
        fns = None
    return (fns, "reference") if fns is not None else (None, "port")


def cpu_step_seconds(out_slice, threads, fns):
    import torch
    from oracle import torch_fallback
    torch.set_num_threads(threads)
    return torch_fallback.time_training_slice(layer_dims(HEADLINE), HEADLINE["keep"], INF, HEADLINE["eps"],
                                              out_slice=out_slice, rows=32, functions=fns)


CPU_SAMPLE = ("32 rows (one sub-batch) x %d of the kept outputs of every wide layer x all inputs, all 6 layers: masked "
              "l-inf forward + autograd backward + dense interval-bound forward through %s, on the host; each part "
              "scaled by outputs_full / outputs_timed; %.2f s of CPU work per step")
CPU_HOW = {"reference": "the reference's own norm_dist / bound_inf_dist with use_custom_cuda_func=False",
           "port": "a restatement of the reference's PyTorch branches (its Python is not staged here)"}


def run_reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    threads = os.cpu_count() or 1
    fns, kind = cpu_functions()
    out_slice = 128
    for _ in range(max(args.warmup, 1)):
        cpu_step_seconds(out_slice, threads, fns)
    t, raw = [], []
    for _ in range(args.steps):
        s, info = cpu_step_seconds(out_slice, threads, fns)
        t.append(s)
        raw.append(info["raw_seconds"])
    value = 32.0 / statistics.mean(t)
    line = {
        "impl": "reference", "metric": "train samples/s (fwd+bwd+IBP step)", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * 512 / value,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_block(args.gpus, None),
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": threads, "kind": kind,
                         "sample": CPU_SAMPLE % (out_slice, CPU_HOW[kind], statistics.mean(raw))},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def config_block(n, exchange):
    return {
        "workload": HEADLINE["label"],
        "global_batch": HEADLINE["batch"] * n, "batch_per_gpu": HEADLINE["batch"],
        "parallelism": "dp%d" % n,
        "optimizer": "AdamW, fused flat-buffer kernel" + ("; gradient exchange: " + exchange if exchange and n > 1 else ""),
        "l2": "weights alone are 482 MB per step, larger than the 126 MB L2; no explicit flush",
    }


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------

class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read only) every 50 ms."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(0.05)

    def finish(self):
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def mixture_loss(logits, margin, targets, lam=0.1, clip=1.0):
    """The reference's `mixture` loss (main.py:357-364): clipped worst-case margin + lam * cross-entropy."""
    import torch.nn.functional as F
    res = margin.clamp(min=0, max=clip)
    return res.max(dim=1)[0].mean() + lam * F.cross_entropy(logits, targets)


class Job:
    """One model of one configuration on this rank with its optimiser, synthetic data and step."""

    def __init__(self, cfg, dev, world, rank, exchange="none", batch=None, seed=0):
        import torch
        from sortnet_b200 import layers
        from sortnet_b200.dist import broadcast_parameters
        from sortnet_b200.optim import FlatAdamW
        self.cfg, self.dev, self.world, self.rank = cfg, dev, world, rank
        self.B = batch or cfg["batch"]
        torch.manual_seed(seed)
        self.model = layers.SortMLPModel(depth=cfg["depth"], width=cfg["width"], input_dim=cfg["input_dim"],
                                         num_classes=cfg["classes"], dropout=cfg["keep"]).to(dev)
        self.model.set_p(INF)
        if world > 1 and exchange != "none":
            broadcast_parameters(self.model)
        torch.manual_seed(1 + rank)  # masks and data differ per rank, like the reference's seed + rank
        self.exchange = exchange
        if exchange == "copies":
            self.opt = FlatAdamW(self.model, peer_memory=True, overlap=True, barrier_timeout_s=PEER_WAIT_S, **ADAM)
        elif exchange == "fused":
            self.opt = FlatAdamW(self.model, peer_memory=True, overlap=False, barrier_timeout_s=PEER_WAIT_S, **ADAM)
        else:                                   # "nccl": one flat all-reduce; "none": local optimiser
            self.opt = FlatAdamW(self.model, peer_memory=False, **ADAM)
        pool = 4
        gen = torch.Generator().manual_seed(100 + rank)
        self.host_x = [torch.rand(self.B, *cfg["input_dim"], generator=gen).pin_memory() for _ in range(pool)]
        self.host_t = [torch.randint(0, cfg["classes"], (self.B,), generator=gen).pin_memory() for _ in range(pool)]
        self.dev_x = [t.to(dev) for t in self.host_x]
        self.dev_t = [t.to(dev) for t in self.host_t]
        self.up, self.down = 1.0, 0.0           # the box is clipped to the pixel range [0, 1]
        self.pool = pool

    def bound_pass(self, x, t, after_layer=None):
        """The l-inf interval-bound forward of the whole net (point value + bounds, running means
        subtracted, certified fraction): the plain l-inf distance in every layer, see
        SortMLPModel.certified_margin(sort_eval=False)."""
        import torch
        with torch.no_grad():
            return self.model.certified_margin(x, t, self.cfg["eps"], self.up, self.down, sort_eval=False,
                                               after_layer=after_layer)

    def step(self, x, t, update=True, bounds=True):
        model, opt = self.model, self.opt
        model.train()
        loss = model.mixture_loss(x, t, self.cfg["eps"])      # forward + margin + the reference's mixture loss
        opt.zero_grad()
        loss.backward()
        opt.gather_grads()
        cert = None
        if not update:
            if bounds:
                cert = self.bound_pass(x, t)
        elif opt.overlap:
            opt.begin_exchange()              # side stream: "my gradients are complete"
            if bounds:
                # reads the pre-update weights.  After the first layer the side stream pulls the
                # gradient shards (the peers have signalled by then), after the third the shard's
                # update runs on this stream, and the pushes run beside the remaining layers.
                def stage(k):
                    if k == 0:
                        opt.start_pulls()
                    elif k == 2:
                        opt.apply_update()
                cert = self.bound_pass(x, t, after_layer=stage)
            opt.end_exchange()
        else:
            # same order as the overlapped path: the bound pass reads the pre-update weights
            if bounds:
                cert = self.bound_pass(x, t)
            if self.exchange == "nccl":
                opt.all_reduce()
            opt.step()
        return loss, cert

    def run(self, n, update=True, bounds=True):
        for i in range(n):
            self.step(self.dev_x[i % self.pool], self.dev_t[i % self.pool], update=update, bounds=bounds)

    def timed(self, steps, warmup, barrier, **kw):
        """Device-timed mean milliseconds per step over `steps` steps after `warmup` (this rank)."""
        import torch
        self.run(warmup, **kw)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        self.run(steps, **kw)
        e1.record()
        barrier()
        return e0.elapsed_time(e1) / steps

    def release(self):
        import torch
        self.model = self.opt = self.dev_x = self.dev_t = self.host_x = self.host_t = None
        gc.collect()
        torch.cuda.empty_cache()


def max_over_ranks(values, dev, world):
    import torch
    import torch.distributed as dist
    t = torch.tensor(values, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def dp_check(job, dev, world):
    """Correctness of the data-parallel step, outside the timed regions.
    (i) every rank's flat parameter buffer equals rank 0's, bit for bit;
    (ii) one more step taken two ways from the same local gradients: the selected exchange, and
    a plain all-reduce (NCCL) of the gradients followed by the single-GPU fused AdamW kernel on a
    copy of the parameters with the full moments gathered from the ranks' shards."""
    import torch
    import torch.distributed as dist
    from sortnet_b200 import _lib
    opt = job.opt
    opt.check()
    torch.cuda.synchronize()

    def identical():
        mine = opt.flat_param.detach().clone()
        other = mine.clone()
        dist.broadcast(other, src=0)
        flag = torch.tensor([1.0 if torch.equal(mine, other) else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return bool(flag.item() == 1.0)

    same_before = identical()
    n = opt.numel
    p0 = opt.flat_param.detach().clone()
    g_sum = opt.flat_grad.detach().clone()
    dist.all_reduce(g_sum)
    if opt.peer:                               # moments are sharded: rebuild the full vectors
        m_full = torch.zeros(n, device=dev)
        v_full = torch.zeros(n, device=dev)
        k = opt.hi - opt.lo
        m_full[opt.lo:opt.hi] = opt.exp_avg[:k]
        v_full[opt.lo:opt.hi] = opt.exp_avg_sq[:k]
        dist.all_reduce(m_full)
        dist.all_reduce(v_full)
    else:
        m_full, v_full = opt.exp_avg.clone(), opt.exp_avg_sq.clone()
    rc = _lib.load().snb_adamw_step(p0.data_ptr(), g_sum.data_ptr(), m_full.data_ptr(), v_full.data_ptr(), n,
                                    ADAM["lr"], ADAM["betas"][0], ADAM["betas"][1], ADAM["eps"], ADAM["weight_decay"],
                                    opt.step_count + 1, 1.0 / world, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "adamw_step")
    # the selected exchange on the very same local gradients (mark them as this step's)
    opt.set_flat_grad()
    if job.exchange == "nccl":
        opt.all_reduce()
    opt.step()
    torch.cuda.synchronize()
    opt.check()
    diff = (opt.flat_param - p0).abs().max()
    scale = p0.abs().max().clamp(min=1.0)
    worst = torch.stack([diff / scale])
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    same_after = identical()
    ok = same_before and same_after and float(worst) <= 1e-5
    return {"replicas_identical": same_before and same_after, "max_rel_vs_allreduce": float(worst),
            "tolerance": 1e-5, "exchange": job.exchange, "ok": ok}


def exchange_timeline(job, dev, world, steps=10):
    """Where the overlapped exchange touches the bound pass, from CUDA events on this rank's streams
    over `steps` extra steps: the two parts of the bound pass (before / after the shard's update), the
    update kernel, and the time the main stream had to wait for the pulled gradients and for the
    end of the exchange.  All ranks' rows are gathered on rank 0."""
    import torch
    import torch.distributed as dist
    opt = job.opt
    if not getattr(opt, "overlap", False):
        return None
    new_event = lambda: torch.cuda.Event(enable_timing=True)
    rows = []
    begin0, apply0, end0 = opt.begin_exchange, opt.apply_update, opt.end_exchange

    def begin():
        e = new_event()
        e.record()
        rows.append({"begin": e})
        begin0()

    def apply():
        if opt._stage > 2:
            return
        opt.start_pulls()
        main = torch.cuda.current_stream(dev)
        a, b, c = new_event(), new_event(), new_event()
        a.record()
        main.wait_event(opt._pulled)
        b.record()
        apply0()
        c.record()
        rows[-1].update(a=a, b=b, c=c)

    def end():
        a, b = new_event(), new_event()
        a.record()
        end0()
        b.record()
        rows[-1].update(e0=a, e1=b)

    opt.begin_exchange, opt.apply_update, opt.end_exchange = begin, apply, end
    try:
        job.run(steps + 2)
        torch.cuda.synchronize()
    finally:
        opt.begin_exchange, opt.apply_update, opt.end_exchange = begin0, apply0, end0
    keep = rows[2:]
    mean = lambda f: sum(f(r) for r in keep) / len(keep)
    mine = torch.tensor([mean(lambda r: r["begin"].elapsed_time(r["a"])), mean(lambda r: r["a"].elapsed_time(r["b"])),
                         mean(lambda r: r["b"].elapsed_time(r["c"])), mean(lambda r: r["c"].elapsed_time(r["e0"])),
                         mean(lambda r: r["e0"].elapsed_time(r["e1"]))], device=dev, dtype=torch.float64)
    every = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    names = ("bound_pass_before_update_ms", "wait_for_pulls_ms", "update_kernel_ms", "bound_pass_after_update_ms",
             "wait_at_end_ms")
    return [{k: round(float(v), 3) for k, v in zip(names, t)} for t in every]


def fp32_peak_gflops(dev):
    """FP32 CUDA-core peak of this GPU, measured now with a register-only FMA chain (2 flops per FMA)."""
    import torch
    from sortnet_b200 import _lib
    scratch = torch.zeros(4, device=dev)
    lib = _lib.load()
    flops = ctypes.c_double()
    best = 0.0
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        _lib.check(lib.snb_probe_fp32(scratch.data_ptr(), 4096, ctypes.byref(flops),
                                      torch.cuda.current_stream().cuda_stream), "probe_fp32")
        b.record()
        torch.cuda.synchronize()
        best = max(best, flops.value / (a.elapsed_time(b) * 1e-3))
    return best * 1e-9


PEAK_SOURCE = ("FFMA probe timed in this run (2 flops per FMA); MEASURED_PEAKS.json has no FP32 figure; nominal "
               "148 SM x 128 lanes x 2 x 1.965 GHz = 74.5 TFLOP/s")


def kernel_stats(timeline, entry):
    """Launches of `entry` on the widest layers (mask sizes differ a little from step to step, so
    every shape within 10 % of the largest counts): a representative shape, the mean time per
    launch and the mean element count per launch."""
    rows = {k[1]: v for k, v in timeline.items() if k[0] == entry}
    if not rows:
        return None
    size = lambda t: t[0] * t[1] * t[2]
    biggest = max(size(t) for t in rows)
    picked = {t: v for t, v in rows.items() if size(t) >= 0.9 * biggest}
    launches = sum(len(v) for v in picked.values())
    total_ms = sum(sum(v) for v in picked.values())
    elems = sum(size(t) * len(v) for t, v in picked.items()) / launches
    return max(picked, key=size), total_ms / launches, elems


def profiled_pass(job, steps, **kw):
    """A few steps with a CUDA-event pair around every entry-point call: {(entry, shape): [ms]}.
    The layers are run operator by operator here (the same kernels in the same order as the
    one-call-per-layer path of the headline regions), so that every kernel gets its own events."""
    from sortnet_b200 import layers, norm_dist_cuda as C
    layers.FUSED_LAYERS = False
    try:
        job.run(1, **kw)                      # first use of the operator-by-operator path, untimed
        C.start_profile()
        job.run(steps, **kw)
        return C.stop_profile()
    finally:
        layers.FUSED_LAYERS = True


def roofline_blocks(timeline, peak_gflops):
    by_entry = {}
    for (entry, tag), v in timeline.items():
        by_entry[entry] = by_entry.get(entry, 0.0) + sum(v)
    total = sum(by_entry.values())
    shares = {k[4:]: round(v / total, 4) for k, v in sorted(by_entry.items(), key=lambda kv: -kv[1])}
    roofs = {}
    for entry, ops_per_elem in (("snb_bound_inf_dist_forward_nograd", 6.0), ("snb_inf_dist_forward_sorted_ws", 2.0),
                                ("snb_inf_dist_forward_ws", 2.0), ("snb_inf_dist_forward_nograd", 2.0)):
        ks = kernel_stats(timeline, entry)
        if ks is None:
            continue
        (b_, co_, ci_), mean_ms, mean_elems = ks
        achieved = ops_per_elem * mean_elems / (mean_ms * 1e-3) * 1e-9
        roofs[entry] = {
            "bound": "fp32", "kernel": entry[4:], "shape_B_CO_CI": [b_, co_, ci_],
            "ops_per_element": ops_per_elem, "ms_per_launch": round(mean_ms, 4),
            "achieved": round(achieved, 1), "peak": round(peak_gflops, 1), "unit": "GFLOP/s",
            "frac": round(achieved / peak_gflops, 4), "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(entry),
            "peak_source": PEAK_SOURCE,
        }
    dominant = max(roofs.values(), key=lambda r: by_entry.get("snb_" + r["kernel"], 0.0)) if roofs else None
    return shares, roofs, dominant, total


def lp_blocks(job, peak_gflops, sm_mhz):
    """The p-annealed phases of the recipe (p = 8, then a general p) on the headline model: one masked
    training step without the bound pass, device-timed over 10 steps, plus the generic-p kernels
    against the special-function-unit roof (2 transcendentals per element; 16 per clock per SM)."""
    import torch
    out, roof = {}, None
    for p_val in (8.0, 31.6):
        job.model.set_p(p_val)
        ms = job.timed(10, 2, torch.cuda.synchronize, bounds=False)
        out["p=%g" % p_val] = {"ms_per_step": round(ms, 3), "samples_per_s": round(job.B / (ms * 1e-3), 1), "steps": 10}
        if p_val == 31.6:
            tl = profiled_pass(job, 2, bounds=False)
            sms = torch.cuda.get_device_properties(job.dev).multi_processor_count
            xu_peak = 16.0 * sms * (sm_mhz or 1965.0) * 1e6 * 1e-9          # G transcendentals / s
            roof = {"bound": "xu (special-function unit)", "peak": round(xu_peak, 1), "unit": "G transcendental/s",
                    "peak_source": "16 per clock per SM x %d SMs x %s MHz (median SM clock of this run)" % (sms, sm_mhz),
                    "ops_per_element": 2.0, "p": 31.6}
            for entry, key in (("snb_norm_dist_forward_ws", "forward"), ("snb_norm_dist_backward_input_weight", "backward")):
                ks = kernel_stats(tl, entry)
                if ks is None:
                    continue
                shape, mean_ms, elems = ks
                ach = 2.0 * elems / (mean_ms * 1e-3) * 1e-9
                roof[key] = {"shape_B_CO_CI": list(shape), "ms_per_launch": round(mean_ms, 4),
                             "achieved": round(ach, 1), "frac": round(ach / xu_peak, 4)}
            roof["note"] = "the forward's time includes the l-inf pass that supplies the normaliser and the root kernel"
    job.model.set_p(INF)
    return out, roof


def hbm_block(job):
    """The HBM-bound kernel of the step (fused AdamW: 4 reads + 3 writes of 4 bytes per parameter)
    against the measured copy bandwidth of this pool's B200s."""
    import torch
    opt = job.opt
    hbm_peak, hbm_src = 6650.0, "fallback 6.65 TB/s (MEASURED_PEAKS.json absent)"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            hbm_peak = float(json.load(f)["hbm_gbs"])
            hbm_src = "MEASURED_PEAKS.json hbm_gbs (STREAM-style copy)"
    except Exception:
        pass
    def one_step():
        opt.set_flat_grad()                    # keep the gradients of the last backward: the step then
        opt.step()                             # is the update kernel alone, as inside a training step

    a_ev, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    one_step()
    torch.cuda.synchronize()
    a_ev.record()
    for _ in range(5):
        one_step()
    b_ev.record()
    torch.cuda.synchronize()
    adam_ms = a_ev.elapsed_time(b_ev) / 5
    adam_gbs = 28.0 * opt.numel / (adam_ms * 1e-3) * 1e-9
    return {"bound": "hbm", "kernel": "adamw_kernel", "ms_per_launch": round(adam_ms, 4),
            "achieved": round(adam_gbs, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(adam_gbs / hbm_peak, 4),
            "traffic": round(NCU_ADAMW_BYTES_PER_PARAMETER * opt.numel), "algorithmic_bytes": 28 * opt.numel,
            "peak_source": hbm_src}


def single_layer_block(dev, peak_gflops):
    """configs[0]: one l-inf layer, x [128, 784], W [5120, 784], box [x - 0.3, x + 0.3] clipped to
    [0, 1]: forward with argmax words, sparse backward, interval bounds, each device-timed.  The
    weights rotate through 9 copies (145 MB) so that no launch finds its operands in L2."""
    import torch
    from sortnet_b200 import norm_dist_cuda as C
    B, CI, CO = 128, 784, 5120
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.rand(B, CI, 1, device=dev, generator=g)
    ws = [torch.randn(CO, CI, device=dev, generator=g) for _ in range(9)]
    xl, xu = (x - 0.3).clamp(0, 1), (x + 0.3).clamp(0, 1)
    gy = torch.randn(B, CO, 1, device=dev, generator=g)
    y, pos = torch.empty(B, CO, 1, device=dev), torch.empty(B, CO, 1, device=dev, dtype=torch.int32)
    yl, yu = torch.empty_like(y), torch.empty_like(y)
    gx, gw = torch.empty_like(x), torch.empty_like(ws[0])

    def timed(fn, iters=27):
        for i in range(3):
            fn(ws[i % 9])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(iters):
            fn(ws[i % 9])
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters

    E = B * CI * CO
    t_f = timed(lambda w: C.inf_dist_forward(x, w, y, pos, 1))
    t_b = timed(lambda w: C.inf_dist_backward_input_weight(gy, pos, gx, gw, 1))
    t_i = timed(lambda w: C.bound_inf_dist_forward_nograd(xl, xu, w, yl, yu, 1))
    frac = lambda ops, ms: round(ops * E / (ms * 1e-3) * 1e-9 / peak_gflops, 4)
    bwd_bytes = 8 * B * CO + 4 * B * CI + 4 * CO * CI      # g + pos read, grad_x written, grad_w zero-filled
    return {"workload": "configs[0]: single l-inf layer 128 x 784 -> 5120, fwd + argmax, sparse bwd, interval bounds",
            "forward_ms": round(t_f, 4), "forward_frac_fp32": frac(2.0, t_f),
            "backward_ms": round(t_b, 4), "backward_gbs": round(bwd_bytes / (t_b * 1e-3) * 1e-9, 1),
            "bounds_ms": round(t_i, 4), "bounds_frac_fp32": frac(6.0, t_i),
            "samples_per_s": round(B / ((t_f + t_b + t_i) * 1e-3), 1), "l2": "weights rotate through 145 MB"}


def config_step_block(idx, dev, steps=10, warmup=3):
    """A secondary configuration at N = 1: the same step definition as the headline."""
    import torch
    cfg = CONFIGS[idx]
    job = Job(cfg, dev, 1, 0, exchange="none")
    ms = job.timed(steps, warmup, torch.cuda.synchronize)
    out = {"workload": cfg["label"], "ms_per_step": round(ms, 3), "samples_per_s": round(job.B / (ms * 1e-3), 1),
           "steps": steps}
    job.release()
    return out


def gpu_comparator_block(job, steps=10, warmup=3):
    """The headline step through the reference itself on this GPU: its unmodified SortMLPModel and
    operator layer (staged under oracle/_ref/py) over its own CUDA extension compiled for sm_100a
    (oracle/_ref/norm_dist_cuda.so), torch.optim.AdamW, same weights, same data.  The bound pass is
    the reference's own keep-rate-1 path (norm_dist no-grad + bound_inf_dist per layer, running
    means subtracted), i.e. the work the headline step does.  `eval_faithful_bound_pass` times, for
    both sides, the evaluation forward the reference's certified_test really runs on this model
    (sort neuron + its bounds, K = 10)."""
    import torch
    from oracle import build_ref
    ext = build_ref.load()
    if ext is None or build_ref.staged_python() is None:
        return {"unavailable": "oracle/_ref holds no build of the reference (no reference checkout on the build machine)"}
    cfg, dev = job.cfg, job.dev
    ref_ops, ref_models, ref_nets = build_ref.import_reference_python(ext)
    ref_models.NormDistBase.dropout_list.clear()
    ref_models.NormDistBase.dropout_buffer = None
    torch.manual_seed(0)
    model = ref_nets.SortMLPModel(depth=cfg["depth"], width=cfg["width"], input_dim=cfg["input_dim"],
                                  num_classes=cfg["classes"], dropout=cfg["keep"]).to(dev)
    model.load_state_dict(job.model.state_dict())
    opt = torch.optim.AdamW(model.parameters(), **ADAM)
    eps = cfg["eps"]
    drop_list = ref_models.NormDistBase.dropout_list
    up, down = torch.ones(1, device=dev), torch.zeros(1, device=dev)

    def bound_pass(x, t, faithful):
        model.eval()
        saved = dict(drop_list)
        if not faithful:
            drop_list.clear()                 # the reference's own branch for layers without a keep rate
        try:
            with torch.no_grad():
                _, margin = model(x, targets=t, eps=eps, up=up, down=down)
        finally:
            drop_list.clear()
            drop_list.update(saved)
        return (margin.scatter(1, t.view(-1, 1), float("-inf")).max(dim=1)[0] < 0).float().mean()

    def step(x, t):
        model.train()
        logits, margin = model(x, targets=t, eps=eps)
        loss = mixture_loss(logits, margin, t)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        cert = bound_pass(x, t, False)
        opt.step()
        return loss, cert

    def timed(fn, n, w):
        for i in range(w):
            fn(job.dev_x[i % job.pool], job.dev_t[i % job.pool])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            fn(job.dev_x[i % job.pool], job.dev_t[i % job.pool])
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    # the faster of two blocks: the reference's step reads a count back from the GPU for every layer
    # (its sampler's .item()), so its ~2000 launches per step are exposed to the host and the time
    # swings with the load on the host's cores (seen: 40 ms on a quiet host, 79-182 ms on busy ones)
    ms_blocks = [timed(step, steps, warmup), timed(step, steps, 0)]
    ms_ref = min(ms_blocks)
    ms_ref_faithful = timed(lambda x, t: bound_pass(x, t, True), 3, 1)
    with torch.no_grad():
        ms_ours_faithful = timed(lambda x, t: job.model.certified_margin(x, t, eps, job.up, job.down), 3, 1)
    del model, opt
    gc.collect()
    torch.cuda.empty_cache()
    return {"what": "configs[1] step through the reference's SortMLPModel + core/norm_dist.py over its own CUDA "
                    "extension built for sm_100a, torch.optim.AdamW, l-inf bound pass via its keep-rate-1 branch",
            "ms_per_step": round(ms_ref, 3), "samples_per_s": round(job.B / (ms_ref * 1e-3), 1), "steps": steps,
            "ms_per_step_blocks": [round(v, 3) for v in ms_blocks],
            "eval_faithful_bound_pass": {"what": "evaluation forward with the sort neuron and its bounds (K = 10), no grad",
                                         "reference_ms": round(ms_ref_faithful, 3), "ours_ms": round(ms_ours_faithful, 3),
                                         "speedup": round(ms_ref_faithful / ms_ours_faithful, 3)}}


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from sortnet_b200 import _lib, norm_dist_cuda as C

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # stdout carries exactly one JSON line.  Libraries write there too (NCCL prints its version
    # banner with printf when NCCL_DEBUG asks for it), so file descriptor 1 points at stderr for the
    # duration of the run and the result goes to the saved descriptor.
    sys.stdout.flush()
    result_fd = os.dup(1)
    os.dup2(2, 1)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    # N > 1: the gradient exchange runs as device-to-device copies over NVLink on a side stream,
    # beside the bound pass, with a local sum + AdamW kernel for this rank's shard in between
    # ("copies"); "fused" = one kernel doing reduce-scatter + AdamW + all-gather over peer pointers,
    # not overlapped; "nccl" = one flat all-reduce followed by the local fused AdamW.
    exchange = "none"
    if world > 1:
        exchange = args.exchange
        if exchange != "nccl":
            try:
                job = Job(HEADLINE, dev, world, rank, exchange=exchange)
            except Exception as exc:                      # symmetric memory not available: use NCCL
                print("rank %d: peer-memory step unavailable (%s); using one NCCL all-reduce" % (rank, exc), file=sys.stderr)
                exchange = "nccl"
        flag = torch.tensor([1.0 if exchange == "nccl" else 0.0], device=dev)
        dist.all_reduce(flag)
        if 0.0 < float(flag) < world:
            raise SystemExit("ranks disagree on the gradient-exchange path")
    if exchange in ("none", "nccl"):
        job = Job(HEADLINE, dev, world, rank, exchange=exchange)
    exchange_text = {
        "none": "none (single GPU)",
        "copies": "device-to-device copies over NVLink (reduce-scatter, all-gather) beside the bound pass, the shard's "
                  "sum/AdamW kernel between two of its layers, ordered by bounded peer barriers",
        "fused": "fused reduce-scatter + AdamW + all-gather kernel over NVLink peer memory",
        "nccl": "one flat NCCL all-reduce + local fused AdamW"}[exchange]
    B = job.B

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Warm-up.  A peer-memory exchange that fails here with an error the process survives (a rank
    # whose GPU-side wait for a peer ran into its time limit raises from FlatAdamW.check()) makes
    # all ranks start over with one NCCL all-reduce per step; the JSON line says so.
    fallback = None
    try:
        job.run(args.warmup)
        torch.cuda.synchronize()
        if world > 1:
            job.opt.check()
            if args.inject_exchange_failure and rank == world - 1:
                raise RuntimeError("injected on the host by --inject-exchange-failure")
    except RuntimeError as exc:
        if world == 1 or exchange == "nccl":
            raise
        fallback = str(exc).splitlines()[0][:200]
        print("rank %d: %s exchange failed in warm-up (%s)" % (rank, exchange, fallback), file=sys.stderr)
    if world > 1 and exchange != "nccl":
        flag = torch.tensor([1.0 if fallback else 0.0], device=dev)
        dist.all_reduce(flag)
        if float(flag) > 0:
            torch.cuda.synchronize()
            job.release()
            fallback = fallback or "another rank's exchange failed"
            exchange = "nccl"
            exchange_text = ("one flat NCCL all-reduce + local fused AdamW (the peer-memory exchange failed in "
                             "warm-up: %s)" % fallback)
            job = Job(HEADLINE, dev, world, rank, exchange=exchange)
            job.run(args.warmup)
    barrier()

    # ---- timed region 1: inputs resident in HBM, no per-call events ---------------------
    sampler = ClockSampler(local)
    sampler.start()
    C.reset_counters()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    job.run(args.steps)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    launches = C.launch_count
    job.opt.check()

    # ---- timed region 2: end to end from pinned host memory ------------------------------
    warm_x, warm_t = torch.empty_like(job.dev_x[0]), torch.empty_like(job.dev_t[0])
    warm_out = torch.zeros(2, pin_memory=True)
    for i in range(2):                                     # first use of the copy paths, untimed
        warm_x.copy_(job.host_x[i % job.pool], non_blocking=True)
        warm_t.copy_(job.host_t[i % job.pool], non_blocking=True)
        loss, cert = job.step(warm_x, warm_t)
        warm_out[0].copy_(loss.detach(), non_blocking=True)
        warm_out[1].copy_(cert, non_blocking=True)
    gc.collect()
    gc.disable()
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    # Every step copies its inputs from pinned host memory into two resident buffers and copies its
    # loss and certified fraction to pinned host memory; the host reads those one step later, so
    # it never waits for the step it has just enqueued.  All copies and reads are inside the
    # timed region.
    main_stream = torch.cuda.current_stream(dev)
    in_x = [torch.empty_like(job.dev_x[0]) for _ in range(2)]
    in_t = [torch.empty_like(job.dev_t[0]) for _ in range(2)]
    results = torch.zeros(args.steps, 2, pin_memory=True)
    sink = 0.0
    done = []
    for i in range(args.steps):
        x, t = in_x[i % 2], in_t[i % 2]
        x.copy_(job.host_x[i % job.pool], non_blocking=True)
        t.copy_(job.host_t[i % job.pool], non_blocking=True)
        loss, cert = job.step(x, t)
        results[i, 0].copy_(loss.detach(), non_blocking=True)
        results[i, 1].copy_(cert, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(main_stream)
        done.append(ev)
        if i > 0:
            done[i - 1].synchronize()
            sink += float(results[i - 1, 0]) + float(results[i - 1, 1])
    done[-1].synchronize()
    sink += float(results[-1, 0]) + float(results[-1, 1])
    e3.record()
    barrier()
    gc.enable()
    clocks = sampler.finish()
    ms_e2e = e2.elapsed_time(e3) / args.steps
    job.opt.check()
    if not math.isfinite(sink):
        raise SystemExit("the step produced a non-finite loss")
    # a bounded device-side wait (the mbarrier waits of the TMA-staged kernel) that gave up would have
    # left partly written bounds: read the library's flag where results are read anyway
    if _lib.load().snb_device_wait_failed() != 0:
        raise SystemExit("a bounded device-side wait gave up during the run (snb_device_wait_failed)")
    ms, ms_e2e = max_over_ranks([ms, ms_e2e], dev, world)

    # ---- a short separate pass with an event pair around every entry-point call ---------
    timeline = profiled_pass(job, 3)
    barrier()
    peak_gflops = fp32_peak_gflops(dev) if rank == 0 else None

    extra = {}
    failed = False
    if world > 1:
        extra["dp_check"] = dp_check(job, dev, world)
        failed = not extra["dp_check"]["ok"]
        extra["exchange_timeline_per_rank"] = exchange_timeline(job, dev, world)
        # what the exchange leaves exposed: the same step without exchange and update
        ms_compute = job.timed(5, 1, barrier, update=False)
        (ms_compute,) = max_over_ranks([ms_compute], dev, world)
        extra["exchange_ms_exposed"] = round(ms - ms_compute, 3)
        # strong scaling: the global batch of the single-GPU run (512) split over the ranks
        if HEADLINE["batch"] % (32 * world) == 0:
            sub = HEADLINE["batch"] // world
            small = [(x[:sub].contiguous(), t[:sub].contiguous()) for x, t in zip(job.dev_x, job.dev_t)]

            def strong(n, **kw):
                for i in range(n):
                    job.step(*small[i % job.pool], **kw)

            def timed_strong(**kw):
                strong(3, **kw)
                barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                strong(args.steps, **kw)
                b.record()
                barrier()
                return a.elapsed_time(b) / args.steps

            ms_strong, ms_strong_compute = max_over_ranks([timed_strong(), timed_strong(update=False)], dev, world)
            # the single-GPU step on the whole batch, timed here on every rank without any exchange
            # (full local AdamW on a private copy of the model), slowest rank
            solo = Job(HEADLINE, dev, world, rank, exchange="none")
            (ms_solo,) = max_over_ranks([solo.timed(5, 3, barrier)], dev, world)
            solo.release()
            extra["strong_scaling"] = {
                "global_batch": HEADLINE["batch"], "batch_per_gpu": sub, "ms_per_step": round(ms_strong, 3),
                "samples_per_s": round(HEADLINE["batch"] / (ms_strong * 1e-3), 1),
                "n1_ms_per_step_same_run": round(ms_solo, 3),
                "efficiency_vs_n1": round(ms_solo / (world * ms_strong), 4),
                "exchange_ms_exposed": round(ms_strong - ms_strong_compute, 3)}
            job.opt.check()
    if (world == 8 or (args.configs4 and world > 1)) and not args.no_extras:
        job.release()
        cfg = CONFIGS[4]
        big = Job(cfg, dev, world, rank, exchange=exchange)
        ms_big = big.timed(10, 3, barrier)
        ms_big_compute = big.timed(5, 1, barrier, update=False)
        ms_big, ms_big_compute = max_over_ranks([ms_big, ms_big_compute], dev, world)
        chk = dp_check(big, dev, world)
        failed = failed or not chk["ok"]
        extra["configs[4]"] = {"workload": cfg["label"], "global_batch": cfg["batch"] * world, "batch_per_gpu": cfg["batch"],
                               "parameters": big.opt.numel, "ms_per_step": round(ms_big, 3),
                               "samples_per_s": round(cfg["batch"] * world / (ms_big * 1e-3), 1),
                               "exchange_ms_exposed": round(ms_big - ms_big_compute, 3), "dp_check": chk}
        big.release()

    line = None
    if rank == 0:
        value = world * B / (ms * 1e-3)
        e2e = world * B / (ms_e2e * 1e-3)
        h2d = sum(t.numel() * t.element_size() for t in (in_x[0], in_t[0]))
        line = {
            "metric": "train samples/s (fwd+bwd+IBP step)", "value": round(value, 1), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_block(world, exchange_text),
            "e2e": {"value": round(e2e, 1), "unit": "samples/s", "ms_per_step": round(ms_e2e, 3),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8},
            "gpu_launches": launches,
            "gradient_exchange": exchange_text,
            "clocks": clocks,
        }
        if timeline:
            shares, roofs, dominant, total_kernel_ms = roofline_blocks(timeline, peak_gflops)
            line.update({"roofline": dominant, "roofline_linf_forward": roofs.get("snb_inf_dist_forward_sorted_ws") or roofs.get("snb_inf_dist_forward_ws"),
                         "roofline_linf_point_forward": roofs.get("snb_inf_dist_forward_nograd"),
                         "kernel_time_share": shares, "kernel_ms_per_step": round(total_kernel_ms / 3, 3),
                         "kernel_time_source": "3 extra steps, run operator by operator with a CUDA-event pair around "
                                               "every entry-point call; the headline regions run one library call "
                                               "per layer without those events"})
        line.update(extra)
        if world == 1 and not args.no_extras:
            line["roofline_hbm"] = hbm_block(job)
            lp, lp_roof = lp_blocks(job, peak_gflops, clocks.get("sm_mhz"))
            line["lp_training_step"] = lp
            if lp_roof:
                line["roofline_lp"] = lp_roof
            try:
                cmp_block = gpu_comparator_block(job)
            except Exception as exc:
                cmp_block = {"unavailable": "the reference step failed here: %s" % (str(exc).splitlines() or ["?"])[0]}
            if "ms_per_step" in cmp_block:
                cmp_block["ours_ms_per_step"] = round(ms, 3)
                cmp_block["speedup"] = round(cmp_block["ms_per_step"] / ms, 3)
            line["gpu_comparator"] = cmp_block
            job.release()
            line["configs[0]"] = single_layer_block(dev, peak_gflops)
            line["configs[2]"] = config_step_block(2, dev)
            line["configs[3]"] = config_step_block(3, dev)
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            fns, kind = cpu_functions()
            cpu_step_seconds(64, threads, fns)                      # warm-up
            scaled, info = cpu_step_seconds(256, threads, fns)
            line["cpu_baseline"] = {"value": round(32.0 / scaled, 4), "unit": "samples/s", "cores": threads, "kind": kind,
                                    "sample": CPU_SAMPLE % (256, CPU_HOW[kind], info["raw_seconds"])}
        sys.stdout.flush()
        os.write(result_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit("dp_check failed: the data-parallel step does not match all-reduce + AdamW")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--exchange", default="copies", choices=["copies", "fused", "nccl"],
                    help="gradient exchange at N > 1 (default: overlapped device-to-device copies)")
    ap.add_argument("--configs4", action="store_true", help="run the configs[4] block (width 10240, 128 rows per GPU) at "
                                                           "this N > 1 as well; by default it runs at N = 8 only")
    ap.add_argument("--inject-exchange-failure", action="store_true",
                    help="N > 1: the last rank raises on the host after the warm-up, as if its exchange had failed, "
                         "to exercise the switch to the NCCL exchange")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary blocks (other configurations, finite p, "
                                                              "GPU comparator)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
