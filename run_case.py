"""Runs one operator on one synthetic shape and prints its time (CUDA events).

    python run_case.py --op bound_nograd --B 512 --CI 5120 --CO 5120 --iters 5

Used for quick timing of a single kernel and as the small, self-terminating command that
profilers attach to.  Ops: inf_fwd (argmax words; masked when --keep < 1), inf_fwd_sorted (its ascending-list form), inf_nograd,
inf_bwd, bound_nograd, bound_fwd, lp_fwd, lp_bwd, lp_bwd_x (grad_x only), mean_shift, sort_nograd,
sort_bound, sort_fwd (values + positions), sort_bwd (K = 10, q = 0.9), adamw (the fused optimiser kernel on
--n parameters), bound_pass_update (the model's bound pass with the optimiser update beside it), probe (hardware probes).
"""
import argparse
import ctypes
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from sortnet_b200 import _lib                      # noqa: E402
from sortnet_b200 import norm_dist_cuda as C       # noqa: E402
from sortnet_b200.layers import sample_mask        # noqa: E402

OPS_PER_ELEMENT = {"inf_fwd": 2, "inf_fwd_sorted": 2, "inf_nograd": 2, "bound_nograd": 6, "bound_fwd": 6, "lp_fwd": 4, "lp_bwd": 6, "lp_bwd_x": 6}


PROBES = ["packed sub + max3abs", "2 scalar sub + 2 max", "2 scalar sub + max3abs", "packed sub + 2 max",
          "max3abs alone", "interval-bound step (2 sub, min3, max3 per element)", "p=8 step (sub2, mul2, mul2, fma2)",
          "2 scalar sub + 2 sign clears + integer max3", "integer max3 alone"]


def probe():
    """Times the FP32 FMA probe and every instruction form of the inner step; prints element
    rates per clock per SM using the SM clock NVML reports while the probes run."""
    lib = _lib.load()
    # declared in sortnet_b200/csrc/probe.h (bench-only, not part of the product header)
    lib.snb_probe_step.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_double),
                                   ctypes.c_void_p]
    lib.snb_probe_step.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    scratch = torch.linspace(0, 1, 2 * sms * 256 + 64, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    mhz = None
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(0)
    except Exception:
        h = None

    def timed(launch):
        best = float("inf")
        for _ in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            launch()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return best

    flops = ctypes.c_double()
    for _ in range(3):   # let the clocks ramp
        lib.snb_probe_fp32(scratch.data_ptr(), 1 << 16, ctypes.byref(flops), st)
    torch.cuda.synchronize()
    ms = timed(lambda: lib.snb_probe_fp32(scratch.data_ptr(), 1 << 14, ctypes.byref(flops), st))
    if h is not None:
        mhz = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
    print("FP32 FMA probe: %.1f GFLOP/s (2 flops per FMA), SM clock %s MHz, %d SMs" % (flops.value / ms * 1e-6, mhz, sms))
    clk = (mhz or 1965) * 1e6
    pairs = ctypes.c_double()
    for v, name in enumerate(PROBES):
        ms = timed(lambda: lib.snb_probe_step(v, scratch.data_ptr(), 4000, ctypes.byref(pairs), st))
        elems = 2 * pairs.value
        print("variant %d %-52s %7.3f ms  %6.2f elements/clock/SM  %5.2f issue-cycles per element per scheduler"
              % (v, name, ms, elems / (ms * 1e-3) / clk / sms, 128.0 / (elems / (ms * 1e-3) / clk / sms)))


def adamw(a, dev):
    """The fused flat-buffer AdamW kernel alone on --n parameters (28 bytes of traffic each)."""
    lib = _lib.load()
    n = a.n // 4 * 4
    param, grad = torch.randn(n, device=dev), torch.randn(n, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def run(step):
        _lib.check(lib.snb_adamw_step(param.data_ptr(), grad.data_ptr(), m.data_ptr(), v.data_ptr(), n, 0.02, 0.9,
                                      0.99, 1e-10, 0.0, step, 1.0, stream), "adamw_step")

    for i in range(a.warmup):
        run(1 + i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.iters):
        run(1 + a.warmup + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    print("adamw n=%d: %.4f ms  %.1f GB/s (28 bytes / parameter)" % (n, ms, 28.0 * n / ms * 1e-6))


def bound_pass_update(a, dev):
    """The interval-bound pass of the headline model with the single-GPU optimiser update (sum of one
    gradient part + AdamW into a second parameter buffer, 120.6 M parameters) launched after its second
    layer: --update none | main (same stream) | side (another stream)."""
    import bench
    lib = _lib.load()
    job = bench.Job(bench.HEADLINE, dev, 1, 0, exchange="none")
    job.run(3)
    x, t = job.dev_x[0], job.dev_t[0]
    n = job.opt.numel
    src = job.opt.flat_param
    dst, grad = torch.empty_like(src), torch.randn(n, device=dev) * 1e-3
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    side = torch.cuda.Stream()
    parts = (ctypes.c_void_p * 1)(grad.data_ptr())
    bound_ms = update_ms = 0.0
    for it in range(a.iters + a.warmup):
        main = torch.cuda.current_stream()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ready = torch.cuda.Event()

        def hook(k):
            if k != 1 or a.update == "none":
                return
            stream = main
            if a.update == "side":
                ready.record(main)
                side.wait_event(ready)
                stream = side
            e[2].record(stream)
            _lib.check(lib.snb_adamw_reduce_step(src.data_ptr(), dst.data_ptr(), parts, 1, m.data_ptr(), v.data_ptr(), n,
                                                 0.02, 0.9, 0.99, 1e-10, 0.0, it + 1, 1.0, stream.cuda_stream), "adamw")
            e[3].record(stream)

        e[0].record()
        job.bound_pass(x, t, after_layer=hook)
        e[1].record()
        main.wait_stream(side)
        torch.cuda.synchronize()
        if it >= a.warmup:
            bound_ms += e[0].elapsed_time(e[1])
            if a.update != "none":
                update_ms += e[2].elapsed_time(e[3])
    print("bound pass with the update on '%s': %.3f ms, update kernel %.3f ms" % (a.update, bound_ms / a.iters,
                                                                                 update_ms / a.iters))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True)
    ap.add_argument("--B", type=int, default=512)
    ap.add_argument("--CI", type=int, default=5120)
    ap.add_argument("--CO", type=int, default=5120)
    ap.add_argument("--keep", type=float, default=1.0)
    ap.add_argument("--p", type=float, default=8.0)
    ap.add_argument("--n", type=int, default=30_000_000, help="adamw: number of parameters")
    ap.add_argument("--update", choices=("none", "main", "side"), default="side",
                    help="bound_pass_update: where the optimiser update is launched")
    ap.add_argument("--mask", choices=("both", "ci", "co"), default="both",
                    help="with --keep < 1: which index lists to draw (co = kept rows of W only, like a first layer)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--rotate", type=int, default=1,
                    help="number of weight matrices to rotate through (> 1: the weights of a call are not in L2, "
                         "as inside a network whose layers have different weights)")
    ap.add_argument("--beside-wait-ms", type=float, default=0.0,
                    help="run every timed call beside a barrier kernel on another stream that waits this long for a "
                         "flag nothing sets (what a waiting kernel costs the kernels beside it)")
    a = ap.parse_args()
    if a.op == "probe":
        return probe()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    if a.op == "adamw":
        return adamw(a, dev)
    if a.op == "bound_pass_update":
        return bound_pass_update(a, dev)
    S = (a.B + 31) // 32
    ci = co = None
    if a.keep < 1.0:
        ci = sample_mask(S, 1, a.CI, a.keep, dev) if a.mask in ("both", "ci") else None
        co = sample_mask(S, 1, a.CO, a.keep, dev) if a.mask in ("both", "co") else None
    ci_n = a.CI if ci is None else ci.size(-1)
    co_n = a.CO if co is None else co.size(-1)
    ws = [torch.randn(a.CO, a.CI, device=dev) for _ in range(max(a.rotate, 1))]
    w = ws[0]
    x = torch.rand(a.B, ci_n, 1, device=dev)
    y = torch.empty(a.B, co_n, 1, device=dev)
    pos = torch.zeros(a.B, co_n, 1, device=dev, dtype=torch.int32)
    g = torch.randn(a.B, co_n, 1, device=dev)
    gx, gw = torch.empty_like(x), torch.empty_like(w)
    xl, xu = (x - 0.03).clamp(0, 1), (x + 0.03).clamp(0, 1)
    y2, pos2 = torch.empty_like(y), torch.empty_like(pos)
    mean = torch.empty(a.CO, device=dev)

    if a.op in ("inf_bwd",):
        C.inf_dist_forward(x, w, y, pos, 1, ci, co)
    if a.op in ("lp_bwd", "lp_bwd_x"):
        C.norm_dist_forward(x, w, y, 1, a.p, ci, co)
    SORT_K, SORT_Q = 10, 0.9
    posk = None
    if a.op in ("sort_fwd", "sort_bwd"):
        posk = torch.zeros(SORT_K, a.B, co_n, 1, device=dev, dtype=torch.int32)
        C.sort_neuron_forward(x, w, y, posk, 1, SORT_Q, SORT_K)

    calls = [0]

    def run():
        w = ws[calls[0] % len(ws)]
        calls[0] += 1
        if a.op == "inf_fwd":
            C.inf_dist_forward(x, w, y, pos, 1, ci, co)
        elif a.op == "inf_fwd_sorted":
            C.inf_dist_forward_sorted(x, w, y, pos, ci, co)
        elif a.op == "inf_nograd":
            C.inf_dist_forward_nograd(x, w, y, 1)
        elif a.op == "inf_bwd":
            C.inf_dist_backward_input_weight(g, pos, gx, gw, 1, ci, co)
        elif a.op == "bound_nograd":
            C.bound_inf_dist_forward_nograd(xl, xu, w, y, y2, 1)
        elif a.op == "bound_fwd":
            C.bound_inf_dist_forward(xl, xu, w, y, y2, pos, pos2, 1)
        elif a.op == "lp_fwd":
            C.norm_dist_forward(x, w, y, 1, a.p, ci, co)
        elif a.op == "lp_bwd":
            C.norm_dist_backward_input_weight(g, x, w, y, gx, gw, 1, a.p, ci, co)
        elif a.op == "lp_bwd_x":
            C.norm_dist_backward_input(g, x, w, y, gx, 1, a.p, ci, co)
        elif a.op == "sort_nograd":
            C.sort_neuron_forward_nograd(x, w, y, 1, SORT_Q, SORT_K)
        elif a.op == "sort_bound":
            C.bound_sort_neuron_forward(xl, xu, w, y, y2, 1, SORT_Q, SORT_K)
        elif a.op == "sort_fwd":
            C.sort_neuron_forward(x, w, y, posk, 1, SORT_Q, SORT_K)
        elif a.op == "sort_bwd":
            C.sort_neuron_backward_input_weight(g, posk, gx, gw, 1, SORT_Q, SORT_K)
        elif a.op == "mean_shift":
            C.mean_shift_stats(y.copy_(g), co, mean, None, 0.1)
            C.mean_shift_apply(y, mean, co, y)
        else:
            raise SystemExit("unknown op " + a.op)

    for _ in range(a.warmup):
        run()
    torch.cuda.synchronize()
    if a.beside_wait_ms > 0:
        # two "ranks" whose flag arrays live on this GPU; rank 1 never signals, so the barrier kernel
        # waits until its time limit, records that in `status` and returns
        lib = _lib.load()
        side = torch.cuda.Stream()
        flags = [torch.zeros(4, dtype=torch.int32, device=dev) for _ in range(2)]
        ptrs = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flags])
        status = torch.zeros(1, dtype=torch.int32).pin_memory()
        total = 0.0
        for it in range(a.iters):
            ready = torch.cuda.Event()
            ready.record()
            side.wait_event(ready)
            _lib.check(lib.snb_peer_barrier(ptrs, 0, 2, it + 1, int(a.beside_wait_ms * 1e6), status.data_ptr(),
                                            side.cuda_stream), "peer_barrier")
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        ms = total / a.iters
    else:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
    elems = a.B * ci_n * co_n
    msg = "%s B=%d CI=%d CO=%d: %.4f ms" % (a.op, a.B, ci_n, co_n, ms)
    if a.op in OPS_PER_ELEMENT:
        msg += "  %.1f GOP/s (%d ops/element)" % (OPS_PER_ELEMENT[a.op] * elems / ms * 1e-6, OPS_PER_ELEMENT[a.op])
    print(msg)


if __name__ == "__main__":
    main()
