"""Runs one operator on one synthetic shape and prints its time (CUDA events).

    python -m sortnet_b200.run_case --op bound_nograd --B 512 --CI 5120 --CO 5120 --iters 5

Used for quick timing of a single kernel and as the small, self-terminating command that
profilers attach to.  Ops: inf_fwd (argmax words; masked when --keep < 1), inf_nograd,
inf_bwd, bound_nograd, bound_fwd, lp_fwd, lp_bwd, mean_shift.
"""
import argparse

import torch

from . import norm_dist_cuda as C
from .layers import sample_mask

OPS_PER_ELEMENT = {"inf_fwd": 2, "inf_nograd": 2, "bound_nograd": 6, "bound_fwd": 6, "lp_fwd": 4, "lp_bwd": 6}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True)
    ap.add_argument("--B", type=int, default=512)
    ap.add_argument("--CI", type=int, default=5120)
    ap.add_argument("--CO", type=int, default=5120)
    ap.add_argument("--keep", type=float, default=1.0)
    ap.add_argument("--p", type=float, default=8.0)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    S = (a.B + 31) // 32
    ci = co = None
    if a.keep < 1.0:
        ci = sample_mask(S, 1, a.CI, a.keep, dev)
        co = sample_mask(S, 1, a.CO, a.keep, dev)
    ci_n = a.CI if ci is None else ci.size(-1)
    co_n = a.CO if co is None else co.size(-1)
    w = torch.randn(a.CO, a.CI, device=dev)
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
    if a.op == "lp_bwd":
        C.norm_dist_forward(x, w, y, 1, a.p, ci, co)

    def run():
        if a.op == "inf_fwd":
            C.inf_dist_forward(x, w, y, pos, 1, ci, co)
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
        elif a.op == "mean_shift":
            C.mean_shift_stats(y.copy_(g), co, mean, None, 0.1)
            C.mean_shift_apply(y, mean, co, y)
        else:
            raise SystemExit("unknown op " + a.op)

    for _ in range(a.warmup):
        run()
    torch.cuda.synchronize()
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
