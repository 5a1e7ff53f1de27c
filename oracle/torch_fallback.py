"""CPU baseline: the reference's pure-PyTorch way of computing this path, restated.

TEST / BENCHMARK INFRASTRUCTURE ONLY (the `cpu_baseline` leg and `--impl reference`).

The reference's operators have a `use_custom_cuda_func=False` branch that evaluates the
distances with ordinary PyTorch tensor ops: it materialises the [rows, outputs, inputs]
difference tensor and reduces it with torch.norm (core/norm_dist.py:180-185 for the point
value with the detached max-normalisation, :194-213 for the masked variant which gathers the
kept rows / columns of W per sub-batch first, :250-259 for the interval bounds), and gets
gradients from autograd.  The functions below do the same tensor operations in the same
order on CPU tensors, on a slice of the workload small enough to time in seconds:
32 rows (one sub-batch) x `out_slice` outputs per wide layer x all inputs.  Cost is linear
in rows and outputs, so the slice time scales to the full layer.
"""
import math
import time

import torch


def lp_distance(x, w, p):
    """x [R, CI], w [CO, CI] -> [R, CO]; difference tensor, detached l-inf normaliser, l-p norm."""
    d = x.unsqueeze(1) - w.unsqueeze(0)
    with torch.no_grad():
        scale = torch.norm(d, dim=2, p=float("inf"), keepdim=True)
    return (torch.norm(d / scale, dim=2, p=p, keepdim=True) * scale).squeeze(2)


def masked_lp_distance(x, w, ci, co, p):
    """One sub-batch: pick the kept rows (co) and columns (ci) of w, then the dense distance."""
    ws = w
    if co is not None:
        ws = ws[co.long()]
    if ci is not None:
        ws = ws[:, ci.long()]
    return lp_distance(x, ws, p)


def interval_bounds(xl, xu, w):
    a = w.unsqueeze(0) - xl.unsqueeze(1)
    b = xu.unsqueeze(1) - w.unsqueeze(0)
    hi = torch.maximum(a, b).clamp(min=1e-10)
    lo = torch.minimum(a, b).clamp(max=-1e-10)
    return torch.norm(-lo, dim=2, p=float("inf")), torch.norm(hi, dim=2, p=float("inf"))


def reference_functions():
    """The reference's own operator functions on their PyTorch branches, when the reference's Python
    has been staged under oracle/_ref/py (oracle/build_ref.py): (distance, bounds) taking the 2-D
    tensors used here, or None.  `norm_dist(..., use_custom_cuda_func=False)` is
    core/norm_dist.py:180-185, `bound_inf_dist(..., use_custom_cuda_func=False)` is :250-259."""
    import types
    from . import build_ref
    if build_ref.staged_python() is None:
        return None
    stub = types.ModuleType("norm_dist_cuda")          # the PyTorch branches never touch the extension
    ops, _, _ = build_ref.import_reference_python(stub)

    def distance(x, w, p):
        return ops.norm_dist(x.unsqueeze(-1), w, p, use_custom_cuda_func=False).squeeze(-1)

    def bounds(xl, xu, w):
        lo, hi = ops.bound_inf_dist(xl.unsqueeze(-1), xu.unsqueeze(-1), w, use_custom_cuda_func=False)
        return lo.squeeze(-1), hi.squeeze(-1)

    return distance, bounds


def time_training_slice(layer_dims, keep, p, eps, out_slice=128, rows=32, seed=0, functions=None):
    """Times, layer by layer, (a) forward + autograd backward of the masked distance and
    (b) the dense interval-bound forward, on `rows` rows x `out_slice` outputs x all inputs
    (a fresh graph per layer, so only one layer's difference tensors are alive).  Each part
    is scaled by (outputs of the full layer / outputs of the slice).  Returns the scaled
    seconds for `rows` rows of the whole step and a breakdown.

    `functions` = (distance, bounds) replaces the restated formulas by the reference's own
    functions (see reference_functions()).  The masked layer is what the reference's
    `norm_dist_dropout` PyTorch branch does for one sub-batch (core/norm_dist.py:194-213): gather
    the kept rows and columns of W, then the dense distance.  The weight leaf here is the
    `out_slice` kept rows only, so the backward's cost (including the zero-filled gradient of
    the gathered columns) scales with the outputs like the rest."""
    distance, bounds = functions if functions is not None else (lp_distance, interval_bounds)
    g = torch.Generator().manual_seed(seed)
    total, raw, details = 0.0, 0.0, []
    for k, (ci_full, co_full) in enumerate(layer_dims):
        first, last = k == 0, k == len(layer_dims) - 1
        ci_kept = ci_full if first else max(1, int(round(keep * ci_full)))
        co_kept = co_full if last else max(1, int(round(keep * co_full)))
        co_s = min(out_slice, co_kept)
        w_rows = torch.randn(co_s, ci_full, generator=g).requires_grad_()      # the kept rows of W
        x = torch.rand(rows, ci_kept, generator=g).requires_grad_()
        ci = None if (first or ci_kept == ci_full) else torch.randperm(ci_full, generator=g)[:ci_kept].sort()[0]
        gy = torch.randn(rows, co_s, generator=g)
        xl = (torch.rand(rows, ci_full, generator=g) - eps).clamp(0, 1)
        xu = (xl + 2 * eps).clamp(0, 1)
        t0 = time.perf_counter()
        ws = w_rows if ci is None else w_rows[:, ci]
        y = distance(x, ws, p)
        y.backward(gy)
        t1 = time.perf_counter()
        with torch.no_grad():
            bounds(xl, xu, w_rows.detach())
        t2 = time.perf_counter()
        train_s, bound_s = t1 - t0, t2 - t1
        raw += train_s + bound_s
        total += train_s * (co_kept / co_s) + bound_s * (co_full / co_s)
        details.append({"layer": k, "inputs": ci_kept, "outputs_timed": co_s, "train_s": round(train_s, 4),
                        "bound_s": round(bound_s, 4)})
        del w_rows, x, y
    return total, {"raw_seconds": raw, "layers": details}
