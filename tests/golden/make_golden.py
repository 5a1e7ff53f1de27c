"""Generate the golden fixtures in this directory from the reference's own Python code.

Run once, in a container that has the reference checkout (path in $SORTNET_REFERENCE, default
a directory `reference` beside this repository):   python tests/golden/make_golden.py

The reference's pure-PyTorch branches are imported unmodified with a CPU stand-in for
its CUDA extension module, evaluated on CPU on small seeded inputs, and their outputs and
autograd gradients are stored as .npz files.  The tests then check the CPU oracle (and,
through it, the CUDA kernels) against these files; nothing at test time reads the
reference checkout.

Branches used: core/norm_dist.py:180-185 (norm_dist), :194-213 (norm_dist_dropout, with the
inner norm_dist call forced onto the PyTorch branch), :224-230 (sort_neuron), :250-259
(bound_inf_dist); core/models/bound_basic_module.py:123-157 (MeanShiftDropout);
core/models/norm_dist.py:14-17 (sample_mask).
"""
import functools
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

ROOT = os.path.dirname(os.path.dirname(HERE))
# checkout of zbh2047/SortNet: $SORTNET_REFERENCE, else a directory "reference" beside this repository
REF = os.environ.get("SORTNET_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
sys.path.insert(0, ROOT)
from oracle import ref_module  # noqa: E402

# Stand-in for the reference's CUDA extension: the PyTorch branches never call it; the
# model-level case runs the reference's autograd Functions on it (oracle/ref_module.py).
ref_module.install()
sys.path.insert(0, REF)
import core.norm_dist as ref_ops  # noqa: E402
from core.models.bound_basic_module import MeanShiftDropout  # noqa: E402
from core.models.norm_dist import sample_mask  # noqa: E402

INF = float("inf")


def gen(seed, B, CI, CO):
    g = torch.Generator().manual_seed(seed)
    x = torch.rand(B, CI, generator=g)
    w = torch.randn(CO, CI, generator=g)
    gy = torch.randn(B, CO, generator=g)
    return x, w, gy


def no_ties_inf(x, w):
    d = (x[:, None, :] - w[None]).abs()
    top2 = d.topk(2, dim=-1)[0]
    return bool((top2[..., 0] > top2[..., 1]).all())


def case_norm_dist(seed, B, CI, CO, p):
    x, w, gy = gen(seed, B, CI, CO)
    if p == INF:
        assert no_ties_inf(x, w), "pick another seed: tie in the max"
    x3 = x.unsqueeze(-1).requires_grad_()
    wp = w.clone().requires_grad_()
    y = ref_ops.norm_dist(x3, wp, p, use_custom_cuda_func=False)
    y.backward(gy.unsqueeze(-1))
    return dict(x=x, w=w, gy=gy, p=np.float64(p), y=y.detach().squeeze(-1),
                gx=x3.grad.squeeze(-1), gw=wp.grad)


def case_dropout(seed, B, CI_full, CO_full, q, p):
    torch.manual_seed(seed)
    S = (B - 1) // 32 + 1
    ci = sample_mask(S, 1, CI_full, q, device="cpu")
    co = sample_mask(S, 1, CO_full, q, device="cpu")
    g = torch.Generator().manual_seed(seed + 1000)
    x = torch.rand(B, ci.size(-1), generator=g)
    w = torch.randn(CO_full, CI_full, generator=g)
    gy = torch.randn(B, co.size(-1), generator=g)
    x3 = x.unsqueeze(-1).requires_grad_()
    wp = w.clone().requires_grad_()
    saved = ref_ops.norm_dist
    ref_ops.norm_dist = functools.partial(saved, use_custom_cuda_func=False)
    try:
        y = ref_ops.norm_dist_dropout(x3, wp, ci, co, p, use_custom_cuda_func=False)
    finally:
        ref_ops.norm_dist = saved
    y.backward(gy.unsqueeze(-1))
    if p == INF:
        for s in range(S):
            ws = w[co[s, 0].long()][:, ci[s, 0].long()]
            assert no_ties_inf(x[s * 32:(s + 1) * 32], ws), "pick another seed"
    return dict(x=x, w=w, gy=gy, p=np.float64(p), ci=ci[:, 0], co=co[:, 0],
                y=y.detach().squeeze(-1), gx=x3.grad.squeeze(-1), gw=wp.grad)


def case_bound(seed, B, CI, CO, eps):
    x, w, gl = gen(seed, B, CI, CO)
    gu = torch.randn(B, CO, generator=torch.Generator().manual_seed(seed + 7))
    xl = (x - eps).clamp(0, 1)
    xu = (x + eps).clamp(0, 1)
    l3 = xl.unsqueeze(-1).requires_grad_()
    u3 = xu.unsqueeze(-1).requires_grad_()
    wp = w.clone().requires_grad_()
    yl, yu = ref_ops.bound_inf_dist(l3, u3, wp, use_custom_cuda_func=False)
    # uniqueness of the extremal coordinate, so autograd and the index rule agree
    x1 = w[None] - xl[:, None, :]
    x2 = xu[:, None, :] - w[None]
    hi = torch.maximum(x1, x2).topk(2, dim=-1)[0]
    lo = (-torch.minimum(x1, x2)).topk(2, dim=-1)[0]
    assert bool((hi[..., 0] > hi[..., 1]).all()) and bool((lo[..., 0] > lo[..., 1]).all())
    assert bool((x1 != x2).all())
    (yl * gl.unsqueeze(-1)).sum().add((yu * gu.unsqueeze(-1)).sum()).backward()
    return dict(xl=xl, xu=xu, w=w, gl=gl, gu=gu, yl=yl.detach().squeeze(-1),
                yu=yu.detach().squeeze(-1), gxl=l3.grad.squeeze(-1), gxu=u3.grad.squeeze(-1),
                gw=wp.grad)


def case_sort(seed, B, CI, CO, q, K):
    x, w, _ = gen(seed, B, CI, CO)
    y = ref_ops.sort_neuron(x.unsqueeze(-1), w, q=q, truncate=K, use_custom_cuda_func=False)
    return dict(x=x, w=w, q=np.float64(q), K=np.int64(K), y=y.squeeze(-1))


def case_mean_shift(seed, B, C_full, q):
    torch.manual_seed(seed)
    S = (B - 1) // 32 + 1
    out = {}
    m = MeanShiftDropout(C_full, affine=False)
    m.running_mean.copy_(torch.randn(C_full))
    out["running_mean0"] = m.running_mean.clone()
    if q is None:
        index = None
        C = C_full
    else:
        index = sample_mask(S, 1, C_full, q, device="cpu")
        C = index.size(-1)
        out["index"] = index[:, 0]
    x = torch.randn(B, C, 1, requires_grad=True)
    gy = torch.randn(B, C, 1)
    m.train()
    y, _, _ = m(x, None, None, index=None if index is None else index.long())
    y.backward(gy)
    out.update(x=x.detach().squeeze(-1), gy=gy.squeeze(-1), y=y.detach().squeeze(-1),
               gx=x.grad.squeeze(-1), running_mean1=m.running_mean.clone())
    m.eval()
    lo = x.detach() - 0.1
    up = x.detach() + 0.2
    if index is None:
        ye, le, ue = m(x.detach(), lo, up)
        out.update(eval_y=ye.squeeze(-1), eval_l=le.squeeze(-1), eval_u=ue.squeeze(-1))
    return out


def case_model(seed, B, depth, width, input_dim, classes, q, p, eps):
    """The reference's unmodified SortMLPModel on CPU, with its CUDA extension replaced by the
    oracle-backed stand-in (oracle/ref_module.py) and its mask sampler fed fixed masks."""
    import ell_inf_models
    ref_layers = sys.modules["core.models.norm_dist"]
    ref_layers.NormDistBase.dropout_list = dict()
    ref_layers.NormDistBase.dropout_buffer = None
    ref_layers.NormDistBase.tag = 0
    torch.manual_seed(seed)
    model = ell_inf_models.SortMLPModel(depth=depth, width=width, input_dim=input_dim,
                                        num_classes=classes, dropout=q)
    for m in model.modules():
        if isinstance(m, ref_layers.NormDistBase):
            m.p = p
    S = (B - 1) // 32 + 1
    masks = [sample_mask(S, 1, width, q, device="cpu") for _ in range(depth - 1)]
    feed = iter(masks)
    ref_layers.sample_mask = lambda *a, **k: next(feed)
    x = torch.rand(B, *input_dim)
    targets = torch.randint(0, classes, (B,))
    out = {"x": x.reshape(B, -1), "targets": targets, "p": np.float64(p), "eps": np.float64(eps),
           "q": np.float64(q)}
    for i, mk in enumerate(masks):
        out["mask%d" % i] = mk[:, 0]
    state0 = {k: v.clone() for k, v in model.state_dict().items()}
    model.train()
    logits, margin = model(x, targets=targets, eps=eps)
    loss = margin.clamp(min=0).max(dim=1)[0].mean() + 0.5 * torch.nn.functional.cross_entropy(logits, targets)
    loss.backward()
    out.update(logits=logits.detach(), margin=margin.detach(), loss=loss.detach())
    for k, v in state0.items():
        out["state0." + k] = v
    for k, v in model.state_dict().items():
        if "running_mean" in k:
            out["state1." + k] = v
    for k, prm in model.named_parameters():
        out["grad." + k] = prm.grad
    if q == 1.0 and math.isinf(p):
        model.eval()
        with torch.no_grad():
            lg, mg = model(x, targets=targets, eps=eps, up=torch.ones(1), down=torch.zeros(1))
        out.update(eval_logits=lg, eval_margin=mg)
    return out


# ---- grouped / spatial shapes: x [B, G*CIg, HW], w [G*COg, CIg] ------------------------------

def gen_g(seed, B, G, CIg, COg, HW):
    g = torch.Generator().manual_seed(seed)
    x = torch.rand(B, G * CIg, HW, generator=g)
    w = torch.randn(G * COg, CIg, generator=g)
    gy = torch.randn(B, G * COg, HW, generator=g)
    return x, w, gy


def no_ties_inf_g(x, w, G):
    B, C, HW = x.shape
    d = (x.view(B, G, 1, -1, HW) - w.view(G, -1, w.size(-1), 1)).abs()
    top2 = d.topk(2, dim=3)[0]
    return bool((top2[:, :, :, 0] > top2[:, :, :, 1]).all())


def case_norm_dist_g(seed, B, G, CIg, COg, HW, p):
    x, w, gy = gen_g(seed, B, G, CIg, COg, HW)
    if p == INF:
        assert no_ties_inf_g(x, w, G), "pick another seed: tie in the max"
    xp = x.clone().requires_grad_()
    wp = w.clone().requires_grad_()
    y = ref_ops.norm_dist(xp, wp, p, groups=G, use_custom_cuda_func=False)
    y.backward(gy)
    return dict(x=x, w=w, gy=gy, p=np.float64(p), G=np.int64(G), y=y.detach(), gx=xp.grad, gw=wp.grad)


def case_dropout_g(seed, B, G, CIg_full, COg_full, HW, q, p):
    torch.manual_seed(seed)
    S = (B - 1) // 32 + 1
    ci = sample_mask(S, G, CIg_full, q, device="cpu")
    co = sample_mask(S, G, COg_full, q, device="cpu")
    g = torch.Generator().manual_seed(seed + 1000)
    x = torch.rand(B, G * ci.size(-1), HW, generator=g)
    w = torch.randn(G * COg_full, CIg_full, generator=g)
    gy = torch.randn(B, G * co.size(-1), HW, generator=g)
    xp = x.clone().requires_grad_()
    wp = w.clone().requires_grad_()
    saved = ref_ops.norm_dist
    ref_ops.norm_dist = functools.partial(saved, use_custom_cuda_func=False)
    try:
        y = ref_ops.norm_dist_dropout(xp, wp, ci, co, p, groups=G, use_custom_cuda_func=False)
    finally:
        ref_ops.norm_dist = saved
    y.backward(gy)
    if p == INF:
        w3 = w.view(G, COg_full, CIg_full)
        for s in range(S):
            ws = torch.stack([w3[k][co[s, k].long()][:, ci[s, k].long()] for k in range(G)])
            assert no_ties_inf_g(x[s * 32:(s + 1) * 32], ws.view(-1, ws.size(-1)), G), "pick another seed"
    return dict(x=x, w=w, gy=gy, p=np.float64(p), G=np.int64(G), ci=ci, co=co, y=y.detach(),
                gx=xp.grad, gw=wp.grad)


def case_bound_g(seed, B, G, CIg, COg, HW, eps):
    x, w, gl = gen_g(seed, B, G, CIg, COg, HW)
    gu = torch.randn(gl.shape, generator=torch.Generator().manual_seed(seed + 7))
    xl = (x - eps).clamp(0, 1)
    xu = (x + eps).clamp(0, 1)
    lp = xl.clone().requires_grad_()
    up = xu.clone().requires_grad_()
    wp = w.clone().requires_grad_()
    yl, yu = ref_ops.bound_inf_dist(lp, up, wp, groups=G, use_custom_cuda_func=False)
    w4 = w.view(G, -1, w.size(-1), 1)
    x1 = w4 - xl.view(B, G, 1, -1, HW)
    x2 = xu.view(B, G, 1, -1, HW) - w4
    hi = torch.maximum(x1, x2).topk(2, dim=3)[0]
    lo = (-torch.minimum(x1, x2)).topk(2, dim=3)[0]
    assert bool((hi[:, :, :, 0] > hi[:, :, :, 1]).all()) and bool((lo[:, :, :, 0] > lo[:, :, :, 1]).all())
    assert bool((x1 != x2).all())
    (yl * gl).sum().add((yu * gu).sum()).backward()
    return dict(xl=xl, xu=xu, w=w, gl=gl, gu=gu, G=np.int64(G), yl=yl.detach(), yu=yu.detach(),
                gxl=lp.grad, gxu=up.grad, gw=wp.grad)


def case_sort_g(seed, B, G, CIg, COg, HW, q, K):
    x, w, gy = gen_g(seed, B, G, CIg, COg, HW)
    xp = x.clone().requires_grad_()
    wp = w.clone().requires_grad_()
    y = ref_ops.sort_neuron(xp, wp, groups=G, q=q, truncate=K, use_custom_cuda_func=False)
    y.backward(gy)
    return dict(x=x, w=w, gy=gy, q=np.float64(q), K=np.int64(K), G=np.int64(G), y=y.detach(),
                gx=xp.grad, gw=wp.grad)


def case_conv_stack(seed, B, q, p):
    """Three of the reference's NormDistConv layers (3x3 grouped, then two 1x1) run through its
    PyTorch branches: training forward/backward (masked when q < 1), then evaluation (sort neurons
    when q < 1; interval bounds when q == 1 and p == inf)."""
    ref_layers = sys.modules["core.models.norm_dist"]
    ref_layers.NormDistBase.dropout_list = dict()
    ref_layers.NormDistBase.dropout_buffer = None
    ref_layers.NormDistBase.tag = 0
    torch.manual_seed(seed)
    drop = None if q == 1.0 else q
    G = 2
    layers = [ref_layers.NormDistConv(4, 12, 3, stride=1, groups=G, bias=False, mean_shift=True, p=p),
              ref_layers.NormDistConv(12, 12, 1, groups=G, bias=True, mean_shift=True, dropout=drop, p=p),
              ref_layers.NormDistConv(12, 8, 1, groups=G, bias=True, mean_shift=False, dropout=drop, p=p)]
    with torch.no_grad():
        for l in layers:
            if l.bias is not None:
                l.bias.normal_()
    S = (B - 1) // 32 + 1
    masks = [sample_mask(S, G, 6, q, device="cpu").sort(dim=-1)[0] for _ in range(2)] if drop else []
    feed = iter(masks)
    saved = {n: getattr(ref_layers, n) for n in ("sample_mask", "norm_dist", "norm_dist_dropout",
                                                  "bound_inf_dist", "sort_neuron")}
    saved_ops = ref_ops.norm_dist
    ref_layers.sample_mask = lambda *a, **k: next(feed)
    ref_ops.norm_dist = functools.partial(saved_ops, use_custom_cuda_func=False)
    for n in ("norm_dist", "norm_dist_dropout", "bound_inf_dist", "sort_neuron"):
        setattr(ref_layers, n, functools.partial(getattr(ref_ops, n), use_custom_cuda_func=False))
    try:
        x = torch.rand(B, 4, 5, 5)
        gy = torch.randn(B, 8, 3, 3)
        out = {"x": x, "gy": gy, "p": np.float64(p), "q": np.float64(q), "G": np.int64(G)}
        for i, mk in enumerate(masks):
            out["mask%d" % i] = mk
        for i, l in enumerate(layers):
            for k, v in l.state_dict().items():
                out["state0.%d.%s" % (i, k)] = v.clone()
            l.train()
        xp = x.clone().requires_grad_()
        z = (xp, None, None)
        for l in layers:
            z = l(*z)
        z[0].backward(gy)
        out.update(y=z[0].detach(), gx=xp.grad)
        for i, l in enumerate(layers):
            for k, prm in l.named_parameters():
                out["grad.%d.%s" % (i, k)] = prm.grad
            if l.mean_shift is not None:
                out["state1.%d.mean_shift.running_mean" % i] = l.mean_shift.running_mean.clone()
            l.eval()
        with torch.no_grad():
            if drop is None and math.isinf(p):
                z = (x, (x - 0.05).clamp(0, 1), (x + 0.05).clamp(0, 1))
            else:
                z = (x, None, None)
            if math.isinf(p):
                for l in layers:
                    z = l(*z)
                out["eval_y"] = z[0]
                if z[1] is not None:
                    out.update(eval_lower=z[1], eval_upper=z[2])
    finally:
        for n, f in saved.items():
            setattr(ref_layers, n, f)
        ref_ops.norm_dist = saved_ops
        ref_layers.NormDistBase.dropout_list = dict()
        ref_layers.NormDistBase.dropout_buffer = None
    return out


def save(name, d):
    arrs = {k: (v.detach().numpy() if torch.is_tensor(v) else np.asarray(v)) for k, v in d.items()}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrs)
    print(name, {k: tuple(a.shape) for k, a in arrs.items()})


def main():
    """With arguments, only the fixtures whose name starts with one of them are (re)written."""
    torch.set_num_threads(8)
    want = sys.argv[1:]
    cases = [
        ("norm_dist_inf_a", case_norm_dist, (0, 70, 48, 40, INF,)),
        ("norm_dist_inf_b", case_norm_dist, (1, 33, 17, 5, INF,)),
        ("norm_dist_p2", case_norm_dist, (2, 37, 29, 21, 2.0,)),
        ("norm_dist_p8", case_norm_dist, (3, 70, 48, 40, 8.0,)),
        ("norm_dist_p31", case_norm_dist, (4, 40, 50, 24, 31.6,)),
        ("norm_dist_p3", case_norm_dist, (5, 19, 23, 11, 3.0,)),
        ("dropout_inf", case_dropout, (10, 70, 48, 40, 0.8, INF,)),
        ("dropout_p8", case_dropout, (11, 70, 48, 40, 0.8, 8.0,)),
        ("dropout_p20", case_dropout, (12, 45, 30, 36, 0.7, 20.0,)),
        ("bound_a", case_bound, (20, 70, 48, 40, 0.3,)),
        ("bound_b", case_bound, (21, 33, 17, 5, 0.03,)),
        ("sort_a", case_sort, (30, 20, 48, 12, 0.6, 10,)),
        ("mean_shift_masked", case_mean_shift, (40, 70, 40, 0.8,)),
        ("mean_shift_plain", case_mean_shift, (41, 45, 24, None,)),
        ("model_inf_masked", case_model, (50, 70, 4, 96, (3, 4, 4), 10, 0.8, INF, 0.03,)),
        ("model_p8_masked", case_model, (51, 70, 4, 96, (3, 4, 4), 10, 0.8, 8.0, 0.03,)),
        ("model_inf_plain", case_model, (52, 45, 3, 64, (3, 4, 4), 10, 1.0, INF, 0.03,)),
        ("general_inf", case_norm_dist_g, (60, 37, 2, 24, 20, 3, INF,)),
        ("general_inf_hw", case_norm_dist_g, (61, 10, 1, 19, 7, 5, INF,)),
        ("general_p8", case_norm_dist_g, (62, 37, 2, 24, 20, 3, 8.0,)),
        ("general_p20_groups", case_norm_dist_g, (63, 21, 3, 16, 9, 1, 20.0,)),
        ("general_dropout_inf", case_dropout_g, (64, 40, 2, 30, 26, 3, 0.8, INF,)),
        ("general_dropout_p8", case_dropout_g, (65, 40, 2, 30, 26, 3, 0.8, 8.0,)),
        ("general_bound", case_bound_g, (66, 37, 2, 24, 20, 3, 0.1,)),
        ("general_sort", case_sort_g, (67, 12, 2, 24, 8, 3, 0.6, 6,)),
        ("conv_stack_masked_inf", case_conv_stack, (70, 40, 0.7, INF,)),
        ("conv_stack_masked_p8", case_conv_stack, (71, 40, 0.7, 8.0,)),
        ("conv_stack_plain_inf", case_conv_stack, (72, 37, 1.0, INF,)),
    ]
    for name, fn, args in cases:
        if not want or any(name.startswith(p) for p in want):
            save(name, fn(*args))

if __name__ == "__main__":
    main()
