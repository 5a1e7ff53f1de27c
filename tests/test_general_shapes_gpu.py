"""Grouped (G > 1) and spatial (HW > 1) shapes of every operator on the GPU: the fixtures made by
the reference's PyTorch branches, and seeded cases against the grouped CPU oracle.  l-infinity and
interval-bound values and position words bit-exact, l-p and gradients to 1e-5 relative."""
import numpy as np
import pytest
import torch

from gpu_util import dev, rel
from oracle import general as og

pytestmark = pytest.mark.gpu
INF = float("inf")


def np_(t):
    return t.detach().cpu().numpy()


def masks_g(rng, B, G, C_full, keep):
    """[S, G, count] int32: one count for the layer, a random subset per sub-batch and group (in
    the order the reference's top-k leaves them, i.e. not sorted)."""
    S = (B + 31) // 32
    count = max(int((rng.random(C_full) < keep).sum()), 1)
    return np.stack([[rng.permutation(C_full)[:count] for _ in range(G)] for _ in range(S)]).astype(np.int32)


# ---- fixtures from the reference ------------------------------------------------------------

@pytest.mark.parametrize("name", ["general_inf", "general_inf_hw", "general_p8", "general_p20_groups"])
def test_golden_norm_dist(golden, name):
    from sortnet_b200 import ops
    g = golden(name)
    p, G = float(g["p"]), int(g["G"])
    x = dev(g["x"]).requires_grad_()
    w = dev(g["w"]).requires_grad_()
    y = ops.norm_dist(x, w, p, groups=G)
    y.backward(dev(g["gy"]))
    if p == INF:
        assert np.array_equal(np_(y), g["y"])
    else:
        assert rel(np_(y), g["y"]) < 1e-5
    assert rel(np_(x.grad), g["gx"]) < 1e-5 and rel(np_(w.grad), g["gw"]) < 1e-5


@pytest.mark.parametrize("name", ["general_dropout_inf", "general_dropout_p8"])
def test_golden_dropout(golden, name):
    from sortnet_b200 import ops
    g = golden(name)
    p, G = float(g["p"]), int(g["G"])
    x = dev(g["x"]).requires_grad_()
    w = dev(g["w"]).requires_grad_()
    y = ops.norm_dist_dropout(x, w, dev(g["ci"], torch.int32), dev(g["co"], torch.int32), p, groups=G)
    y.backward(dev(g["gy"]))
    if p == INF:
        assert np.array_equal(np_(y), g["y"])
    else:
        assert rel(np_(y), g["y"]) < 1e-5
    assert rel(np_(x.grad), g["gx"]) < 1e-5 and rel(np_(w.grad), g["gw"]) < 1e-5


def test_golden_bound(golden):
    from sortnet_b200 import ops
    g = golden("general_bound")
    G = int(g["G"])
    xl = dev(g["xl"]).requires_grad_()
    xu = dev(g["xu"]).requires_grad_()
    w = dev(g["w"]).requires_grad_()
    yl, yu = ops.bound_inf_dist(xl, xu, w, groups=G)
    assert np.array_equal(np_(yl), g["yl"]) and np.array_equal(np_(yu), g["yu"])
    ((yl * dev(g["gl"])).sum() + (yu * dev(g["gu"])).sum()).backward()
    assert rel(np_(xl.grad), g["gxl"]) < 1e-5 and rel(np_(xu.grad), g["gxu"]) < 1e-5
    assert rel(np_(w.grad), g["gw"]) < 1e-5
    with torch.no_grad():
        yl2, yu2 = ops.bound_inf_dist(xl.detach(), xu.detach(), w.detach(), groups=G)
    assert torch.equal(yl2, yl) and torch.equal(yu2, yu)


def test_golden_sort(golden):
    from sortnet_b200 import ops
    g = golden("general_sort")
    G, q, K = int(g["G"]), float(g["q"]), int(g["K"])
    x = dev(g["x"]).requires_grad_()
    w = dev(g["w"]).requires_grad_()
    y = ops.sort_neuron(x, w, groups=G, q=q, truncate=K)
    assert rel(np_(y), g["y"]) < 2e-6
    y.backward(dev(g["gy"]))
    assert rel(np_(x.grad), g["gx"]) < 1e-5 and rel(np_(w.grad), g["gw"]) < 1e-5
    with torch.no_grad():
        y2 = ops.sort_neuron(x.detach(), w.detach(), groups=G, q=q, truncate=K)
        yl, yu = ops.bound_sort_neuron(x.detach(), x.detach(), w.detach(), groups=G, q=q, truncate=K)
    assert rel(np_(y2), g["y"]) < 2e-6 and rel(np_(yl), g["y"]) < 2e-6 and rel(np_(yu), g["y"]) < 2e-6


# ---- seeded cases against the grouped oracle ------------------------------------------------

SHAPES = [  # B, G, CIg, COg, HW
    (37, 2, 24, 20, 3),      # partial last sub-batch
    (64, 3, 33, 17, 1),      # groups only, odd sizes
    (10, 1, 19, 7, 5),       # spatial only
    (96, 2, 300, 130, 4),    # several tiles per group
    (33, 4, 8, 5, 2),
]


@pytest.mark.parametrize("B,G,CIg,COg,HW", SHAPES)
def test_inf_vs_oracle(B, G, CIg, COg, HW):
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(B * 7 + G)
    x = rng.random((B, G * CIg, HW), dtype=np.float32)
    w = rng.standard_normal((G * COg, CIg)).astype(np.float32)
    gy = rng.standard_normal((B, G * COg, HW)).astype(np.float32)
    y_o, pos_o = og.inf_dist_forward_g(x, w, G)
    X, W = dev(x), dev(w)
    y = torch.empty(B, G * COg, HW, device="cuda")
    pos = torch.empty(B, G * COg, HW, device="cuda", dtype=torch.int32)
    C.inf_dist_forward(X, W, y, pos, G)
    assert np.array_equal(np_(y), y_o) and np.array_equal(np_(pos), pos_o)
    y2 = torch.empty_like(y)
    C.inf_dist_forward_nograd(X, W, y2, G)
    assert torch.equal(y2, y)
    gx_o, gw_o = og.inf_dist_backward_g(gy, pos_o, G * CIg, w.shape, G)
    gx = torch.full_like(X, float("nan"))
    gw = torch.full_like(W, float("nan"))
    C.inf_dist_backward_input_weight(dev(gy), pos, gx, gw, G)
    assert rel(np_(gx), gx_o) < 1e-5 and rel(np_(gw), gw_o) < 1e-5
    gx2 = torch.full_like(X, float("nan"))
    C.inf_dist_backward_input(dev(gy), pos, gx2, G)
    assert rel(np_(gx2), gx_o) < 1e-5


@pytest.mark.parametrize("B,G,CIg,COg,HW", SHAPES)
@pytest.mark.parametrize("p", [INF, 8.0, 20.0])
def test_masked_vs_oracle(B, G, CIg, COg, HW, p):
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(B * 11 + G + int(min(p, 99)))
    ci = masks_g(rng, B, G, CIg, 0.8)
    co = masks_g(rng, B, G, COg, 0.8)
    CIk, COk = ci.shape[-1], co.shape[-1]
    x = rng.random((B, G * CIk, HW), dtype=np.float32)
    w = rng.standard_normal((G * COg, CIg)).astype(np.float32)
    gy = rng.standard_normal((B, G * COk, HW)).astype(np.float32)
    X, W, GY = dev(x), dev(w), dev(gy)
    CI_, CO_ = dev(ci), dev(co)
    y = torch.empty(B, G * COk, HW, device="cuda")
    gx = torch.full_like(X, float("nan"))
    gw = torch.full_like(W, float("nan"))
    if p == INF:
        y_o, pos_o = og.inf_dist_forward_g(x, w, G, ci, co)
        pos = torch.empty(B, G * COk, HW, device="cuda", dtype=torch.int32)
        C.inf_dist_forward(X, W, y, pos, G, CI_, CO_)
        assert np.array_equal(np_(y), y_o) and np.array_equal(np_(pos), pos_o)
        gx_o, gw_o = og.inf_dist_backward_g(gy, pos_o, G * CIk, w.shape, G, ci, co)
        C.inf_dist_backward_input_weight(GY, pos, gx, gw, G, CI_, CO_)
    else:
        y_o = og.norm_dist_forward_g(x, w, p, G, ci, co)
        C.norm_dist_forward(X, W, y, G, p, CI_, CO_)
        assert rel(np_(y), y_o) < 1e-5
        gx_o, gw_o = og.norm_dist_backward_g(gy, x, w, np_(y), p, G, ci, co)
        C.norm_dist_backward_input_weight(GY, X, W, y, gx, gw, G, p, CI_, CO_)
        gx2 = torch.full_like(X, float("nan"))
        C.norm_dist_backward_input(GY, X, W, y, gx2, G, p, CI_, CO_)
        assert rel(np_(gx2), gx_o) < 1e-5
    assert rel(np_(gx), gx_o) < 1e-5 and rel(np_(gw), gw_o) < 1e-5


@pytest.mark.parametrize("B,G,CIg,COg,HW", SHAPES)
def test_bound_vs_oracle(B, G, CIg, COg, HW):
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(B * 13 + G)
    x = rng.random((B, G * CIg, HW), dtype=np.float32)
    xl = np.clip(x - np.float32(0.05), 0, 1)
    xu = np.clip(x + np.float32(0.05), 0, 1)
    w = rng.standard_normal((G * COg, CIg)).astype(np.float32)
    gl = rng.standard_normal((B, G * COg, HW)).astype(np.float32)
    gu = rng.standard_normal((B, G * COg, HW)).astype(np.float32)
    yl_o, yu_o, pl_o, pu_o = og.bound_inf_dist_forward_g(xl, xu, w, G)
    XL, XU, W = dev(xl), dev(xu), dev(w)
    yl = torch.empty(B, G * COg, HW, device="cuda")
    yu = torch.empty_like(yl)
    pl = torch.empty(B, G * COg, HW, device="cuda", dtype=torch.int32)
    pu = torch.empty_like(pl)
    C.bound_inf_dist_forward(XL, XU, W, yl, yu, pl, pu, G)
    assert np.array_equal(np_(yl), yl_o) and np.array_equal(np_(yu), yu_o)
    assert np.array_equal(np_(pl), pl_o) and np.array_equal(np_(pu), pu_o)
    yl2, yu2 = torch.empty_like(yl), torch.empty_like(yl)
    C.bound_inf_dist_forward_nograd(XL, XU, W, yl2, yu2, G)
    assert torch.equal(yl2, yl) and torch.equal(yu2, yu)
    gxl_o, gxu_o, gw_o = og.bound_inf_dist_backward_g(gl, gu, pl_o, pu_o, G * CIg, G)
    gxl, gxu = torch.full_like(XL, float("nan")), torch.full_like(XL, float("nan"))
    gw = torch.full_like(W, float("nan"))
    C.bound_inf_dist_backward_input_weight(dev(gl), dev(gu), pl, pu, gxl, gxu, gw, G)
    assert rel(np_(gxl), gxl_o) < 1e-5 and rel(np_(gxu), gxu_o) < 1e-5 and rel(np_(gw), gw_o) < 1e-5
    gxl2, gxu2 = torch.full_like(XL, float("nan")), torch.full_like(XL, float("nan"))
    C.bound_inf_dist_backward_input(dev(gl), dev(gu), pl, pu, gxl2, gxu2, G)
    assert rel(np_(gxl2), gxl_o) < 1e-5 and rel(np_(gxu2), gxu_o) < 1e-5


@pytest.mark.parametrize("B,G,CIg,COg,HW", SHAPES[:3] + SHAPES[4:])
def test_sort_vs_oracle(B, G, CIg, COg, HW):
    from sortnet_b200 import norm_dist_cuda as C
    q, K = 0.7, min(6, CIg)
    rng = np.random.default_rng(B * 17 + G)
    x = rng.random((B, G * CIg, HW), dtype=np.float32)
    w = rng.standard_normal((G * COg, CIg)).astype(np.float32)
    gy = rng.standard_normal((B, G * COg, HW)).astype(np.float32)
    y_o, pos_o = og.sort_forward_g(x, w, q, K, G)
    X, W = dev(x), dev(w)
    y = torch.empty(B, G * COg, HW, device="cuda")
    pos = torch.empty(K, B, G * COg, HW, device="cuda", dtype=torch.int32)
    C.sort_neuron_forward(X, W, y, pos, G, q, K)
    assert rel(np_(y), y_o) < 2e-6 and np.array_equal(np_(pos), pos_o)
    y2 = torch.empty_like(y)
    C.sort_neuron_forward_nograd(X, W, y2, G, q, K)
    assert rel(np_(y2), y_o) < 2e-6
    gx_o, gw_o = og.sort_backward_g(gy, pos_o, G * CIg, q, K, G)
    gx = torch.full_like(X, float("nan"))
    gw = torch.full_like(W, float("nan"))
    C.sort_neuron_backward_input_weight(dev(gy), pos, gx, gw, G, q, K)
    assert rel(np_(gx), gx_o) < 1e-5 and rel(np_(gw), gw_o) < 1e-5
    xl = np.clip(x - np.float32(0.03), 0, 1)
    xu = np.clip(x + np.float32(0.03), 0, 1)
    yl_o, yu_o = og.sort_bound_forward_g(xl, xu, w, q, K, G)
    yl, yu = torch.empty_like(y), torch.empty_like(y)
    C.bound_sort_neuron_forward(dev(xl), dev(xu), W, yl, yu, G, q, K)
    assert rel(np_(yl), yl_o) < 2e-6 and rel(np_(yu), yu_o) < 2e-6


def test_bad_group_shapes_are_rejected():
    from sortnet_b200 import norm_dist_cuda as C
    x = torch.zeros(4, 10, 2, device="cuda")
    w = torch.zeros(6, 5, device="cuda")
    y = torch.empty(4, 6, 2, device="cuda")
    with pytest.raises(RuntimeError):
        C.inf_dist_forward_nograd(x, w, y, 3)          # 10 channels do not split into 3 groups
    ci = torch.zeros(1, 1, 5, device="cuda", dtype=torch.int32)
    pos = torch.empty(4, 6, 2, device="cuda", dtype=torch.int32)
    with pytest.raises(RuntimeError):
        C.inf_dist_forward(x, w, y, pos, 2, ci, None)  # index list lacks the group dimension
