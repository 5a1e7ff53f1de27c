"""GPU parity of the sort-neuron kernels: values to 2e-6 relative (the weighted sum is a handful
of fp32 multiply-adds whose contraction the compiler chooses), positions exact, gradients 1e-5."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import col3, dev, host, rel

pytestmark = pytest.mark.gpu
VTOL = 2e-6


def test_golden_forward(golden):
    from sortnet_b200 import ops
    g = golden("sort_a")
    with torch.no_grad():
        y = ops.sort_neuron(col3(g["x"]), dev(g["w"]), q=float(g["q"]), truncate=int(g["K"]))
    assert rel(host(y), g["y"]) < VTOL


@pytest.mark.parametrize("B,CI,CO,q,K", [(20, 48, 12, 0.6, 10), (70, 130, 100, 0.9, 10), (33, 17, 70, 0.75, 10),
                                         (64, 300, 65, 0.5, 4), (40, 64, 40, 0.85, 25), (5, 3, 2, 0.7, 3),
                                         (128, 784, 256, 0.9, 10)])
def test_vs_oracle(B, CI, CO, q, K):
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(B + CO)
    x = rng.random((B, CI), dtype=np.float32)
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    y_o, pos_o = oracle.sort_forward(x, w, q, K)
    X, W = col3(x), dev(w)
    y = torch.empty(B, CO, 1, device="cuda")
    C.sort_neuron_forward_nograd(X, W, y, 1, q, K)
    assert rel(host(y), y_o) < VTOL
    y2 = torch.empty(B, CO, 1, device="cuda")
    pos = torch.empty(K, B, CO, 1, device="cuda", dtype=torch.int32)
    C.sort_neuron_forward(X, W, y2, pos, 1, q, K)
    assert rel(host(y2), y_o) < VTOL
    assert np.array_equal(pos.squeeze(-1).cpu().numpy(), pos_o)
    g = rng.standard_normal((B, CO)).astype(np.float32)
    gx_o, gw_o = oracle.sort_backward(g, pos_o, CI, q, K)
    gx = torch.full((B, CI, 1), float("nan"), device="cuda")
    gw = torch.full((CO, CI), float("nan"), device="cuda")
    C.sort_neuron_backward_input_weight(col3(g), pos, gx, gw, 1, q, K)
    assert rel(host(gx), gx_o) < 1e-5 and rel(gw.cpu().numpy(), gw_o) < 1e-5
    gx2 = torch.full((B, CI, 1), float("nan"), device="cuda")
    C.sort_neuron_backward_input(col3(g), pos, gx2, 1, q, K)
    assert rel(host(gx2), gx_o) < 1e-5
    # interval bounds
    xl = np.clip(x - np.float32(0.03), 0, 1)
    xu = np.clip(x + np.float32(0.03), 0, 1)
    yl_o, yu_o = oracle.sort_bound_forward(xl, xu, w, q, K)
    yl = torch.empty(B, CO, 1, device="cuda")
    yu = torch.empty(B, CO, 1, device="cuda")
    C.bound_sort_neuron_forward(col3(xl), col3(xu), W, yl, yu, 1, q, K)
    assert rel(host(yl), yl_o) < VTOL and rel(host(yu), yu_o) < VTOL
    assert (host(yl) <= host(y) * (1 + 1e-6)).all() and (host(y) <= host(yu) * (1 + 1e-6)).all()


def test_ties_and_short_lists():
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(2)
    B, CI, CO, q, K = 40, 24, 30, 0.8, 10
    x = (rng.integers(0, 3, (B, CI)) / 2).astype(np.float32)
    w = (rng.integers(0, 3, (CO, CI)) / 2).astype(np.float32)      # many zeros and ties
    x[1] = 0.5
    w[2] = 0.5                                                     # all-zero differences
    y_o, pos_o = oracle.sort_forward(x, w, q, K)
    y = torch.empty(B, CO, 1, device="cuda")
    pos = torch.empty(K, B, CO, 1, device="cuda", dtype=torch.int32)
    C.sort_neuron_forward(col3(x), dev(w), y, pos, 1, q, K)
    assert rel(host(y), y_o) < VTOL and np.array_equal(pos.squeeze(-1).cpu().numpy(), pos_o)
    assert (pos.squeeze(-1).cpu().numpy()[:, 1, 2] == 0).all()


def test_autograd_function_and_model_eval():
    from sortnet_b200 import ops
    from sortnet_b200.layers import SortMLPModel
    x = torch.rand(40, 30, 1, device="cuda", requires_grad=True)
    w = torch.randn(20, 30, device="cuda", requires_grad=True)
    y = ops.sort_neuron(x, w, q=0.8)
    y.sum().backward()
    assert torch.isfinite(x.grad).all() and torch.isfinite(w.grad).all()
    with torch.no_grad():
        y_inf = ops.norm_dist(x, w, float("inf"))
    assert (y.detach() <= y_inf * (1 + 1e-6)).all()
    # evaluation of a masked model goes through the sort neuron and its bounds
    model = SortMLPModel(depth=4, width=64, input_dim=(1, 4, 4), num_classes=5, dropout=0.8).cuda().eval()
    xin = torch.rand(33, 1, 4, 4, device="cuda")
    t = torch.randint(0, 5, (33,), device="cuda")
    with torch.no_grad():
        logits, margin = model(xin, targets=t, eps=0.01, up=torch.ones(1, device="cuda"),
                               down=torch.zeros(1, device="cuda"))
        plain = model(xin)
    assert torch.allclose(logits, plain) and torch.isfinite(margin).all()
    # the certified margin is an upper bound of the clean margin
    clean = logits - torch.gather(logits, 1, t.view(-1, 1))
    assert (margin * (2 * 0.01) + 1e-5 >= clean.scatter(1, t.view(-1, 1), 0)).all()
