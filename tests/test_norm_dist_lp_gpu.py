"""GPU parity of the finite-p kernels against the exact-math (float64) oracle.

Tolerance: 1e-5 relative (max-abs error over max-abs value per tensor) for outputs and
gradients at p <= 32.  For larger p the fp32 rounding of |t| / y alone is amplified by p - 1
(6e-8 * (p - 1)), so the gradient tolerance is widened to 3e-7 * p there."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import col3, dev, host, idx3, make_masks, rel

pytestmark = pytest.mark.gpu

TOL = 1e-5


def run_fwd(x, w, p, ci=None, co=None):
    from sortnet_b200 import norm_dist_cuda as C
    CO = co.shape[-1] if co is not None else w.shape[0]
    y = torch.empty(x.shape[0], CO, 1, device="cuda")
    C.norm_dist_forward(col3(x), dev(w), y, 1, p, idx3(ci), idx3(co))
    return host(y)


def run_bwd(g, x, w, y, p, ci=None, co=None, weight=True):
    from sortnet_b200 import norm_dist_cuda as C
    gx = torch.full((x.shape[0], x.shape[1], 1), float("nan"), device="cuda")
    if weight:
        gw = torch.full(w.shape, float("nan"), device="cuda")
        C.norm_dist_backward_input_weight(col3(g), col3(x), dev(w), col3(y), gx, gw, 1, p, idx3(ci), idx3(co))
        return host(gx), gw.cpu().numpy()
    C.norm_dist_backward_input(col3(g), col3(x), dev(w), col3(y), gx, 1, p, idx3(ci), idx3(co))
    return host(gx), None


@pytest.mark.parametrize("name", ["norm_dist_p2", "norm_dist_p3", "norm_dist_p8", "norm_dist_p31",
                                  "dropout_p8", "dropout_p20"])
def test_golden(golden, name):
    g = golden(name)
    p = float(g["p"])
    ci, co = g.get("ci"), g.get("co")
    y = run_fwd(g["x"], g["w"], p, ci, co)
    assert rel(y, g["y"]) < TOL
    gx, gw = run_bwd(g["gy"], g["x"], g["w"], y, p, ci, co)
    assert rel(gx, g["gx"]) < 2e-5 and rel(gw, g["gw"]) < 2e-5   # the fixture itself is fp32 torch


@pytest.mark.parametrize("p", [1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0, 2.5, 9.3, 10.0, 10.5, 16.0, 31.6, 100.0, 1000.0])
@pytest.mark.parametrize("B,CI,CO", [(70, 48, 40), (33, 130, 257), (128, 784, 300)])
def test_unmasked_vs_oracle(p, B, CI, CO):
    rng = np.random.default_rng(int(p * 10) + B)
    x = rng.random((B, CI), dtype=np.float32)
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    y_o = oracle.norm_dist_forward(x, w, p)
    y = run_fwd(x, w, p)
    assert rel(y, y_o) < TOL
    g = rng.standard_normal((B, CO)).astype(np.float32)
    gx_o, gw_o = oracle.norm_dist_backward(g, x, w, y, p)
    gx, gw = run_bwd(g, x, w, y, p)
    tol = max(TOL, 3e-7 * p)
    assert rel(gx, gx_o) < tol and rel(gw, gw_o) < tol
    gx2, _ = run_bwd(g, x, w, y, p, weight=False)
    assert rel(gx2, gx_o) < tol


@pytest.mark.parametrize("p", [8.0, 3.0, 20.0, 31.6])
@pytest.mark.parametrize("which", ["both", "ci", "co"])
def test_masked_vs_oracle(p, which):
    B, CI, CO, keep = 96, 300, 520, 0.9
    rng = np.random.default_rng(int(p) + len(which))
    ci = make_masks(rng, B, CI, keep) if which in ("both", "ci") else None
    co = make_masks(rng, B, CO, keep) if which in ("both", "co") else None
    x = rng.random((B, ci.shape[1] if ci is not None else CI), dtype=np.float32)
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    y_o = oracle.norm_dist_forward(x, w, p, ci, co)
    y = run_fwd(x, w, p, ci, co)
    assert rel(y, y_o) < TOL
    g = rng.standard_normal(y.shape).astype(np.float32)
    gx_o, gw_o = oracle.norm_dist_backward(g, x, w, y, p, ci, co)
    gx, gw = run_bwd(g, x, w, y, p, ci, co)
    assert rel(gx, gx_o) < TOL and rel(gw, gw_o) < TOL


def test_degenerate_rows():
    # identical x and w row: p <= 10 gives FLT_MIN^(1/p), p > 10 gives 1e-10 (the seed term)
    x = np.full((3, 16), 0.25, np.float32)
    w = np.full((2, 16), 0.25, np.float32)
    for p in (2.0, 8.0, 20.0):
        y = run_fwd(x, w, p)
        y_o = oracle.norm_dist_forward(x, w, p)
        assert rel(y, y_o) < TOL


def test_large_p_approaches_inf():
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(11)
    x = rng.random((64, 512), dtype=np.float32)
    w = rng.standard_normal((96, 512)).astype(np.float32)
    y_inf = torch.empty(64, 96, 1, device="cuda")
    C.inf_dist_forward_nograd(col3(x), dev(w), y_inf, 1)
    y = run_fwd(x, w, 1000.0)
    assert (y >= host(y_inf) * (1 - 1e-6)).all() and rel(y, host(y_inf)) < 1e-2
