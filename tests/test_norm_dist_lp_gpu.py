"""GPU parity of the finite-p kernels against the exact-math (float64) oracle.

Tolerance: outputs are gated element by element, |y - y_o| <= 1e-5 * |y_o| (all distances are
positive and of order one, so every element can be held to the bar).  Gradients are sums of
signed terms accumulated with atomics in run-dependent order, so they are gated tensor-wise:
max-abs error over max-abs value <= 1e-5 at every p up to 1000.  The fp32 rounding of the ratio
|t| / y (6e-8 relative) would be amplified by the exponent p - 1 (6e-5 at p = 1000); the backward
kernel carries the exact remainders of the reciprocal and of the product (one fma each) through the
logarithm from p = 41 on.  Measured on B200 against the same oracle, on the same inputs
(128 x 784 x 300 and 64 x 2048 x 1024): this library 1.3e-7 / 1.2e-7 / 8e-8 at p = 100 / 316 / 1000
(4.8e-6 / 1.4e-5 / 4.3e-5 without the remainders), the reference's own kernels (compiled for
sm_100a) 7.2e-6 / 2.4e-5 / 6.8e-5."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import col3, dev, host, idx3, make_masks, rel

pytestmark = pytest.mark.gpu

TOL = 1e-5


def rel_each(y, y_o):
    """Largest element-wise relative error of positive outputs."""
    y = np.asarray(y, np.float64)
    y_o = np.asarray(y_o, np.float64)
    return float((np.abs(y - y_o) / np.abs(y_o)).max())


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
    assert rel_each(y, g["y"]) < 2e-5                  # the fixture itself is fp32 torch
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
    assert rel_each(y, y_o) < TOL
    g = rng.standard_normal((B, CO)).astype(np.float32)
    gx_o, gw_o = oracle.norm_dist_backward(g, x, w, y, p)
    gx, gw = run_bwd(g, x, w, y, p)
    tol = TOL
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
    assert rel_each(y, y_o) < TOL
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
        assert rel_each(y, y_o) < TOL


def test_large_p_approaches_inf():
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(11)
    x = rng.random((64, 512), dtype=np.float32)
    w = rng.standard_normal((96, 512)).astype(np.float32)
    y_inf = torch.empty(64, 96, 1, device="cuda")
    C.inf_dist_forward_nograd(col3(x), dev(w), y_inf, 1)
    y = run_fwd(x, w, 1000.0)
    assert (y >= host(y_inf) * (1 - 1e-6)).all() and rel(y, host(y_inf)) < 1e-2


@pytest.mark.parametrize("p", [8.0, 12.5, 100.0])
@pytest.mark.parametrize("B,CI,CO,keep", [(70, 150, 300, None), (96, 300, 520, 0.8), (512, 640, 1100, 0.9)])
def test_entry_point_without_scratch(p, B, CI, CO, keep):
    """snb_norm_dist_forward (no scratch: one thread block per output tile when p > 10) against the
    oracle and against snb_norm_dist_forward_ws (thread blocks share tiles, partial sums merge with
    atomics): both within the tolerance of the exact value, and within 2e-6 of each other."""
    from sortnet_b200 import _lib
    rng = np.random.default_rng(int(p) + B)
    ci = co = None
    if keep is not None:
        ci, co = make_masks(rng, B, CI, keep), make_masks(rng, B, CO, keep)
    ci_n = CI if ci is None else ci.shape[-1]
    co_n = CO if co is None else co.shape[-1]
    x = rng.random((B, ci_n), dtype=np.float32)
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    y_o = oracle.norm_dist_forward(x, w, p, ci, co)
    X, W, CI_, CO_ = col3(x), dev(w), idx3(ci), idx3(co)
    ptr = lambda t: None if t is None else t.data_ptr()
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    y_plain = torch.full((B, co_n, 1), float("nan"), device="cuda")
    rc = lib.snb_norm_dist_forward(X.data_ptr(), W.data_ptr(), B, co_n, ci_n, 1, 1, y_plain.data_ptr(), p,
                                   ptr(CI_), ptr(CO_), CO, CI, stream)
    assert rc == 0
    n_ws = lib.snb_norm_dist_forward_workspace_bytes(B, co_n, p)
    assert n_ws == (4 * B * co_n if p > 10 else 0)
    ws = torch.empty(max(n_ws, 16) // 4, device="cuda")
    y_ws = torch.full((B, co_n, 1), float("nan"), device="cuda")
    rc = lib.snb_norm_dist_forward_ws(X.data_ptr(), W.data_ptr(), B, co_n, ci_n, 1, 1, y_ws.data_ptr(), p,
                                      ptr(CI_), ptr(CO_), CO, CI, ws.data_ptr(), n_ws, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert rel_each(host(y_plain), y_o) < TOL and rel_each(host(y_ws), y_o) < TOL
    assert rel(host(y_plain), host(y_ws)) < 2e-6
    # a misaligned scratch pointer is refused, a short one falls back to the scratch-free kernel
    if p > 10:
        assert lib.snb_norm_dist_forward_ws(X.data_ptr(), W.data_ptr(), B, co_n, ci_n, 1, 1, y_ws.data_ptr(), p,
                                            ptr(CI_), ptr(CO_), CO, CI, ws.data_ptr() + 4, n_ws, stream) == 6
        y_short = torch.full((B, co_n, 1), float("nan"), device="cuda")
        assert lib.snb_norm_dist_forward_ws(X.data_ptr(), W.data_ptr(), B, co_n, ci_n, 1, 1, y_short.data_ptr(), p,
                                            ptr(CI_), ptr(CO_), CO, CI, ws.data_ptr(), n_ws - 4, stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(y_short, y_plain)


@pytest.mark.parametrize("p", [3.0, 8.0, 31.6])
@pytest.mark.parametrize("masked", [False, True], ids=["dense 64x5120x5120", "masked 64x4619x4596"])
def test_wide_layers_vs_oracle(p, masked):
    """Two sub-batches of a 5120-wide layer: more than 10 000 backward work units, so every thread
    block's range spans several units and both the plain-store and the atomic branch of the
    backward run; the forward runs shared tiles with atomically merged partial sums followed by
    the root kernel.  Every element of y and both gradients against the exact-math oracle."""
    B, CI, CO = 64, 5120, 5120
    rng = np.random.default_rng(int(p * 10) + masked)
    ci = co = None
    if masked:
        S = B // 32
        ci = np.stack([np.sort(rng.permutation(CI)[:4619]) for _ in range(S)]).astype(np.int32)
        co = np.stack([np.sort(rng.permutation(CO)[:4596]) for _ in range(S)]).astype(np.int32)
    x = rng.random((B, ci.shape[1] if masked else CI), dtype=np.float32)
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    y_o = oracle.norm_dist_forward(x, w, p, ci, co)
    y = run_fwd(x, w, p, ci, co)
    assert rel_each(y, y_o) < TOL
    g = rng.standard_normal(y.shape).astype(np.float32)
    gx_o, gw_o = oracle.norm_dist_backward(g, x, w, y, p, ci, co)
    gx, gw = run_bwd(g, x, w, y, p, ci, co)
    assert rel(gx, gx_o) < TOL and rel(gw, gw_o) < TOL
    gx2, _ = run_bwd(g, x, w, y, p, ci, co, weight=False)
    assert rel(gx2, gx_o) < TOL
