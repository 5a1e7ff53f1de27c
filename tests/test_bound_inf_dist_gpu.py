"""GPU parity of the interval-bound kernels: bounds and words bit-exact, gradients to 1e-5."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import col3, dev, host, rel

pytestmark = pytest.mark.gpu


def run_nograd(xl, xu, w):
    from sortnet_b200 import norm_dist_cuda as C
    yl = torch.empty(xl.shape[0], w.shape[0], 1, device="cuda")
    yu = torch.empty_like(yl)
    C.bound_inf_dist_forward_nograd(col3(xl), col3(xu), dev(w), yl, yu, 1)
    return host(yl), host(yu)


def run_pos(xl, xu, w):
    from sortnet_b200 import norm_dist_cuda as C
    yl = torch.empty(xl.shape[0], w.shape[0], 1, device="cuda")
    yu = torch.empty_like(yl)
    pl = torch.empty_like(yl, dtype=torch.int32)
    pu = torch.empty_like(pl)
    C.bound_inf_dist_forward(col3(xl), col3(xu), dev(w), yl, yu, pl, pu, 1)
    return host(yl), host(yu), host(pl), host(pu)


def run_bwd(gl, gu, pl, pu, CI, weight=True):
    from sortnet_b200 import norm_dist_cuda as C
    B, CO = gl.shape
    gxl = torch.full((B, CI, 1), float("nan"), device="cuda")
    gxu = torch.full((B, CI, 1), float("nan"), device="cuda")
    args = (col3(gl), col3(gu), col3(pl, torch.int32), col3(pu, torch.int32), gxl, gxu)
    if weight:
        gw = torch.full((CO, CI), float("nan"), device="cuda")
        C.bound_inf_dist_backward_input_weight(*args, gw, 1)
        return host(gxl), host(gxu), gw.cpu().numpy()
    C.bound_inf_dist_backward_input(*args, 1)
    return host(gxl), host(gxu), None


@pytest.mark.parametrize("name", ["bound_a", "bound_b"])
def test_golden(golden, name):
    g = golden(name)
    yl, yu = run_nograd(g["xl"], g["xu"], g["w"])
    assert np.array_equal(yl, g["yl"]) and np.array_equal(yu, g["yu"])
    yl, yu, pl, pu = run_pos(g["xl"], g["xu"], g["w"])
    assert np.array_equal(yl, g["yl"]) and np.array_equal(yu, g["yu"])
    gxl, gxu, gw = run_bwd(g["gl"], g["gu"], pl, pu, g["xl"].shape[1])
    assert rel(gxl, g["gxl"]) < 1e-5 and rel(gxu, g["gxu"]) < 1e-5 and rel(gw, g["gw"]) < 1e-5


@pytest.mark.parametrize("B,CI,CO,eps", [(1, 1, 1, 0.1), (5, 3, 2, 0.3), (33, 65, 67, 0.03), (128, 784, 200, 0.3),
                                         (100, 130, 257, 0.01), (260, 100, 300, 0.5), (64, 516, 129, 8 / 255),
                                         (512, 640, 1100, 2 / 255)])
def test_vs_oracle(B, CI, CO, eps):
    rng = np.random.default_rng(B + CI * 7 + CO)
    x = rng.random((B, CI), dtype=np.float32)
    xl = np.clip(x - np.float32(eps), 0, 1).astype(np.float32)
    xu = np.clip(x + np.float32(eps), 0, 1).astype(np.float32)
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    yl_o, yu_o, pl_o, pu_o = oracle.bound_inf_dist_forward(xl, xu, w)
    yl, yu = run_nograd(xl, xu, w)
    assert np.array_equal(yl, yl_o) and np.array_equal(yu, yu_o)
    yl, yu, pl, pu = run_pos(xl, xu, w)
    assert np.array_equal(yl, yl_o) and np.array_equal(yu, yu_o)
    assert np.array_equal(pl, pl_o) and np.array_equal(pu, pu_o)
    gl = rng.standard_normal((B, CO)).astype(np.float32)
    gu = rng.standard_normal((B, CO)).astype(np.float32)
    o = oracle.bound_inf_dist_backward(gl, gu, pl_o, pu_o, CI)
    r = run_bwd(gl, gu, pl_o, pu_o, CI)
    assert all(rel(a, b) < 1e-5 for a, b in zip(r, o))
    r2 = run_bwd(gl, gu, pl_o, pu_o, CI, weight=False)
    assert rel(r2[0], o[0]) < 1e-5 and rel(r2[1], o[1]) < 1e-5


def test_inverted_intervals_floors_and_ties():
    rng = np.random.default_rng(3)
    B, CI, CO = 70, 100, 90
    xl = (rng.integers(0, 5, (B, CI)) / 4).astype(np.float32)
    xu = (rng.integers(0, 5, (B, CI)) / 4).astype(np.float32)      # about half are inverted
    w = (rng.integers(-4, 5, (CO, CI)) / 4).astype(np.float32)
    xl[2] = xu[2] = 0.5
    w[4] = 0.5                                                     # degenerate: floors, posL = -1
    o = oracle.bound_inf_dist_forward(xl, xu, w)
    yl, yu = run_nograd(xl, xu, w)
    assert np.array_equal(yl, o[0]) and np.array_equal(yu, o[1])
    r = run_pos(xl, xu, w)
    assert all(np.array_equal(a, b) for a, b in zip(r, o))
    assert r[2][2, 4] == -1 and r[3][2, 4] == 0 and r[0][2, 4] == np.float32(1e-10)
    gl = rng.standard_normal((B, CO)).astype(np.float32)
    gu = rng.standard_normal((B, CO)).astype(np.float32)
    ob = oracle.bound_inf_dist_backward(gl, gu, o[2], o[3], CI)
    rb = run_bwd(gl, gu, o[2], o[3], CI)
    assert all(rel(a, b) < 1e-5 for a, b in zip(rb, ob))


def test_bounds_enclose_the_point_value():
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(5)
    B, CI, CO = 256, 3072, 512
    x = rng.random((B, CI), dtype=np.float32)
    xl = np.clip(x - np.float32(8 / 255), 0, 1)
    xu = np.clip(x + np.float32(8 / 255), 0, 1)
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    yl, yu = run_nograd(xl, xu, w)
    y = torch.empty(B, CO, 1, device="cuda")
    C.inf_dist_forward_nograd(col3(x), dev(w), y, 1)
    y = host(y)
    assert (yl <= y).all() and (y <= yu).all()
    # degenerate box reproduces the point value exactly
    yl0, yu0 = run_nograd(x, x, w)
    assert np.array_equal(yu0, y) and np.array_equal(yl0, y)


@pytest.mark.parametrize("B,CI,CO", [(512, 1024, 2600), (500, 1028, 2500), (130, 2048, 9600)])
def test_large_aligned_shapes_take_the_tma_path(B, CI, CO):
    """Shapes big enough for the TMA-staged kernel (ragged rows, CI not a multiple of the k-tile,
    some inverted intervals); results must still be bit-identical and no device wait may time out."""
    from sortnet_b200 import _lib
    rng = np.random.default_rng(B + CO)
    x = rng.random((B, CI), dtype=np.float32)
    xl = np.clip(x - np.float32(0.05), 0, 1).astype(np.float32)
    xu = np.clip(x + np.float32(0.05), 0, 1).astype(np.float32)
    flip = rng.random((B, CI)) < 0.01
    xl[flip], xu[flip] = xu[flip] + np.float32(0.1), xl[flip]
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    yl_o, yu_o, _, _ = oracle.bound_inf_dist_forward(xl, xu, w, want_pos=False)
    yl, yu = run_nograd(xl, xu, w)
    assert np.array_equal(yl, yl_o) and np.array_equal(yu, yu_o)
    assert _lib.load().snb_device_wait_failed() == 0
