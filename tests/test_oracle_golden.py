"""The CPU oracle against the fixtures produced by the reference's own PyTorch branches."""
import numpy as np
import pytest

import oracle

SIGN = np.int32(-2**31)


def rel(a, b):
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)


@pytest.mark.parametrize("name", ["norm_dist_inf_a", "norm_dist_inf_b"])
def test_inf_forward_backward(golden, name):
    g = golden(name)
    y, pos = oracle.inf_dist_forward(g["x"], g["w"])
    assert np.array_equal(y, g["y"])                     # bit-exact
    idx = pos & 0x7fffffff
    t = g["x"][np.arange(len(idx))[:, None], idx] - g["w"][np.arange(g["w"].shape[0])[None], idx]
    assert np.array_equal(np.abs(t), y)
    assert np.array_equal(pos < 0, t < 0)
    gx, gw = oracle.inf_dist_backward(g["gy"], pos, g["x"].shape[1], g["w"].shape)
    assert rel(gx, g["gx"]) < 1e-6 and rel(gw, g["gw"]) < 1e-6


def test_inf_forward_nograd_same_values(golden):
    g = golden("norm_dist_inf_a")
    y, pos = oracle.inf_dist_forward(g["x"], g["w"], want_pos=False)
    assert pos is None and np.array_equal(y, g["y"])


@pytest.mark.parametrize("name", ["norm_dist_p2", "norm_dist_p3", "norm_dist_p8", "norm_dist_p31"])
def test_lp_forward_backward(golden, name):
    g = golden(name)
    p = float(g["p"])
    y = oracle.norm_dist_forward(g["x"], g["w"], p)
    assert rel(y, g["y"]) < 2e-6                          # fixture is fp32 torch
    gx, gw = oracle.norm_dist_backward(g["gy"], g["x"], g["w"], y.astype(np.float32), p)
    assert rel(gx, g["gx"]) < 2e-5 and rel(gw, g["gw"]) < 2e-5


def test_masked_inf(golden):
    g = golden("dropout_inf")
    y, pos = oracle.inf_dist_forward(g["x"], g["w"], g["ci"], g["co"])
    assert np.array_equal(y, g["y"])
    gx, gw = oracle.inf_dist_backward(g["gy"], pos, g["x"].shape[1], g["w"].shape, g["ci"], g["co"])
    assert rel(gx, g["gx"]) < 1e-6 and rel(gw, g["gw"]) < 1e-6


@pytest.mark.parametrize("name", ["dropout_p8", "dropout_p20"])
def test_masked_lp(golden, name):
    g = golden(name)
    p = float(g["p"])
    y = oracle.norm_dist_forward(g["x"], g["w"], p, g["ci"], g["co"])
    assert rel(y, g["y"]) < 2e-6
    gx, gw = oracle.norm_dist_backward(g["gy"], g["x"], g["w"], y.astype(np.float32), p,
                                       g["ci"], g["co"])
    assert rel(gx, g["gx"]) < 2e-5 and rel(gw, g["gw"]) < 2e-5


@pytest.mark.parametrize("name", ["bound_a", "bound_b"])
def test_bound(golden, name):
    g = golden(name)
    yl, yu, pl, pu = oracle.bound_inf_dist_forward(g["xl"], g["xu"], g["w"])
    assert np.array_equal(yl, g["yl"]) and np.array_equal(yu, g["yu"])
    yl2, yu2, _, _ = oracle.bound_inf_dist_forward(g["xl"], g["xu"], g["w"], want_pos=False)
    assert np.array_equal(yl2, yl) and np.array_equal(yu2, yu)
    gxl, gxu, gw = oracle.bound_inf_dist_backward(g["gl"], g["gu"], pl, pu, g["xl"].shape[1])
    assert rel(gxl, g["gxl"]) < 1e-6 and rel(gxu, g["gxu"]) < 1e-6 and rel(gw, g["gw"]) < 1e-6


def test_bound_edge_rules():
    # xL > xU is repaired to the midpoint; a row that never leaves the EPS floor keeps
    # posL = 0xffffffff / posU = 0 (bound_inf_dist_cuda.cu:63,148-151)
    xl = np.array([[0.75, 0.5]], np.float32)
    xu = np.array([[0.25, 0.5]], np.float32)
    w = np.array([[0.5, 0.5]], np.float32)
    yl, yu, pl, pu = oracle.bound_inf_dist_forward(xl, xu, w)
    assert yl[0, 0] == np.float32(1e-10) and yu[0, 0] == np.float32(1e-10)
    assert pl[0, 0] == -1 and pu[0, 0] == 0


def test_inf_edge_rules():
    # all-equal row stays at the 1e-10 floor with pos 0 (+); first index wins ties
    x = np.array([[0.5, 0.5, 0.5], [0.0, 2.0, -1.0]], np.float32)
    w = np.array([[0.5, 0.5, 0.5], [1.0, 1.0, 0.0]], np.float32)
    y, pos = oracle.inf_dist_forward(x, w)
    assert y[0, 0] == np.float32(1e-10) and pos[0, 0] == 0
    assert y[1, 1] == 1.0 and pos[1, 1] == (0 | SIGN)     # |0-1| first, negative
    assert y[1, 0] == 1.5 and pos[1, 0] == 1              # 2-0.5 = 1.5 at c=1 (c=2 ties later)


@pytest.mark.parametrize("name", ["mean_shift_masked", "mean_shift_plain"])
def test_mean_shift(golden, name):
    g = golden(name)
    index = g.get("index")
    C = g["running_mean0"].shape[0]
    y, mean = oracle.mean_shift_train(g["x"], index, C)
    assert rel(y, g["y"]) < 1e-6
    rm = 0.9 * g["running_mean0"] + 0.1 * mean
    assert rel(rm, g["running_mean1"]) < 1e-6
    gx = oracle.mean_shift_train_backward(g["gy"], index, C)
    assert rel(gx, g["gx"]) < 1e-6
