"""The grouped / spatial oracle wrappers (oracle/general.py) against fixtures made by the reference's
PyTorch branches with groups > 1 and HW > 1."""
import numpy as np
import pytest

from oracle import general as og


def rel(a, b):
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)


@pytest.mark.parametrize("name", ["general_inf", "general_inf_hw"])
def test_inf(golden, name):
    g = golden(name)
    G = int(g["G"])
    y, pos = og.inf_dist_forward_g(g["x"], g["w"], G)
    assert np.array_equal(y, g["y"])                      # bit-exact
    gx, gw = og.inf_dist_backward_g(g["gy"], pos, g["x"].shape[1], g["w"].shape, G)
    assert rel(gx, g["gx"]) < 1e-6 and rel(gw, g["gw"]) < 1e-6


@pytest.mark.parametrize("name", ["general_p8", "general_p20_groups"])
def test_lp(golden, name):
    g = golden(name)
    G, p = int(g["G"]), float(g["p"])
    y = og.norm_dist_forward_g(g["x"], g["w"], p, G)
    assert rel(y, g["y"]) < 2e-6
    gx, gw = og.norm_dist_backward_g(g["gy"], g["x"], g["w"], y.astype(np.float32), p, G)
    assert rel(gx, g["gx"]) < 2e-5 and rel(gw, g["gw"]) < 2e-5


def test_masked_inf(golden):
    g = golden("general_dropout_inf")
    G = int(g["G"])
    y, pos = og.inf_dist_forward_g(g["x"], g["w"], G, g["ci"], g["co"])
    assert np.array_equal(y, g["y"])
    gx, gw = og.inf_dist_backward_g(g["gy"], pos, g["x"].shape[1], g["w"].shape, G, g["ci"], g["co"])
    assert rel(gx, g["gx"]) < 1e-6 and rel(gw, g["gw"]) < 1e-6


def test_masked_lp(golden):
    g = golden("general_dropout_p8")
    G, p = int(g["G"]), float(g["p"])
    y = og.norm_dist_forward_g(g["x"], g["w"], p, G, g["ci"], g["co"])
    assert rel(y, g["y"]) < 2e-6
    gx, gw = og.norm_dist_backward_g(g["gy"], g["x"], g["w"], y.astype(np.float32), p, G, g["ci"], g["co"])
    assert rel(gx, g["gx"]) < 2e-5 and rel(gw, g["gw"]) < 2e-5


def test_bound(golden):
    g = golden("general_bound")
    G = int(g["G"])
    yl, yu, pl, pu = og.bound_inf_dist_forward_g(g["xl"], g["xu"], g["w"], G)
    assert np.array_equal(yl, g["yl"]) and np.array_equal(yu, g["yu"])
    gxl, gxu, gw = og.bound_inf_dist_backward_g(g["gl"], g["gu"], pl, pu, g["xl"].shape[1], G)
    assert rel(gxl, g["gxl"]) < 1e-6 and rel(gxu, g["gxu"]) < 1e-6 and rel(gw, g["gw"]) < 1e-6


def test_sort(golden):
    g = golden("general_sort")
    G, q, K = int(g["G"]), float(g["q"]), int(g["K"])
    y, pos = og.sort_forward_g(g["x"], g["w"], q, K, G)
    assert rel(y, g["y"]) < 2e-6
    gx, gw = og.sort_backward_g(g["gy"], pos, g["x"].shape[1], q, K, G)
    assert rel(gx, g["gx"]) < 1e-5 and rel(gw, g["gw"]) < 1e-5
    yl, yu = og.sort_bound_forward_g(g["x"], g["x"], g["w"], q, K, G)   # degenerate interval
    assert rel(yl, g["y"]) < 2e-6 and rel(yu, g["y"]) < 2e-6
