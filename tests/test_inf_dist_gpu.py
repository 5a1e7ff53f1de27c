"""GPU parity of the l-infinity kernels against the CPU oracle and the golden fixtures.
Bit-exact for y and pos; gradients to 1e-5 relative (fp32 atomics vs correctly rounded sums)."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import col3, dev, host, idx3, make_masks, rel

pytestmark = pytest.mark.gpu


def run_forward(x, w, ci=None, co=None):
    from sortnet_b200 import norm_dist_cuda as C
    X, W = col3(x), dev(w)
    CO = co.shape[-1] if co is not None else w.shape[0]
    y = torch.empty(x.shape[0], CO, 1, device="cuda")
    pos = torch.empty_like(y, dtype=torch.int32)
    C.inf_dist_forward(X, W, y, pos, 1, idx3(ci), idx3(co))
    return host(y), host(pos)


def run_backward(g, pos, CI, wshape, ci=None, co=None, weight=True):
    from sortnet_b200 import norm_dist_cuda as C
    G, P = col3(g), col3(pos, torch.int32)
    gx = torch.full((g.shape[0], CI, 1), float("nan"), device="cuda")
    if weight:
        gw = torch.full(wshape, float("nan"), device="cuda")
        C.inf_dist_backward_input_weight(G, P, gx, gw, 1, idx3(ci), idx3(co))
        return host(gx), gw.cpu().numpy()
    C.inf_dist_backward_input(G, P, gx, 1)
    return host(gx), None


@pytest.mark.parametrize("name", ["norm_dist_inf_a", "norm_dist_inf_b"])
def test_golden_unmasked(golden, name):
    g = golden(name)
    y, pos = run_forward(g["x"], g["w"])
    assert np.array_equal(y, g["y"])
    y_o, pos_o = oracle.inf_dist_forward(g["x"], g["w"])
    assert np.array_equal(pos, pos_o)
    gx, gw = run_backward(g["gy"], pos, g["x"].shape[1], g["w"].shape)
    assert rel(gx, g["gx"]) < 1e-5 and rel(gw, g["gw"]) < 1e-5


def test_golden_masked(golden):
    g = golden("dropout_inf")
    y, pos = run_forward(g["x"], g["w"], g["ci"], g["co"])
    assert np.array_equal(y, g["y"])
    _, pos_o = oracle.inf_dist_forward(g["x"], g["w"], g["ci"], g["co"])
    assert np.array_equal(pos, pos_o)
    gx, gw = run_backward(g["gy"], pos, g["x"].shape[1], g["w"].shape, g["ci"], g["co"])
    assert rel(gx, g["gx"]) < 1e-5 and rel(gw, g["gw"]) < 1e-5


SHAPES = [(1, 1, 1), (5, 3, 2), (32, 64, 64), (33, 65, 67), (70, 48, 40), (128, 784, 200),
          (100, 130, 257), (260, 100, 300), (64, 516, 129)]


@pytest.mark.parametrize("B,CI,CO", SHAPES)
def test_unmasked_vs_oracle(B, CI, CO):
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(B * 1000 + CI)
    x = rng.random((B, CI), dtype=np.float32)
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    y_o, pos_o = oracle.inf_dist_forward(x, w)
    y, pos = run_forward(x, w)
    assert np.array_equal(y, y_o) and np.array_equal(pos, pos_o)
    yn = torch.empty(B, CO, 1, device="cuda")
    C.inf_dist_forward_nograd(col3(x), dev(w), yn, 1)
    assert np.array_equal(host(yn), y_o)
    g = rng.standard_normal((B, CO)).astype(np.float32)
    gx_o, gw_o = oracle.inf_dist_backward(g, pos_o, CI, w.shape)
    gx, gw = run_backward(g, pos_o, CI, w.shape)
    assert rel(gx, gx_o) < 1e-5 and rel(gw, gw_o) < 1e-5
    gx2, _ = run_backward(g, pos_o, CI, w.shape, weight=False)
    assert rel(gx2, gx_o) < 1e-5


@pytest.mark.parametrize("B,CI,CO,keep", [(70, 48, 40, 0.8), (96, 300, 520, 0.9), (33, 70, 90, 0.5),
                                          (160, 1030, 260, 0.9), (32, 64, 64, 1.0)])
@pytest.mark.parametrize("which", ["both", "ci", "co"])
def test_masked_vs_oracle(B, CI, CO, keep, which):
    rng = np.random.default_rng(B + CI + CO)
    ci = make_masks(rng, B, CI, keep) if which in ("both", "ci") else None
    co = make_masks(rng, B, CO, keep) if which in ("both", "co") else None
    x = rng.random((B, ci.shape[1] if ci is not None else CI), dtype=np.float32)
    w = rng.standard_normal((CO, CI)).astype(np.float32)
    y_o, pos_o = oracle.inf_dist_forward(x, w, ci, co)
    y, pos = run_forward(x, w, ci, co)
    assert np.array_equal(y, y_o) and np.array_equal(pos, pos_o)
    g = rng.standard_normal(y_o.shape).astype(np.float32)
    gx_o, gw_o = oracle.inf_dist_backward(g, pos_o, x.shape[1], w.shape, ci, co)
    gx, gw = run_backward(g, pos_o, x.shape[1], w.shape, ci, co)
    assert rel(gx, gx_o) < 1e-5 and rel(gw, gw_o) < 1e-5


def run_forward_sorted(x, w, ci=None, co=None):
    from sortnet_b200 import norm_dist_cuda as C
    CO = co.shape[-1] if co is not None else w.shape[0]
    y = torch.full((x.shape[0], CO, 1), float("nan"), device="cuda")
    pos = torch.full_like(y, -7, dtype=torch.int32)
    C.inf_dist_forward_sorted(col3(x), dev(w), y, pos, idx3(ci), idx3(co))
    return host(y), host(pos)


# full-width form (W_CI a multiple of 4, >= 3/4 of the columns kept) and the cases that fall back
# to the general masked path (few columns kept, odd W_CI); ragged last sub-batch and tile edges
@pytest.mark.parametrize("B,CI,CO,keep", [(70, 48, 40, 0.8), (96, 300, 520, 0.9), (33, 72, 90, 0.5),
                                          (160, 1032, 260, 0.9), (32, 64, 64, 1.0), (100, 131, 70, 0.9),
                                          (512, 1280, 1100, 0.9)])
@pytest.mark.parametrize("which", ["both", "ci", "co"])
@pytest.mark.parametrize("ties", [False, True])
def test_sorted_lists_entry_vs_oracle(B, CI, CO, keep, which, ties):
    """snb_inf_dist_forward_sorted_ws: y and pos bit-identical to the oracle, also when many
    columns tie for the maximum (quantised operands), where the position must be the lowest one."""
    rng = np.random.default_rng(B + CI + CO + (7 if ties else 0))
    ci = make_masks(rng, B, CI, keep) if which in ("both", "ci") else None
    co = make_masks(rng, B, CO, keep) if which in ("both", "co") else None
    n_in = ci.shape[1] if ci is not None else CI
    if ties:
        x = (rng.integers(0, 4, (B, n_in)) / 4).astype(np.float32)
        w = (rng.integers(-4, 5, (CO, CI)) / 4).astype(np.float32)
    else:
        x = rng.random((B, n_in), dtype=np.float32)
        w = rng.standard_normal((CO, CI)).astype(np.float32)
    y_o, pos_o = oracle.inf_dist_forward(x, w, ci, co)
    y, pos = run_forward_sorted(x, w, ci, co)
    assert np.array_equal(y, y_o) and np.array_equal(pos, pos_o)


def test_sorted_lists_entry_all_equal_operands():
    """x == w in every kept column: nothing exceeds 1e-10, y = 1e-10 and pos = 0 (as the reference);
    the dropped columns' weights are huge and must not be seen."""
    rng = np.random.default_rng(3)
    B, CI, CO = 64, 128, 96
    ci = make_masks(rng, B, CI, 0.8)
    w = np.full((CO, CI), 1e6, np.float32)
    x = np.full((B, ci.shape[1]), 0.5, np.float32)
    for s in range(ci.shape[0]):
        w[:, ci[s]] = 0.5
    y_o, pos_o = oracle.inf_dist_forward(x, w, ci, None)
    y, pos = run_forward_sorted(x, w, ci, None)
    assert np.array_equal(y, y_o) and np.array_equal(pos, pos_o)
    assert np.all(y == np.float32(1e-10)) and np.all(pos == 0)


@pytest.mark.parametrize("B,CI,CO", [(128, 784, 5120), (512, 1024, 2100), (100, 130, 257)])
def test_workspace_and_plain_entry_points_agree(B, CI, CO):
    """Unmasked forward through the C ABI three ways: without scratch, with scratch (tiles split
    along the reduction axis), with a too-small scratch (falls back).  All bit-identical."""
    from sortnet_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(CO)
    x = (rng.integers(0, 8, (B, CI)) / 8).astype(np.float32)      # plenty of exact ties
    w = (rng.integers(-16, 17, (CO, CI)) / 8).astype(np.float32)
    y_o, pos_o = oracle.inf_dist_forward(x, w)
    X, W = col3(x), dev(w)
    st = torch.cuda.current_stream().cuda_stream
    need = lib.snb_inf_dist_forward_workspace_bytes(B, CO)
    assert need == 8 * B * CO
    for ws_bytes in (None, need, 64):
        y = torch.zeros(B, CO, 1, device="cuda")
        pos = torch.zeros(B, CO, 1, device="cuda", dtype=torch.int32)
        if ws_bytes is None:
            rc = lib.snb_inf_dist_forward(X.data_ptr(), W.data_ptr(), B, CO, CI, 1, 1, y.data_ptr(),
                                          pos.data_ptr(), None, None, CO, CI, st)
        else:
            ws = torch.full((max(ws_bytes // 8, 1),), -1, dtype=torch.int64, device="cuda")
            rc = lib.snb_inf_dist_forward_ws(X.data_ptr(), W.data_ptr(), B, CO, CI, 1, 1, y.data_ptr(),
                                             pos.data_ptr(), None, None, CO, CI, ws.data_ptr(), ws_bytes, st)
        assert rc == 0
        assert np.array_equal(host(y), y_o) and np.array_equal(host(pos), pos_o)


@pytest.mark.parametrize("B,CI,CO,keep", [(512, 1024, 2100, 0.9), (96, 300, 520, 0.8), (500, 640, 5000, 0.9)])
def test_masked_workspace_and_plain_entry_points_agree(B, CI, CO, keep):
    from sortnet_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(CO + 1)
    ci, co = make_masks(rng, B, CI, keep), make_masks(rng, B, CO, keep)
    x = (rng.integers(0, 8, (B, ci.shape[1])) / 8).astype(np.float32)
    w = (rng.integers(-16, 17, (CO, CI)) / 8).astype(np.float32)
    y_o, pos_o = oracle.inf_dist_forward(x, w, ci, co)
    X, W, CIt, COt = col3(x), dev(w), idx3(ci), idx3(co)
    st = torch.cuda.current_stream().cuda_stream
    n_in, n_out = ci.shape[1], co.shape[1]
    for use_ws in (False, True):
        y = torch.zeros(B, n_out, 1, device="cuda")
        pos = torch.zeros(B, n_out, 1, device="cuda", dtype=torch.int32)
        if use_ws:
            ws = torch.full((B * n_out,), -1, dtype=torch.int64, device="cuda")
            rc = lib.snb_inf_dist_forward_ws(X.data_ptr(), W.data_ptr(), B, n_out, n_in, 1, 1, y.data_ptr(),
                                             pos.data_ptr(), CIt.data_ptr(), COt.data_ptr(), CO, CI,
                                             ws.data_ptr(), ws.numel() * 8, st)
        else:
            rc = lib.snb_inf_dist_forward(X.data_ptr(), W.data_ptr(), B, n_out, n_in, 1, 1, y.data_ptr(),
                                          pos.data_ptr(), CIt.data_ptr(), COt.data_ptr(), CO, CI, st)
        assert rc == 0
        assert np.array_equal(host(y), y_o) and np.array_equal(host(pos), pos_o)


def test_ties_floor_and_sign():
    # quantised inputs force many exact ties: lowest index must win, sign from x - w
    rng = np.random.default_rng(7)
    x = (rng.integers(0, 4, (67, 150)) / 4).astype(np.float32)
    w = (rng.integers(-4, 5, (90, 150)) / 4).astype(np.float32)
    x[3] = 0.5
    w[5] = 0.5                      # all-equal row: stays at the 1e-10 floor with pos 0
    y_o, pos_o = oracle.inf_dist_forward(x, w)
    y, pos = run_forward(x, w)
    assert y[3, 5] == np.float32(1e-10) and pos[3, 5] == 0
    assert np.array_equal(y, y_o) and np.array_equal(pos, pos_o)


def test_tiny_differences_and_denormals():
    rng = np.random.default_rng(8)
    x = rng.random((40, 96), dtype=np.float32)
    w = np.tile(x[:1], (50, 1)) + (rng.standard_normal((50, 96)) * 1e-9).astype(np.float32)
    w[0] = x[0] + np.float32(1e-40)   # denormal difference
    y_o, pos_o = oracle.inf_dist_forward(x, w.astype(np.float32))
    y, pos = run_forward(x, w.astype(np.float32))
    assert np.array_equal(y, y_o) and np.array_equal(pos, pos_o)


def test_nan_inputs_are_skipped_like_the_reference():
    # the reference's `if (|t| > acc)` never takes a NaN; neither does max.f32
    x = np.array([[0.0, np.nan, 2.0, 0.5]], np.float32)
    w = np.array([[1.0, 0.0, 0.0, np.nan]], np.float32)
    y_o, pos_o = oracle.inf_dist_forward(x, w)
    y, pos = run_forward(x, w)
    assert np.array_equal(y, y_o) and np.array_equal(pos, pos_o)
    assert y[0, 0] == 2.0 and pos[0, 0] == 2


def test_run_to_run_identical():
    rng = np.random.default_rng(9)
    x = rng.random((128, 784), dtype=np.float32)
    w = rng.standard_normal((512, 784)).astype(np.float32)
    a = run_forward(x, w)
    b = run_forward(x, w)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_errors():
    from sortnet_b200 import norm_dist_cuda as C
    x = torch.rand(4, 8, 1, device="cuda")
    w = torch.rand(3, 8, device="cuda")
    y = torch.empty(4, 3, 1, device="cuda")
    pos = torch.empty(4, 3, 1, device="cuda", dtype=torch.int32)
    with pytest.raises(RuntimeError):
        C.inf_dist_forward(x.cpu(), w, y, pos, 1)
    with pytest.raises(RuntimeError):
        C.inf_dist_forward(x.transpose(0, 1), w, y, pos, 1)
    with pytest.raises(RuntimeError):
        C.inf_dist_forward(x, w, y, pos, 2)       # groups are not implemented
    with pytest.raises(RuntimeError):
        C.inf_dist_forward(x, w.double(), y, pos, 1)
