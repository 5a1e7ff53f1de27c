"""GPU parity of the mean-shift kernels against the numpy restatement and the fixtures."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import col3, dev, host, idx3, make_masks, rel

pytestmark = pytest.mark.gpu


def run_center(x, index, C_full, running=None, momentum=0.1):
    from sortnet_b200 import norm_dist_cuda as C
    X = col3(x)
    mean = torch.full((C_full,), float("nan"), device="cuda")
    rm = None if running is None else dev(running)
    C.mean_shift_stats(X, idx3(index), mean, rm, momentum)
    y = torch.empty_like(X)
    C.mean_shift_apply(X, mean, idx3(index), y)
    return host(y), mean.cpu().numpy(), None if rm is None else rm.cpu().numpy()


@pytest.mark.parametrize("name", ["mean_shift_masked", "mean_shift_plain"])
def test_golden(golden, name):
    g = golden(name)
    index = g.get("index")
    C_full = g["running_mean0"].shape[0]
    y, mean, rm = run_center(g["x"], index, C_full, g["running_mean0"])
    assert rel(y, g["y"]) < 1e-5 and rel(rm, g["running_mean1"]) < 1e-5
    gx, _, _ = run_center(g["gy"], index, C_full)          # backward = the same centring of grad
    assert rel(gx, g["gx"]) < 1e-5


@pytest.mark.parametrize("B,C_full,keep", [(70, 40, 0.8), (512, 5120, 0.9), (33, 300, 0.5), (64, 128, None),
                                           (100, 77, None)])
def test_vs_oracle(B, C_full, keep):
    rng = np.random.default_rng(B + C_full)
    index = make_masks(rng, B, C_full, keep) if keep is not None else None
    C = index.shape[1] if index is not None else C_full
    x = rng.standard_normal((B, C)).astype(np.float32)
    y_o, mean_o = oracle.mean_shift_train(x, index, C_full)
    y, mean, _ = run_center(x, index, C_full)
    assert rel(y, y_o) < 1e-5 and rel(mean, mean_o) < 1e-5
    a = run_center(x, index, C_full)
    assert np.array_equal(a[0], y) and np.array_equal(a[1], mean)   # deterministic


def test_in_place_apply_and_eval():
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(1)
    x = rng.standard_normal((45, 24)).astype(np.float32)
    rm = rng.standard_normal(24).astype(np.float32)
    X = col3(x)
    C.mean_shift_apply(X, dev(rm), None, X)
    assert rel(host(X), x - rm[None]) < 1e-6
