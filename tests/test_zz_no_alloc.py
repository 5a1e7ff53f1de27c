"""The allocation-free forward entry point (snb_inf_dist_forward_noalloc), called through the C ABI.

A host that binds the library directly may be unable to allocate device memory per call (no
tensor library to lend it scratch; cudaMalloc synchronises the device and can fail under a memory
budget).  For such callers the library carries its own fixed scratch array.  This file checks that
the entry point returns exactly what the ordinary entry point returns (y and argmax words are
compared bit for bit, the bar all l-infinity tests use), on two calls in a row with different
inputs, since the array keeps whatever the previous call left in it; the first shape is also
compared with the CPU oracle directly.  It is named so that pytest
collects it last: if it fails, a run that stops at the first failure has already run every other
test.  It does not depend on any other test having run.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _forward_pair(lib, x, w):
    """Runs the ordinary and the allocation-free entry point on the same device tensors."""
    B, CI = x.shape[0], x.shape[1]
    CO = w.shape[0]
    st = torch.cuda.current_stream().cuda_stream
    out = []
    for entry in ("plain", "noalloc"):
        y = torch.full((B, CO, 1), float("nan"), device="cuda")
        pos = torch.full((B, CO, 1), -7, device="cuda", dtype=torch.int32)
        if entry == "plain":
            rc = lib.snb_inf_dist_forward(x.data_ptr(), w.data_ptr(), B, CO, CI, 1, 1, y.data_ptr(),
                                          pos.data_ptr(), None, None, CO, CI, st)
        else:
            rc = lib.snb_inf_dist_forward_noalloc(x.data_ptr(), w.data_ptr(), B, CO, CI, 1, 1,
                                                  y.data_ptr(), pos.data_ptr(), st)
        assert rc == 0, lib.snb_status_string(rc)
        out.append((y, pos))
    torch.cuda.synchronize()
    return out


def test_noalloc_matches_the_ordinary_entry_point_twice_in_a_row():
    from sortnet_b200 import _lib
    lib = _lib.load()
    assert lib.snb_inf_dist_forward_noalloc_max_outputs() == 1 << 20
    gen = torch.Generator(device="cuda").manual_seed(1234)
    # first call: a shape whose tiles are split along the reduction axis (merge keys are used),
    # quantised values so that many maxima tie; second call: different data and a smaller shape that
    # is split as well, so stale keys of the first call lie inside and beyond the region it uses;
    # third call: a shape small enough to run without merging
    shapes = [(128, 784, 5120), (64, 2048, 2048), (96, 300, 1000)]
    for k, (B, CI, CO) in enumerate(shapes):
        x = (torch.randint(0, 8, (B, CI, 1), device="cuda", generator=gen) / 8).float().contiguous()
        w = (torch.randint(-16, 17, (CO, CI), device="cuda", generator=gen) / 8).float().contiguous()
        (y0, p0), (y1, p1) = _forward_pair(lib, x, w)
        if k == 0:
            import oracle
            y_o, pos_o = oracle.inf_dist_forward(x[:, :, 0].cpu().numpy(), w.cpu().numpy())
            assert np.array_equal(y1[:, :, 0].cpu().numpy(), y_o), "values differ from the oracle"
            assert np.array_equal(p1[:, :, 0].cpu().numpy(), pos_o), "argmax words differ from the oracle"
        assert torch.equal(y0, y1), "values differ from the ordinary entry point"
        assert torch.equal(p0, p1), "argmax words differ from the ordinary entry point"
        assert not torch.isnan(y1).any() and int(p1.min()) != -7
    # and once more with continuous data on the first shape
    x = torch.rand(128, 784, 1, device="cuda", generator=gen)
    w = torch.randn(5120, 784, device="cuda", generator=gen)
    (y0, p0), (y1, p1) = _forward_pair(lib, x, w)
    assert torch.equal(y0, y1) and torch.equal(p0, p1)


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from sortnet_b200 import _lib
    lib = _lib.load()
    B, CI, CO = 512, 64, 5120           # 2.6 M outputs > 1 Mi
    x = torch.rand(B, CI, 1, device="cuda")
    w = torch.randn(CO, CI, device="cuda")
    y = torch.empty(B, CO, 1, device="cuda")
    pos = torch.empty(B, CO, 1, device="cuda", dtype=torch.int32)
    rc = lib.snb_inf_dist_forward_noalloc(x.data_ptr(), w.data_ptr(), B, CO, CI, 1, 1, y.data_ptr(),
                                          pos.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 7
    assert b"scratch" in lib.snb_status_string(rc)
    with pytest.raises(_lib.SortnetB200Error, match="scratch"):
        _lib.check(rc, "inf_dist_forward_noalloc")
