"""The layer shapes of the five benchmark configurations of this project at full size.

The oracle is run on a sample of batch rows (whole sub-batches, so the masks apply unchanged) and
compared bit for bit; every output is additionally checked through size-independent properties:
yL <= y <= yU, the argmax word reproduces y from x and W, degenerate boxes give the point value,
gradients conserve mass (sum of grad_x over a row = sum of +/- g), run-to-run identity."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import make_masks

pytestmark = pytest.mark.gpu

# (name, B, CI_full, CO_full, keep_in, keep_out, eps)
LAYERS = [
    ("cfg1 single layer", 128, 784, 5120, None, None, 0.3),
    ("cfg2 first layer", 512, 3072, 5120, None, 0.9, 8 / 255),
    ("cfg2 hidden layer", 512, 5120, 5120, 0.9, 0.9, 8 / 255),
    ("cfg2 head", 512, 5120, 10, 0.9, None, 8 / 255),
    ("cfg3 hidden layer, no masks", 512, 5120, 5120, None, None, 2 / 255),
    ("cfg4 first layer", 512, 12288, 5120, None, 0.9, 1 / 255),
    ("cfg4 head", 512, 5120, 200, 0.9, None, 1 / 255),
    ("cfg5 first layer per GPU", 128, 12288, 10240, None, 0.9, 1 / 255),
    ("cfg5 hidden layer per GPU", 128, 10240, 10240, 0.9, 0.9, 1 / 255),
    ("cfg5 head per GPU", 128, 10240, 1000, 0.9, None, 1 / 255),
]


@pytest.mark.parametrize("name,B,CI,CO,kin,kout,eps", LAYERS, ids=[l[0] for l in LAYERS])
def test_layer(name, B, CI, CO, kin, kout, eps):
    from sortnet_b200 import norm_dist_cuda as C
    rng = np.random.default_rng(abs(hash(name)) % (2 ** 31))
    ci = make_masks(rng, B, CI, kin) if kin else None
    co = make_masks(rng, B, CO, kout) if kout else None
    n_in = ci.shape[1] if ci is not None else CI
    n_out = co.shape[1] if co is not None else CO
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.rand(B, n_in, 1, device=dev, generator=g)
    w = torch.randn(CO, CI, device=dev, generator=g)
    CIt = None if ci is None else torch.from_numpy(ci).to(dev).unsqueeze(1).contiguous()
    COt = None if co is None else torch.from_numpy(co).to(dev).unsqueeze(1).contiguous()

    # ---- masked / plain l-inf forward with argmax words
    y = torch.empty(B, n_out, 1, device=dev)
    pos = torch.empty(B, n_out, 1, device=dev, dtype=torch.int32)
    C.inf_dist_forward(x, w, y, pos, 1, CIt, COt)
    y2, pos2 = torch.empty_like(y), torch.empty_like(pos)
    C.inf_dist_forward(x, w, y2, pos2, 1, CIt, COt)
    assert torch.equal(y, y2) and torch.equal(pos, pos2)                    # run-to-run identical
    # the word reproduces the value: |x[b, idx] - W[row, col]| == y, sign matches
    idx = (pos.squeeze(-1) & 0x7fffffff).long()
    rows_b = torch.arange(B, device=dev) // 32
    wrow = COt[rows_b, 0].long() if COt is not None else torch.arange(CO, device=dev).expand(B, -1)
    wcol = torch.gather(CIt[rows_b, 0].long(), 1, idx) if CIt is not None else idx
    t = torch.gather(x.squeeze(-1), 1, idx) - w[wrow, wcol]
    floor = y.squeeze(-1) == np.float32(1e-10)
    assert torch.equal(t.abs()[~floor], y.squeeze(-1)[~floor])
    assert torch.equal((pos.squeeze(-1) < 0)[~floor], (t < 0)[~floor])
    # oracle on the first and the last sub-batch
    for s in sorted({0, (B - 1) // 32}):
        sl = slice(32 * s, min(B, 32 * s + 32))
        y_o, pos_o = oracle.inf_dist_forward(x[sl, :, 0].cpu().numpy(), w.cpu().numpy(),
                                             None if ci is None else ci[s:s + 1], None if co is None else co[s:s + 1])
        assert np.array_equal(y[sl, :, 0].cpu().numpy(), y_o) and np.array_equal(pos[sl, :, 0].cpu().numpy(), pos_o)

    # ---- sparse backward: mass conservation per row, oracle on one sub-batch for grad_x
    gr = torch.randn(B, n_out, 1, device=dev, generator=g)
    gx, gw = torch.empty_like(x), torch.empty_like(w)
    C.inf_dist_backward_input_weight(gr, pos, gx, gw, 1, CIt, COt)
    signed = torch.where(pos < 0, -gr, gr)
    assert torch.allclose(gx.sum(dim=1), signed.sum(dim=1), rtol=1e-4, atol=1e-3)
    assert torch.allclose(gw.sum(), -signed.sum(), rtol=1e-3, atol=1e-2)
    gx_o, _ = oracle.inf_dist_backward(gr[:32, :, 0].cpu().numpy(), pos[:32, :, 0].cpu().numpy(), n_in, (1, 1),
                                       want_gw=False)
    err = np.abs(gx[:32, :, 0].cpu().numpy() - gx_o).max() / max(np.abs(gx_o).max(), 1e-30)
    assert err < 1e-5

    # ---- interval bounds on the dense layer (certification runs unmasked)
    xd = torch.rand(B, CI, 1, device=dev, generator=g)
    xl, xu = (xd - eps).clamp(0, 1), (xd + eps).clamp(0, 1)
    yl, yu = torch.empty(B, CO, 1, device=dev), torch.empty(B, CO, 1, device=dev)
    C.bound_inf_dist_forward_nograd(xl, xu, w, yl, yu, 1)
    yp = torch.empty(B, CO, 1, device=dev)
    C.inf_dist_forward_nograd(xd, w, yp, 1)
    assert bool((yl <= yp).all()) and bool((yp <= yu).all())
    yl0, yu0 = torch.empty_like(yl), torch.empty_like(yu)
    C.bound_inf_dist_forward_nograd(xd, xd, w, yl0, yu0, 1)
    assert torch.equal(yl0, yp) and torch.equal(yu0, yp)                    # degenerate box = point value
    rows = [0, B - 1]
    yl_o, yu_o, _, _ = oracle.bound_inf_dist_forward(xl[rows, :, 0].cpu().numpy(), xu[rows, :, 0].cpu().numpy(),
                                                    w.cpu().numpy(), want_pos=False)
    assert np.array_equal(yl[rows, :, 0].cpu().numpy(), yl_o) and np.array_equal(yu[rows, :, 0].cpu().numpy(), yu_o)
    from sortnet_b200 import _lib
    assert _lib.load().snb_device_wait_failed() == 0


def test_non_default_stream_and_second_stream_concurrency():
    """Work is enqueued on PyTorch's current stream; two streams with their own buffers do not
    interfere (no hidden global scratch in the ordinary entry points)."""
    from sortnet_b200 import norm_dist_cuda as C
    dev = torch.device("cuda")
    x = torch.rand(256, 1024, 1, device=dev)
    w = torch.randn(2048, 1024, device=dev)
    ref_y = torch.empty(256, 2048, 1, device=dev)
    ref_p = torch.empty(256, 2048, 1, device=dev, dtype=torch.int32)
    C.inf_dist_forward(x, w, ref_y, ref_p, 1)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for st in (s1, s2):
        with torch.cuda.stream(st):
            y = torch.empty_like(ref_y)
            p = torch.empty_like(ref_p)
            for _ in range(3):
                C.inf_dist_forward(x, w, y, p, 1)
            outs.append((y, p))
    torch.cuda.synchronize()
    for y, p in outs:
        assert torch.equal(y, ref_y) and torch.equal(p, ref_p)
