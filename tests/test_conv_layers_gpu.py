"""NormDistConv (grouped, spatial) and the mean shift over [B, C, HW] on the GPU against fixtures
recorded from the reference's own NormDistConv / MeanShiftDropout layers (PyTorch branches)."""
import numpy as np
import pytest
import torch

from gpu_util import dev, rel

pytestmark = pytest.mark.gpu


def build_stack(g):
    from sortnet_b200.layers import NormDistConv
    p, q, G = float(g["p"]), float(g["q"]), int(g["G"])
    drop = None if q == 1.0 else q
    layers = [NormDistConv(4, 12, 3, stride=1, groups=G, bias=False, mean_shift=True, p=p),
              NormDistConv(12, 12, 1, groups=G, bias=True, mean_shift=True, dropout=drop, p=p),
              NormDistConv(12, 8, 1, groups=G, bias=True, mean_shift=False, dropout=drop, p=p)]
    for i, l in enumerate(layers):
        l.load_state_dict({k: torch.from_numpy(g["state0.%d.%s" % (i, k)]) for k in l.state_dict()})
        l.cuda()
    return layers


@pytest.mark.parametrize("name", ["conv_stack_masked_inf", "conv_stack_masked_p8", "conv_stack_plain_inf"])
def test_conv_stack_training_step(golden, name):
    g = golden(name)
    layers = build_stack(g)
    masked = "mask0" in g
    masks = [dev(g["mask0"], torch.int32), dev(g["mask1"], torch.int32)] if masked else [None, None]
    x = dev(g["x"]).requires_grad_()
    for l in layers:
        l.train()
    z = layers[0](x, mask_out=masks[0])
    z = layers[1](z[0], mask_in=masks[0], mask_out=masks[1])
    z = layers[2](z[0], mask_in=masks[1])
    y = z[0]
    tol = 1e-5
    assert rel(y.detach().cpu().numpy(), g["y"]) < tol
    y.backward(dev(g["gy"]))
    assert rel(x.grad.cpu().numpy(), g["gx"]) < tol
    for i, l in enumerate(layers):
        for k, prm in l.named_parameters():
            assert rel(prm.grad.cpu().numpy(), g["grad.%d.%s" % (i, k)]) < tol, (i, k)
        if l.mean_shift is not None:
            assert rel(l.mean_shift.running_mean.cpu().numpy(), g["state1.%d.mean_shift.running_mean" % i]) < tol


@pytest.mark.parametrize("name", ["conv_stack_masked_inf", "conv_stack_plain_inf"])
def test_conv_stack_evaluation(golden, name):
    g = golden(name)
    layers = build_stack(g)
    for i, l in enumerate(layers):
        if l.mean_shift is not None:
            l.mean_shift.running_mean.copy_(dev(g["state1.%d.mean_shift.running_mean" % i]))
        l.eval()
    x = dev(g["x"])
    with torch.no_grad():
        if "eval_lower" in g:
            z = (x, (x - 0.05).clamp(0, 1), (x + 0.05).clamp(0, 1))
            for l in layers:
                z = l(*z)
            assert rel(z[0].cpu().numpy(), g["eval_y"]) < 1e-6
            assert rel(z[1].cpu().numpy(), g["eval_lower"]) < 1e-6
            assert rel(z[2].cpu().numpy(), g["eval_upper"]) < 1e-6
            assert bool((z[1] <= z[0]).all()) and bool((z[0] <= z[2]).all())
        else:
            z = (x, None, None)
            for l in layers:
                z = l(*z, sort_eval=True)
            assert rel(z[0].cpu().numpy(), g["eval_y"]) < 1e-5
            # interval bounds of the sort neurons enclose the point value
            lo, up = (x - 0.02).clamp(0, 1), (x + 0.02).clamp(0, 1)
            zb = (x, lo, up)
            for l in layers:
                zb = l(*zb, sort_eval=True)
            assert bool((zb[1] <= zb[0] + 1e-5).all()) and bool((zb[0] <= zb[2] + 1e-5).all())


def test_mean_shift_plane_matches_per_channel_mean():
    from sortnet_b200.layers import MeanShiftDropout
    torch.manual_seed(0)
    m = MeanShiftDropout(6, affine=True).cuda()
    with torch.no_grad():
        m.bias.normal_()
    x = torch.randn(45, 6, 7, device="cuda", requires_grad=True)
    m.train()
    y, _, _ = m(x)
    mean = x.detach().mean(dim=(0, 2))
    want = x.detach() - mean.view(1, -1, 1) + m.bias.detach().view(1, -1, 1)
    assert rel(y.detach().cpu().numpy(), want.cpu().numpy()) < 1e-5
    assert rel(m.running_mean.cpu().numpy(), (0.1 * mean).cpu().numpy()) < 1e-5
    gy = torch.randn_like(y)
    y.backward(gy)
    assert rel(x.grad.cpu().numpy(), (gy - gy.mean(dim=(0, 2), keepdim=True)).cpu().numpy()) < 1e-5
