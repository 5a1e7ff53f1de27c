"""The one-call-per-layer entry points (snb_layer_forward / _backward / _bound_forward) and the
fused model head (snb_margin_loss, snb_certified_fraction, snb_input_box) against the same
computation done operator by operator (which the other test files pin to the oracle and to the
reference's fixtures): values bit-exact where the operators are, gradients 1e-5."""
import copy

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from gpu_util import rel

pytestmark = pytest.mark.gpu
INF = float("inf")


def _models(keep, depth=4, width=160, classes=10, seed=2):
    from sortnet_b200.layers import SortMLPModel
    torch.manual_seed(seed)
    a = SortMLPModel(depth=depth, width=width, input_dim=(3, 4, 4), num_classes=classes, dropout=keep).cuda()
    for l in a.fc_dist:
        if l.mean_shift is not None:
            l.mean_shift.running_mean.normal_(0.5, 0.1)
    with torch.no_grad():
        a.fc_dist[-1].bias.normal_(0, 0.3)
    return a, copy.deepcopy(a)


def _train_step(model, fused, x, t, eps, masks, p, use_loss_kernel):
    from sortnet_b200 import layers
    layers.FUSED_LAYERS = fused
    try:
        model.set_p(p)
        model.train()
        model.zero_grad(set_to_none=True)
        if use_loss_kernel:
            loss = model.mixture_loss(x, t, eps, lam=0.1, clip=1.0, masks=masks)
            logits = margin = None
        else:
            logits, margin = model(x, targets=t, eps=eps, masks=masks)
            loss = margin.clamp(min=0, max=1.0).max(dim=1)[0].mean() + 0.1 * F.cross_entropy(logits, t)
        loss.backward()
        torch.cuda.synchronize()
    finally:
        layers.FUSED_LAYERS = True
    grads = {k: v.grad.clone() for k, v in model.named_parameters()}
    means = {k: v.clone() for k, v in model.state_dict().items() if "running_mean" in k}
    return loss.detach(), logits, margin, grads, means


@pytest.mark.parametrize("keep,p,B", [(0.8, INF, 96), (0.8, 8.0, 80), (0.8, 31.6, 64), (1.0, INF, 70), (1.0, 3.0, 64)])
def test_training_step_one_call_per_layer_matches_operator_by_operator(keep, p, B):
    a, b = _models(keep)
    g = torch.Generator().manual_seed(B)
    x = torch.rand(B, 3, 4, 4, generator=g).cuda()
    t = torch.randint(0, 10, (B,), generator=g).cuda()
    torch.manual_seed(7)
    masks = a.draw_masks(B, x.device)
    ra = _train_step(a, True, x, t, 0.03, masks, p, False)
    rb = _train_step(b, False, x, t, 0.03, masks, p, False)
    if p == INF:
        assert torch.equal(ra[1], rb[1]) and torch.equal(ra[2], rb[2])
        for k in ra[4]:
            assert torch.equal(ra[4][k], rb[4][k]), k
    else:
        assert rel(ra[1].detach().cpu().numpy(), rb[1].detach().cpu().numpy()) < 2e-6
    for k in ra[3]:
        assert rel(ra[3][k].cpu().numpy(), rb[3][k].cpu().numpy()) < 1e-5, k
    # and with the loss head as one kernel
    rc = _train_step(a, True, x, t, 0.03, masks, p, True)
    assert abs(float(rc[0]) - float(rb[0])) <= 2e-6 * max(1.0, abs(float(rb[0])))
    for k in rc[3]:
        assert rel(rc[3][k].cpu().numpy(), rb[3][k].cpu().numpy()) < 1e-5, k


@pytest.mark.parametrize("B,K,eps", [(64, 10, 8 / 255), (37, 200, 1 / 255), (130, 1000, 0.3), (5, 3, 0.01)])
def test_margin_loss_kernel_value_margin_and_gradient(B, K, eps):
    from sortnet_b200 import norm_dist_cuda as C, ops
    g = torch.Generator().manual_seed(K)
    d0 = (torch.rand(B, K, generator=g) * 0.2 + 1.0).cuda()
    t = torch.randint(0, K, (B,), generator=g).cuda()
    for scale in (1.0, 2.5):
        d = d0.clone().requires_grad_()
        loss = ops.margin_loss(d, t, eps, 1.0, 0.1, scale)
        (loss * 3.0).backward()
        dr = d0.clone().requires_grad_()
        lo, hi = dr - eps, dr + eps
        score, score_lo, score_hi = -dr, -hi, -lo
        margin = (score_hi - torch.gather(score_lo, 1, t.view(-1, 1))).scatter(1, t.view(-1, 1), 0) / (2 * eps)
        want = margin.clamp(min=0, max=1.0).max(dim=1)[0].mean() + 0.1 * F.cross_entropy(score * scale, t)
        (want * 3.0).backward()
        assert abs(float(loss) - float(want)) <= 2e-6 * max(1.0, abs(float(want)))
        assert rel(d.grad.cpu().numpy(), dr.grad.cpu().numpy()) < 1e-5
        m = torch.empty(B, K, device="cuda")
        C.margin_loss(d0, t, eps, 1.0, 0.1, scale, m, torch.empty(B, device="cuda"), torch.empty((), device="cuda"), None)
        # PyTorch divides by the scalar 2 * eps its own way (a reciprocal held in higher precision):
        # the last bit may differ
        assert rel(m.cpu().numpy(), margin.detach().cpu().numpy()) < 5e-7


@pytest.mark.parametrize("keep", [1.0, 0.8])
def test_bound_pass_one_call_per_layer_matches_operator_by_operator(keep):
    from sortnet_b200 import layers
    a, _ = _models(keep, depth=4, width=200)
    a.set_p(INF)
    x = torch.rand(100, 3, 4, 4, device="cuda")
    with torch.no_grad():
        t = a.eval()(x).argmax(dim=1)
    eps = 0.003
    for sort_eval in (False, None):
        got = a.certified_margin(x, t, eps, 1.0, 0.0, sort_eval=sort_eval)
        layers.FUSED_LAYERS = False
        try:
            want = a.certified_margin(x, t, eps, torch.ones(1, device="cuda"), torch.zeros(1, device="cuda"),
                                      sort_eval=sort_eval)
        finally:
            layers.FUSED_LAYERS = True
        assert round(float(got) * 100) == round(float(want) * 100)      # the same rows are certified
    # the layer call itself: point value and bounds bit-exact against the operators
    layer = a.fc_dist[1].eval()
    h = torch.rand(100, layer.in_features, device="cuda")
    lo, hi = h - 0.01, h + 0.01
    with torch.no_grad():
        y, yl, yu = layer(h, lo, hi)
        layers.FUSED_LAYERS = False
        try:
            y2, yl2, yu2 = layer(h, lo, hi)
        finally:
            layers.FUSED_LAYERS = True
    assert torch.equal(y, y2) and torch.equal(yl, yl2) and torch.equal(yu, yu2)


def test_input_box_and_certified_fraction_kernels():
    from sortnet_b200 import norm_dist_cuda as C
    x = torch.rand(50, 97, device="cuda")
    xl, xu = torch.empty_like(x), torch.empty_like(x)
    C.input_box(x, 0.1, 0.0, 1.0, xl, xu)
    assert torch.equal(xl, (x - 0.1).clamp(min=0.0)) and torch.equal(xu, (x + 0.1).clamp(max=1.0))
    g = torch.Generator().manual_seed(1)
    yl = (0.5 + 0.5 * torch.rand(300, 10, generator=g)).cuda()
    yu = yl + 0.1
    t = torch.randint(0, 10, (300,), generator=g).cuda()
    rows = torch.arange(150, device="cuda")
    yl[rows, t[:150]] = 0.0                  # the first half is certified: upper bound of the target
    yu[rows, t[:150]] = 0.2                  # below every other class's lower bound
    frac = torch.empty((), device="cuda")
    C.certified_fraction(yl, yu, t, torch.empty(300, device="cuda"), frac)
    margin = (-yl) - torch.gather(-yu, 1, t.view(-1, 1))
    want = (margin.scatter(1, t.view(-1, 1), float("-inf")).max(dim=1)[0] < 0).float().mean()
    assert round(float(frac) * 300) == round(float(want) * 300) and 0.0 < float(want) < 1.0
