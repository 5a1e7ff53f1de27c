"""The SortNet-MLP harness on the GPU against fixtures produced by the reference's own model
code (unmodified ell_inf_models.SortMLPModel on CPU over the oracle-backed extension stand-in)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from gpu_util import rel

pytestmark = pytest.mark.gpu


def build(g, depth, width, q):
    from sortnet_b200.layers import SortMLPModel
    model = SortMLPModel(depth=depth, width=width, input_dim=(3, 4, 4), num_classes=10, dropout=q).cuda()
    state = {k[len("state0."):]: torch.from_numpy(v) for k, v in g.items() if k.startswith("state0.")}
    missing, unexpected = model.load_state_dict(state, strict=True)
    model.set_p(float(g["p"]))
    return model


def step(model, g, masks):
    x = torch.from_numpy(g["x"]).cuda()
    t = torch.from_numpy(g["targets"]).cuda()
    model.train()
    logits, margin = model(x, targets=t, eps=float(g["eps"]), masks=masks)
    loss = margin.clamp(min=0).max(dim=1)[0].mean() + 0.5 * F.cross_entropy(logits, t)
    loss.backward()
    return logits, margin, loss


@pytest.mark.parametrize("name,depth,width,q", [("model_inf_masked", 4, 96, 0.8), ("model_p8_masked", 4, 96, 0.8),
                                                ("model_inf_plain", 3, 64, 1.0)])
def test_training_step_matches_reference_model(golden, name, depth, width, q):
    g = golden(name)
    model = build(g, depth, width, q)
    masks = None
    if q != 1.0:
        masks = [torch.from_numpy(g["mask%d" % i]).cuda().unsqueeze(1).contiguous() for i in range(depth - 1)]
    logits, margin, loss = step(model, g, masks)
    assert rel(logits.detach().cpu().numpy(), g["logits"]) < 1e-5
    assert rel(margin.detach().cpu().numpy(), g["margin"]) < 1e-5
    assert abs(loss.item() - float(g["loss"])) < 1e-5 * max(1.0, abs(float(g["loss"])))
    for k, prm in model.named_parameters():
        assert rel(prm.grad.cpu().numpy(), g["grad." + k]) < 2e-5, k
    for k, v in model.state_dict().items():
        if "running_mean" in k:
            assert rel(v.cpu().numpy(), g["state1." + k]) < 1e-5, k


def test_certification_forward_matches_reference_model(golden):
    g = golden("model_inf_plain")
    model = build(g, 3, 64, 1.0)
    x = torch.from_numpy(g["x"]).cuda()
    t = torch.from_numpy(g["targets"]).cuda()
    # the fixture's evaluation pass ran after one training step had updated the running means
    step(model, g, None)
    model.eval()
    with torch.no_grad():
        logits, margin = model(x, targets=t, eps=float(g["eps"]), up=torch.ones(1, device="cuda"),
                               down=torch.zeros(1, device="cuda"))
    assert rel(logits.cpu().numpy(), g["eval_logits"]) < 1e-5
    assert rel(margin.cpu().numpy(), g["eval_margin"]) < 1e-5


def test_reference_operator_layer_runs_on_these_kernels():
    """`install()` makes this package importable as `norm_dist_cuda`, the only thing the
    reference's operator layer needs; the operators in sortnet_b200.ops are written against the
    same module object, so exercising them covers the same calls."""
    import sys
    from sortnet_b200 import norm_dist_cuda, ops
    mod = norm_dist_cuda.install()
    assert sys.modules["norm_dist_cuda"] is mod
    x = torch.rand(40, 30, 1, device="cuda", requires_grad=True)
    w = torch.randn(20, 30, device="cuda", requires_grad=True)
    y = ops.norm_dist(x, w, float("inf"))
    y.sum().backward()
    assert x.grad.shape == x.shape and w.grad.shape == w.shape
    with torch.no_grad():
        y2 = ops.norm_dist(x, w, float("inf"))
    assert torch.equal(y, y2)
    with pytest.raises(RuntimeError):
        ops.norm_dist(x, w, 2.0, use_custom_cuda_func=False)


def test_update_running_means_is_the_average_of_batch_means():
    from sortnet_b200.layers import SortMLPModel, update_running_means
    torch.manual_seed(3)
    model = SortMLPModel(depth=3, width=64, input_dim=(1, 4, 4), num_classes=5, dropout=1.0).cuda()
    model.set_p(8.0)
    batches = [torch.rand(64, 1, 4, 4, device="cuda") for _ in range(3)]
    update_running_means(model, batches)
    assert all(l.p == 8.0 for l in model.fc_dist) and model.training
    assert model.fc_dist[0].mean_shift.momentum == 0.1
    # first layer: its input does not depend on any running mean, so the expected value is direct
    from sortnet_b200 import ops
    w = model.fc_dist[0].weight
    means = [ops.norm_dist(b.reshape(64, -1, 1), w, float("inf")).mean(dim=(0, 2)) for b in batches]
    want = torch.stack(means).mean(dim=0)
    got = model.fc_dist[0].mean_shift.running_mean
    assert (got - want).abs().max() <= 1e-5 * want.abs().max()


@pytest.mark.parametrize("keep", [0.8, 1.0])
def test_certified_margin_agrees_with_the_evaluation_forward(keep):
    """The certified fraction must be the one the evaluation-mode forward certifies (the sort neuron
    and its bounds when the keep rate is below 1); sort_eval=False is the plain l-inf bound
    workload and differs for such a model."""
    from sortnet_b200.layers import SortMLPModel
    torch.manual_seed(5)
    model = SortMLPModel(depth=4, width=128, input_dim=(3, 4, 4), num_classes=10, dropout=keep, std=0.3).cuda()
    for l in model.fc_dist:
        if l.mean_shift is not None:
            l.mean_shift.running_mean.normal_(1.0, 0.2)
    x = torch.rand(96, 3, 4, 4, device="cuda")
    with torch.no_grad():
        t = model.eval()(x).argmax(dim=1)          # labels the network gets right: margins near the boundary
    eps = 0.002
    up, down = torch.ones(1, device="cuda"), torch.zeros(1, device="cuda")
    with torch.no_grad():
        _, margin = model(x, targets=t, eps=eps, up=up, down=down)
    want = (margin.scatter(1, t.view(-1, 1), float("-inf")).max(dim=1)[0] < 0).float().mean()
    got = model.certified_margin(x, t, eps, up, down)
    assert round(float(got) * 96) == round(float(want) * 96)         # the same rows are certified
    assert not model.training
    plain = model.certified_margin(x, t, eps, up, down, sort_eval=False)
    if keep == 1.0:
        assert float(plain) == float(got)
