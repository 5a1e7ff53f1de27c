"""Fused flat-buffer AdamW and the gradient sink against torch.optim.AdamW on the same model."""
import copy

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def loss_of(model, x, t, masks):
    logits, margin = model(x, targets=t, eps=0.03, masks=masks)
    return margin.clamp(min=0, max=1).max(dim=1)[0].mean() + 0.1 * F.cross_entropy(logits, t)


@pytest.mark.parametrize("p_norm,wd", [(float("inf"), 0.0), (8.0, 0.02)])
def test_flat_adamw_matches_torch_adamw(p_norm, wd):
    from sortnet_b200.layers import SortMLPModel
    from sortnet_b200.optim import FlatAdamW
    torch.manual_seed(0)
    ref = SortMLPModel(depth=4, width=96, input_dim=(3, 4, 4), num_classes=10, dropout=0.8, scalar=True).cuda()
    ref.set_p(p_norm)
    mine = copy.deepcopy(ref)
    opt_ref = torch.optim.AdamW(ref.parameters(), lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=wd)
    opt = FlatAdamW(mine, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=wd)
    names = [n for n, _ in mine.named_parameters()]
    for n, p in mine.named_parameters():
        assert p.data_ptr() >= opt.flat_param.data_ptr() and hasattr(p, "grad_sink"), n
    for step in range(3):
        x = torch.rand(70, 3, 4, 4, device="cuda")
        t = torch.randint(0, 10, (70,), device="cuda")
        masks = ref.draw_masks(70, x.device)
        opt_ref.zero_grad(set_to_none=True)
        loss_of(ref.train(), x, t, masks).backward()
        grads_ref = {n: p.grad.clone() for n, p in ref.named_parameters()}
        opt_ref.step()
        opt.zero_grad()
        loss_of(mine.train(), x, t, masks).backward()
        for n, p in mine.named_parameters():
            if n.endswith("weight"):
                assert p.grad is None, "weight gradients go to the sink, not through autograd"
        opt.gather_grads()
        for n, p in mine.named_parameters():
            g = p.grad_sink
            assert (g - grads_ref[n]).abs().max() <= 2e-5 * max(grads_ref[n].abs().max().item(), 1e-12), n
            # Adam with eps = 1e-10 turns a gradient entry that cancels to exactly 0 in one summation
            # order and to 1e-9 in another into updates of 0 and lr: compare the optimiser itself on
            # identical gradients
            g.copy_(grads_ref[n])
        opt.step()
        for (n, a), (_, b) in zip(ref.named_parameters(), mine.named_parameters()):
            assert (a - b).abs().max() <= 1e-5 * max(a.abs().max().item(), 1.0), (step, n)
    assert set(mine.state_dict().keys()) == set(ref.state_dict().keys()) and names


def test_adamw_argument_checks():
    from sortnet_b200 import _lib
    lib = _lib.load()
    buf = torch.zeros(16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    args = (buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr())
    assert lib.snb_adamw_step(*args, 6, 0.1, 0.9, 0.99, 1e-8, 0.0, 1, 1.0, st) == 2      # not a multiple of 4
    assert lib.snb_adamw_step(*args, 16, 0.1, 0.9, 0.99, 1e-8, 0.0, 0, 1.0, st) == 2     # steps count from 1
    assert lib.snb_adamw_step(None, *args[1:], 16, 0.1, 0.9, 0.99, 1e-8, 0.0, 1, 1.0, st) == 1
    assert lib.snb_adamw_step(buf.data_ptr() + 4, *args[1:], 12, 0.1, 0.9, 0.99, 1e-8, 0.0, 1, 1.0, st) == 6


@pytest.mark.parametrize("parts", [1, 3, 8])
def test_reduce_step_equals_plain_step_on_the_summed_gradient(parts):
    """snb_adamw_reduce_step (partial gradient buffers, separate output buffer) against snb_adamw_step
    on their sum."""
    import ctypes
    from sortnet_b200 import _lib
    lib = _lib.load()
    torch.manual_seed(parts)
    n = 4 * 1000 + 4
    w = torch.randn(n, device="cuda")
    gs = [torch.randn(n, device="cuda") for _ in range(parts)]
    m = torch.rand(n, device="cuda") * 0.1
    v = torch.rand(n, device="cuda") * 0.01
    args = (0.02, 0.9, 0.99, 1e-8, 0.01, 3, 1.0 / parts)
    st = torch.cuda.current_stream().cuda_stream
    w_ref, m_ref, v_ref = w.clone(), m.clone(), v.clone()
    total = gs[0].clone()
    for g in gs[1:]:
        total += g
    assert lib.snb_adamw_step(w_ref.data_ptr(), total.data_ptr(), m_ref.data_ptr(), v_ref.data_ptr(), n, *args, st) == 0
    w_dst = torch.full_like(w, float("nan"))
    m2, v2 = m.clone(), v.clone()
    ptrs = (ctypes.c_void_p * parts)(*[g.data_ptr() for g in gs])
    assert lib.snb_adamw_reduce_step(w.data_ptr(), w_dst.data_ptr(), ptrs, parts, m2.data_ptr(), v2.data_ptr(), n,
                                     *args, st) == 0
    torch.cuda.synchronize()
    assert torch.allclose(w_dst, w_ref, rtol=0, atol=1e-6) and torch.allclose(m2, m_ref, atol=1e-7)
    assert torch.allclose(v2, v_ref, atol=1e-7)
    # argument checks
    assert lib.snb_adamw_reduce_step(w.data_ptr(), w_dst.data_ptr(), ptrs, 17, m2.data_ptr(), v2.data_ptr(), n,
                                     *args, st) == 3
    assert lib.snb_adamw_reduce_step(w.data_ptr(), w_dst.data_ptr(), ptrs, parts, m2.data_ptr(), v2.data_ptr(), n + 1,
                                     *args, st) == 2


def test_gradient_sinks_accumulate_and_unreached_parameters_get_zero():
    """Two backwards before one step add up in the sink (like autograd's .grad); a parameter that no
    backward reached since the last step has a zero gradient, not the previous step's."""
    from sortnet_b200.layers import SortMLPModel
    from sortnet_b200.optim import FlatAdamW
    torch.manual_seed(1)
    model = SortMLPModel(depth=3, width=64, input_dim=(1, 4, 4), num_classes=5, dropout=1.0).cuda()
    ref = copy.deepcopy(model)
    opt = FlatAdamW(model, lr=0.01)
    x1, x2 = torch.rand(64, 1, 4, 4, device="cuda"), torch.rand(64, 1, 4, 4, device="cuda")
    t = torch.randint(0, 5, (64,), device="cuda")
    opt.zero_grad()
    loss_of(model.train(), x1, t, None).backward()
    loss_of(model.train(), x2, t, None).backward()
    opt.gather_grads()
    loss_of(ref.train(), x1, t, None).backward()
    loss_of(ref.train(), x2, t, None).backward()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert (p.grad_sink - q.grad).abs().max() <= 2e-5 * max(q.grad.abs().max().item(), 1e-12), n
    opt.step()
    # next step: only the head is used (the hidden layers are bypassed), their gradient must be zero
    before = [p.detach().clone() for p in model.parameters()]
    opt.zero_grad()
    head = model.fc_dist[-1]
    h = torch.rand(64, head.in_features, device="cuda")
    out, _, _ = head(h)
    out.sum().backward()
    opt.gather_grads()
    opt._prepare_grads()
    for n, p in model.named_parameters():
        if not n.startswith("fc_dist.2."):
            assert float(p.grad_sink.abs().max()) == 0.0, n
    assert float(head.weight.grad_sink.abs().max()) > 0.0
    del before


def test_gradient_all_reduce_refuses_parameters_with_sinks():
    from sortnet_b200.dist import GradientAllReduce
    from sortnet_b200.layers import SortMLPModel
    from sortnet_b200.optim import FlatAdamW
    model = SortMLPModel(depth=3, width=32, input_dim=(1, 4, 4), num_classes=5, dropout=1.0).cuda()
    FlatAdamW(model)
    with pytest.raises(ValueError, match="FlatAdamW"):
        GradientAllReduce(model.parameters())
