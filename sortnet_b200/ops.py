"""Operator / autograd layer: the public names and signatures of the reference's
core/norm_dist.py, implemented on the sm_100a kernels.

    norm_dist(input, weight, p, groups=1, use_custom_cuda_func=True, tag=None)            (:176)
    norm_dist_dropout(input, weight, w_index_ci, w_index_co, p, groups=1, ..., tag=None)   (:191)
    sort_neuron(input, weight, groups=1, q=0.5, truncate=10, ..., tag=None)                (:217)
    bound_sort_neuron(x_lower, x_upper, weight, groups=1, q=0.5, truncate=10, tag=None)    (:234)
    bound_inf_dist(x_lower, x_upper, weight, groups=1, use_custom_cuda_func=True, tag=None) (:246)
    NormDistF (:6), NormDistDropoutF (:54), SortNeuronF (:102), BoundInfDistF (:136)

Tensors are (B, C, HW) contiguous fp32 CUDA, weight is (CO, CI / groups), index lists are int32
(S, groups, count) or None.  The reference's `use_custom_cuda_func=False` switch selected a
slow PyTorch path; there is none here, so asking for it raises.
"""
import math

import torch

from . import norm_dist_cuda as _C

INF = float("inf")


def _require_kernels(use_custom_cuda_func):
    if not use_custom_cuda_func:
        raise RuntimeError("sortnet_b200 has no PyTorch fallback: use_custom_cuda_func=False is not supported")


def _wants_grad(*tensors):
    return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)


# One implementation serves the plain and the masked distance operator: the plain one is the
# masked one with both index lists absent.
def _dist_forward(ctx, x, weight, ci, co, group, p, record):
    n_out = weight.size(0) if co is None else co.size(-1) * group
    y = torch.empty(x.size(0), n_out, x.size(2), device=x.device, dtype=torch.float32)
    ctx.group, ctx.p, ctx.masks = group, p, (ci, co)
    if math.isinf(p):
        if record:
            pos = torch.empty(y.shape, device=x.device, dtype=torch.int32)
            _C.inf_dist_forward(x, weight, y, pos, group, ci, co)
            ctx.save_for_backward(x, weight, pos)
        else:
            _C.inf_dist_forward_nograd(x, weight, y, group)
    elif p > 0:
        _C.norm_dist_forward(x, weight, y, group, p, ci, co)
        ctx.save_for_backward(x, weight, y)
    else:
        raise NotImplementedError("p must be positive")
    return y


def _dist_backward(ctx, grad_y):
    grad_y = grad_y.contiguous()
    need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    x, weight, third = ctx.saved_tensors          # third = argmax words (p = inf) or y (finite p)
    ci, co = ctx.masks
    grad_x = torch.empty_like(x)
    # A weight that carries `grad_sink` (a tensor of its shape, see optim.FlatAdamW) gets its
    # gradient written there and autograd receives None for it: nothing is copied or accumulated
    # in the usual case of one backward per step.  The kernels overwrite their grad_weight, so a
    # sink that this step has already written (a second backward before the optimiser step, a
    # weight used twice in one graph) is added to through a temporary instead.
    sink = getattr(weight, "grad_sink", None) if need_w else None
    add_to_sink = sink is not None and getattr(weight, "grad_sink_written", False)
    grad_w = (sink if (sink is not None and not add_to_sink) else torch.empty_like(weight)) if need_w else None
    if math.isinf(ctx.p):
        if need_w:
            _C.inf_dist_backward_input_weight(grad_y, third, grad_x, grad_w, ctx.group, ci, co)
        elif need_x:
            _C.inf_dist_backward_input(grad_y, third, grad_x, ctx.group)
    else:
        if need_w:
            _C.norm_dist_backward_input_weight(grad_y, x, weight, third, grad_x, grad_w, ctx.group, ctx.p, ci, co)
        elif need_x:
            _C.norm_dist_backward_input(grad_y, x, weight, third, grad_x, ctx.group, ctx.p, ci, co)
    if sink is not None:
        if add_to_sink:
            sink.add_(grad_w)
        weight.grad_sink_written = True
    return (grad_x if need_x else None), (None if sink is not None else grad_w)


class NormDistF(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, group, p, need_grad, tag):
        assert weight.size(1) * group == x.size(1)
        ctx.tag = tag
        return _dist_forward(ctx, x, weight, None, None, group, p, need_grad)

    @staticmethod
    def backward(ctx, grad_output):
        return _dist_backward(ctx, grad_output) + (None,) * 4


class NormDistDropoutF(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, w_index_ci, w_index_co, group, p, tag):
        assert weight.size(1) * group == x.size(1) or w_index_ci.size(-1) * group == x.size(1)
        ctx.tag = tag
        return _dist_forward(ctx, x, weight, w_index_ci, w_index_co, group, p, True)

    @staticmethod
    def backward(ctx, grad_output):
        return _dist_backward(ctx, grad_output) + (None,) * 5


class SortNeuronF(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, group, q, truncate, need_grad, tag):
        assert weight.size(1) * group == x.size(1)
        y = torch.empty(x.size(0), weight.size(0), x.size(2), device=x.device, dtype=torch.float32)
        ctx.args, ctx.tag = (group, q, truncate), tag
        if need_grad:
            pos = torch.empty((truncate,) + tuple(y.shape), device=x.device, dtype=torch.int32)
            _C.sort_neuron_forward(x, weight, y, pos, group, q, truncate)
            ctx.save_for_backward(x, weight, pos)
        else:
            _C.sort_neuron_forward_nograd(x, weight, y, group, q, truncate)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        x, weight, pos = ctx.saved_tensors
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        grad_output = grad_output.contiguous()
        grad_x = torch.empty_like(x)
        grad_w = None
        if need_w:
            grad_w = torch.empty_like(weight)
            _C.sort_neuron_backward_input_weight(grad_output, pos, grad_x, grad_w, *ctx.args)
        elif need_x:
            _C.sort_neuron_backward_input(grad_output, pos, grad_x, *ctx.args)
        return (grad_x if need_x else None), grad_w, None, None, None, None, None


class BoundInfDistF(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_lower, x_upper, weight, group, need_grad, tag):
        assert x_lower.size() == x_upper.size()
        assert weight.size(1) * group == x_lower.size(1)
        shape = (x_lower.size(0), weight.size(0), x_lower.size(2))
        y_lower = torch.empty(shape, device=x_lower.device, dtype=torch.float32)
        y_upper = torch.empty_like(y_lower)
        ctx.group, ctx.tag = group, tag
        if need_grad:
            words = torch.empty((2,) + shape, device=x_lower.device, dtype=torch.int32)
            _C.bound_inf_dist_forward(x_lower, x_upper, weight, y_lower, y_upper, words[0], words[1], group)
            ctx.save_for_backward(x_lower, x_upper, weight, words)
        else:
            _C.bound_inf_dist_forward_nograd(x_lower, x_upper, weight, y_lower, y_upper, group)
        return y_lower, y_upper

    @staticmethod
    def backward(ctx, grad_y_lower, grad_y_upper):
        x_lower, x_upper, weight, words = ctx.saved_tensors
        need_l, need_u, need_w = ctx.needs_input_grad[:3]
        grads = (grad_y_lower.contiguous(), grad_y_upper.contiguous(), words[0], words[1])
        grad_xl = torch.zeros_like(x_lower)
        grad_xu = torch.zeros_like(x_upper)
        grad_w = None
        if need_w:
            grad_w = torch.empty_like(weight)
            _C.bound_inf_dist_backward_input_weight(*grads, grad_xl, grad_xu, grad_w, ctx.group)
        elif need_l and need_u:
            _C.bound_inf_dist_backward_input(*grads, grad_xl, grad_xu, ctx.group)
        return (grad_xl if need_l else None), (grad_xu if need_u else None), grad_w, None, None, None


def norm_dist(input, weight, p, groups=1, use_custom_cuda_func=True, tag=None):
    _require_kernels(use_custom_cuda_func)
    return NormDistF.apply(input, weight, groups, p, _wants_grad(input, weight), tag)


def norm_dist_dropout(input, weight, w_index_ci, w_index_co, p, groups=1, use_custom_cuda_func=True, tag=None):
    """`input` is already compact (dropped channels removed); `weight` is the full matrix."""
    _require_kernels(use_custom_cuda_func)
    return NormDistDropoutF.apply(input, weight, w_index_ci, w_index_co, groups, p, tag)


def _sort_is_plain_max(weight, q, truncate):
    return q is None or q == 1.0 or min(weight.size(-1), truncate) == 1


def sort_neuron(input, weight, groups=1, q=0.5, truncate=10, use_custom_cuda_func=True, tag=None):
    if _sort_is_plain_max(weight, q, truncate):
        return norm_dist(input, weight, INF, groups, tag=tag)
    _require_kernels(use_custom_cuda_func)
    k = min(weight.size(-1), truncate)
    return SortNeuronF.apply(input, weight, groups, q, k, _wants_grad(input, weight), tag)


def bound_sort_neuron(x_lower, x_upper, weight, groups=1, q=0.5, truncate=10, tag=None):
    if _sort_is_plain_max(weight, q, truncate):
        return bound_inf_dist(x_lower, x_upper, weight, groups, tag=tag)
    assert not _wants_grad(x_lower, x_upper, weight)
    k = min(weight.size(-1), truncate)
    y_lower = x_lower.new_empty(x_lower.size(0), weight.size(0), x_lower.size(-1))
    y_upper = torch.empty_like(y_lower)
    _C.bound_sort_neuron_forward(x_lower, x_upper, weight, y_lower, y_upper, groups, q, k)
    return y_lower, y_upper


def bound_inf_dist(x_lower, x_upper, weight, groups=1, use_custom_cuda_func=True, tag=None):
    _require_kernels(use_custom_cuda_func)
    need_grad = _wants_grad(x_lower, x_upper, weight)
    return BoundInfDistF.apply(x_lower, x_upper, weight, groups, need_grad, tag)
