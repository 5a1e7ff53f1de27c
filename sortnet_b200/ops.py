"""Operator / autograd layer: the public names and signatures of the reference's
core/norm_dist.py, implemented on the sm_100a kernels.

    norm_dist(input, weight, p, groups=1, use_custom_cuda_func=True, tag=None)            (:176)
    norm_dist_dropout(input, weight, w_index_ci, w_index_co, p, groups=1, ..., tag=None)   (:191)
    sort_neuron(input, weight, groups=1, q=0.5, truncate=10, ..., tag=None)                (:217)
    bound_sort_neuron(x_lower, x_upper, weight, groups=1, q=0.5, truncate=10, tag=None)    (:234)
    bound_inf_dist(x_lower, x_upper, weight, groups=1, use_custom_cuda_func=True, tag=None) (:246)
    NormDistF (:6), NormDistDropoutF (:54), SortNeuronF (:102), BoundInfDistF (:136)

Beyond the reference's names: norm_dist_layer / NormDistLayerF (distance + mean shift + bias of one
fully connected layer in one call per direction) and margin_loss / MarginLossF (the model's margin
and the mixture loss with their gradient), which `sortnet_b200.layers` uses to keep the host time
of a step below its GPU time at small per-GPU batches.

Tensors are (B, C, HW) contiguous fp32 CUDA, weight is (CO, CI / groups), index lists are int32
(S, groups, count) or None.  The reference's `use_custom_cuda_func=False` switch selected a
slow PyTorch path; there is none here, so asking for it raises.
"""
import math

import torch

from . import _lib
from . import norm_dist_cuda as _C

INF = float("inf")


def _require_kernels(use_custom_cuda_func):
    if not use_custom_cuda_func:
        raise RuntimeError("sortnet_b200 has no PyTorch fallback: use_custom_cuda_func=False is not supported")


def _wants_grad(*tensors):
    return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)


# One implementation serves the plain and the masked distance operator: the plain one is the
# masked one with both index lists absent.
def _dist_forward(ctx, x, weight, ci, co, group, p, record, ascending=False):
    n_out = weight.size(0) if co is None else co.size(-1) * group
    y = torch.empty(x.size(0), n_out, x.size(2), device=x.device, dtype=torch.float32)
    ctx.group, ctx.p, ctx.masks = group, p, (ci, co)
    if math.isinf(p):
        if record:
            pos = torch.empty(y.shape, device=x.device, dtype=torch.int32)
            if ascending and group == 1 and x.size(2) == 1 and (ci is not None or co is not None):
                _C.inf_dist_forward_sorted(x, weight, y, pos, ci, co)
            else:
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
    def forward(ctx, x, weight, w_index_ci, w_index_co, group, p, tag, ascending=False):
        assert weight.size(1) * group == x.size(1) or w_index_ci.size(-1) * group == x.size(1)
        ctx.tag = tag
        return _dist_forward(ctx, x, weight, w_index_ci, w_index_co, group, p, True, ascending)

    @staticmethod
    def backward(ctx, grad_output):
        return _dist_backward(ctx, grad_output) + (None,) * 6


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


def _sink_target(param, need):
    """Where the gradient of `param` is written: (tensor to hand to the kernel, add_after, sink)."""
    if not need:
        return None, False, None
    sink = getattr(param, "grad_sink", None)
    add_after = sink is not None and getattr(param, "grad_sink_written", False)
    target = sink if (sink is not None and not add_after) else torch.empty_like(param)
    return target, add_after, sink


def _sink_finish(param, target, add_after, sink):
    """Returns what autograd gets for `param` (None when the gradient went into its sink)."""
    if sink is None:
        return target
    if add_after:
        sink.add_(target)
    param.grad_sink_written = True
    return None


class NormDistLayerF(torch.autograd.Function):
    """One fully connected norm-distance layer in one call per direction: distance (any p, optional
    index lists), training-mode mean shift (batch mean per channel over the rows that kept it,
    momentum update of `running_mean`, gradient through the mean) and bias.  2-D tensors:
    x [B, CI'], weight [W_CO, W_CI], result [B, CO'].  The arithmetic is that of
    norm_dist_dropout -> MeanShiftDropout -> bias add (core/models/norm_dist.py:85-103), enqueued
    by snb_layer_forward / snb_layer_backward."""

    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, momentum, ci, co, p, shift, record):
        x = x.contiguous()
        B = x.size(0)
        n_out = weight.size(0) if co is None else co.size(-1)
        inf = math.isinf(p)
        dev = x.device
        y = torch.empty(B, n_out, device=dev, dtype=torch.float32)
        pos = ws = mean = None
        if inf and (record or ci is not None or co is not None):
            pos = torch.empty(B, n_out, device=dev, dtype=torch.int32)
            if ci is None and co is None:
                ws = torch.empty(B * n_out, device=dev, dtype=torch.int64)
            else:           # merge keys + full-width input + inverse lists of the ascending-list form
                nbytes = _lib.load().snb_inf_dist_forward_sorted_workspace_bytes(B, n_out, weight.size(1))
                ws = torch.empty((nbytes + 7) // 8, device=dev, dtype=torch.int64)
        elif not inf and p > 10:
            ws = torch.empty(B * n_out, device=dev, dtype=torch.float32)
        if shift:
            mean = torch.empty(weight.size(0), device=dev, dtype=torch.float32)
        # the backward of a finite p needs the distances themselves; for p = inf they may be shifted in place
        out = y if (inf or not record or (not shift and bias is None)) else torch.empty_like(y)
        _C.layer_forward(x, weight, p, ci, co, y, pos, ws, running_mean if shift else None, momentum, mean,
                         bias, out)
        ctx.p, ctx.shift, ctx.masks = p, shift, (ci, co)
        ctx.has_bias = bias is not None
        if record:
            ctx.save_for_backward(x, weight, pos if inf else y, bias)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, weight, third, bias = ctx.saved_tensors
        ci, co = ctx.masks
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_b = ctx.has_bias and ctx.needs_input_grad[2]
        grad_out = grad_out.contiguous()
        inf = math.isinf(ctx.p)
        dev = grad_out.device
        grad_x = torch.empty_like(x) if (need_x or need_w) else None
        gw, gw_add, gw_sink = _sink_target(weight, need_w)
        gb, gb_add, gb_sink = _sink_target(bias, need_b)
        mean = centred = None
        if ctx.shift:
            mean = torch.empty(weight.size(0), device=dev, dtype=torch.float32)
            centred = torch.empty_like(grad_out)
        _C.layer_backward(grad_out, x, weight, None if inf else third, third if inf else None, ctx.p, ci, co,
                          ctx.shift, mean, centred, gb, grad_x, gw)
        return (grad_x if need_x else None, _sink_finish(weight, gw, gw_add, gw_sink) if need_w else None,
                _sink_finish(bias, gb, gb_add, gb_sink) if need_b else None, None, None, None, None, None, None,
                None)


class MarginLossF(torch.autograd.Function):
    """Margin of the training forward plus the `mixture` loss on the head's outputs d [B, K]
    (ell_inf_models.py:45-50 with lower = d - eps, upper = d + eps; main.py:357-364): forward and
    gradient in one kernel (snb_margin_loss).  Returns the scalar loss."""

    @staticmethod
    def forward(ctx, d, targets, eps, clip, lam, scale, need):
        d = d.contiguous()
        B = d.size(0)
        loss = torch.empty((), device=d.device, dtype=torch.float32)
        rows = torch.empty(B, device=d.device, dtype=torch.float32)
        grad = torch.empty_like(d) if need else None
        _C.margin_loss(d, targets.contiguous(), eps, clip, lam, scale, None, rows, loss, grad)
        if need:
            ctx.save_for_backward(grad)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        (grad,) = ctx.saved_tensors
        return grad * grad_loss, None, None, None, None, None, None


def norm_dist_layer(x, weight, bias, p, w_index_ci=None, w_index_co=None, running_mean=None, momentum=0.1):
    """y = (||x - w||_p - batch mean) + bias for 2-D x [B, CI'], training-mode statistics; the mean
    shift is applied when `running_mean` is given (it is updated in place with `momentum`)."""
    shift = running_mean is not None
    record = _wants_grad(x, weight) or (bias is not None and _wants_grad(bias))
    return NormDistLayerF.apply(x, weight, bias, running_mean, momentum, w_index_ci, w_index_co, p, shift, record)


def margin_loss(d, targets, eps, clip=1.0, lam=0.1, scale=1.0):
    return MarginLossF.apply(d, targets, eps, clip, lam, scale, _wants_grad(d))


def norm_dist(input, weight, p, groups=1, use_custom_cuda_func=True, tag=None):
    _require_kernels(use_custom_cuda_func)
    return NormDistF.apply(input, weight, groups, p, _wants_grad(input, weight), tag)


def norm_dist_dropout(input, weight, w_index_ci, w_index_co, p, groups=1, use_custom_cuda_func=True, tag=None):
    """`input` is already compact (dropped channels removed); `weight` is the full matrix."""
    _require_kernels(use_custom_cuda_func)
    return NormDistDropoutF.apply(input, weight, w_index_ci, w_index_co, groups, p, tag)


def norm_dist_dropout_ascending(input, weight, w_index_ci, w_index_co, p, groups=1, tag=None):
    """norm_dist_dropout for index lists in ascending order (sample_mask's, and the reference
    sampler's: core/models/norm_dist.py:14-17): same results; the l-inf forward reads W along whole
    rows (norm_dist_cuda.inf_dist_forward_sorted).  No counterpart in the reference."""
    return NormDistDropoutF.apply(input, weight, w_index_ci, w_index_co, groups, p, tag, True)


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
