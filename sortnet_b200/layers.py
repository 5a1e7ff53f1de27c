"""Layers around the operators: mask sampling, the mean-shift module, the norm-distance
layer and a SortNet-MLP built from them.

What is mirrored from the reference
    sample_mask          core/models/norm_dist.py:14-17   (same index-list format)
    MeanShiftDropout     core/models/bound_basic_module.py:107-160  (forward signature, buffer name
                         `running_mean`, momentum rule, gradient through the batch mean)
    NormDist             core/models/norm_dist.py:20-121  (parameters `weight` [CO, CI], `bias`;
                         std / identity initialisation; attribute `p`; returns the triple
                         (x, lower, upper))
    NormDistConv         core/models/norm_dist.py:130-164  (unfold + grouped distance, 4-D in/out)
    SortMLPModel         ell_inf_models.py:17-50           (layer stack, forward signature, margin)
so a reference checkpoint's state_dict loads into SortMLPModel unchanged.

What is designed differently: the reference threads the sub-batch masks from one layer to the
next through class-level globals (NormDistBase.dropout_list / dropout_buffer); here the model
owns its layers and hands each one the masks explicitly, and mean-shift runs in two small
deterministic kernels instead of a dozen PyTorch launches.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import norm_dist_cuda as _C
from . import ops

SUB_BATCH = 32
# One library call per fully connected layer and direction where that applies (see NormDist.forward);
# False takes the operators one by one everywhere (the results are the same).
FUSED_LAYERS = True


def sample_mask(batch, groups, channel, q, device, count=None):
    """Kept-channel lists for `batch` sub-batches: one Binomial(channel, q) count shared by all
    sub-batches (drawn here unless the caller supplies it), a uniformly random subset of that
    size per (sub-batch, group), sorted, int32, shape [batch, groups, count].

    On a CUDA device the count and a 64-bit seed come from PyTorch's host generator (so
    torch.manual_seed makes the masks reproducible and nothing waits for the GPU) and one kernel
    writes all lists; on the CPU the lists are made with PyTorch ops the way the reference does."""
    device = torch.device(device)
    if device.type == "cuda":
        if count is None:
            count = int((torch.rand(channel) < q).sum())
        count = min(max(int(count), 1), channel)
        seed = int(torch.randint(0, 2 ** 62, (1,)))
        out = torch.empty(batch, groups, count, dtype=torch.int32, device=device)
        _C.sample_mask_into(out, channel, seed)
        return out
    if count is None:
        count = int((torch.rand(channel, device=device) < q).sum().item())
    scores = torch.rand(batch, groups, channel, device=device)
    picked = torch.topk(scores, k=count, dim=-1, sorted=False)[1].int()
    return torch.sort(picked)[0]


def _as_index32(index):
    if index is None:
        return None
    if index.dtype != torch.int32:
        index = index.int()
    return index.contiguous()


def _global_index(index, channels):
    """[S, G, kept per group] lists of within-group channels -> [S, G * kept] lists of channels
    of the whole layer (group g owns channels g * channels / G ...), still ascending."""
    S, G, kept = index.shape
    base = torch.arange(G, device=index.device, dtype=torch.long).view(1, G, 1) * (channels // G)
    return (index.long() + base).reshape(S, G * kept)


def _plane_index(index, channels, hw):
    """Index lists over the flattened (channel, position) plane of a [B, C, HW] tensor, in the
    [S, 1, n] int32 form the mean-shift kernels take; None stays None."""
    if index is None:
        return None
    glob = _global_index(index, channels)
    if hw > 1:
        glob = (glob.unsqueeze(-1) * hw + torch.arange(hw, device=glob.device)).reshape(glob.size(0), -1)
    return glob.int().unsqueeze(1).contiguous()


class _MeanShiftPlaneF(torch.autograd.Function):
    """The centring of _MeanShiftTrainF for x [B, C, HW] and grouped index lists
    (core/models/bound_basic_module.py:125-139: the mean runs over rows and positions).  The
    statistics kernel sees the (channel, position) plane as one long channel axis; every
    position of a channel has the same row count, so the channel mean is the plain average of
    its per-position means."""

    @staticmethod
    def forward(ctx, x, plane_index, channels):
        B, hw = x.size(0), x.size(-1)
        flat = x.contiguous().view(B, -1, 1)
        per_pos = torch.empty(channels * hw, device=x.device, dtype=torch.float32)
        _C.mean_shift_stats(flat, plane_index, per_pos, None, 0.0)
        mean = per_pos.view(channels, hw).mean(dim=1)
        y = torch.empty_like(flat)
        _C.mean_shift_apply(flat, mean.repeat_interleave(hw), plane_index, y)
        ctx.plane_index, ctx.channels = plane_index, channels
        ctx.mark_non_differentiable(mean)
        return y.view(x.shape), mean

    @staticmethod
    def backward(ctx, grad_y, _grad_mean):
        B, hw = grad_y.size(0), grad_y.size(-1)
        flat = grad_y.contiguous().view(B, -1, 1)
        per_pos = torch.empty(ctx.channels * hw, device=grad_y.device, dtype=torch.float32)
        _C.mean_shift_stats(flat, ctx.plane_index, per_pos, None, 0.0)
        gmean = per_pos.view(ctx.channels, hw).mean(dim=1)
        grad_x = torch.empty_like(flat)
        _C.mean_shift_apply(flat, gmean.repeat_interleave(hw), ctx.plane_index, grad_x)
        return grad_x.view(grad_y.shape), None, None


class _MeanShiftTrainF(torch.autograd.Function):
    """y = x - mean(x) with the mean taken over the rows whose sub-batch kept the channel.
    The backward applies the same centring to the incoming gradient."""

    @staticmethod
    def forward(ctx, x, index, running_mean, momentum):
        x = x.contiguous()
        mean = torch.empty(running_mean.numel(), device=x.device, dtype=torch.float32)
        _C.mean_shift_stats(x, index, mean, running_mean, momentum)
        y = torch.empty_like(x)
        _C.mean_shift_apply(x, mean, index, y)
        ctx.index = index
        ctx.channels = running_mean.numel()
        ctx.mark_non_differentiable(mean)
        return y, mean

    @staticmethod
    def backward(ctx, grad_y, _grad_mean):
        grad_y = grad_y.contiguous()
        gmean = torch.empty(ctx.channels, device=grad_y.device, dtype=torch.float32)
        _C.mean_shift_stats(grad_y, ctx.index, gmean, None, 0.0)
        grad_x = torch.empty_like(grad_y)
        _C.mean_shift_apply(grad_y, gmean, ctx.index, grad_x)
        return grad_x, None, None, None


class MeanShiftDropout(nn.Module):
    """Subtracts the per-channel batch mean (training) or the running mean (evaluation)."""

    def __init__(self, out_channels, momentum=0.1, affine=True):
        super().__init__()
        self.out_channels = out_channels
        self.momentum = momentum
        self.affine = affine
        self.register_buffer("running_mean", torch.zeros(out_channels))
        if affine:
            self.bias = nn.Parameter(torch.zeros(out_channels))
        else:
            self.register_parameter("bias", None)

    def forward(self, x=None, lower=None, upper=None, index=None):
        """x, lower, upper: (B, C, HW) or None; index: kept channels [S, groups, C / groups] (sorted
        within each group) or None."""
        index = _as_index32(index)
        some = x if x is not None else lower
        hw = some.size(-1)
        plane = hw != 1 or (index is not None and index.size(1) != 1)
        kernel_index = _plane_index(index, self.out_channels, hw) if plane else index
        if self.training:
            assert x is not None, "training needs the activations"
            if plane:
                x, mean = _MeanShiftPlaneF.apply(x, kernel_index, self.out_channels)
                with torch.no_grad():
                    self.running_mean.mul_(1 - self.momentum).add_(mean, alpha=self.momentum)
            else:
                x, mean = _MeanShiftTrainF.apply(x, index, self.running_mean, self.momentum)
            if self.bias is not None:
                x = x + self._gathered(self.bias, index, x.size(0)).unsqueeze(-1)
                mean = mean - self.bias.detach()
            x_done, todo = x, (None, lower, upper)
        else:
            mean = self.running_mean if self.bias is None else self.running_mean - self.bias.detach()
            x_done, todo = None, (x, lower, upper)
        if plane and hw > 1:
            mean = mean.repeat_interleave(hw)
        outs = []
        for z in todo:
            if z is None:
                outs.append(None)
                continue
            z = z.contiguous()
            out = torch.empty_like(z)
            if plane:
                _C.mean_shift_apply(z.view(z.size(0), -1, 1), mean, kernel_index, out.view(z.size(0), -1, 1))
            else:
                _C.mean_shift_apply(z, mean, index, out)
            outs.append(out)
        if x_done is not None:
            outs[0] = x_done
        return tuple(outs)

    @staticmethod
    def _gathered(vec, index, batch):
        """vec [C_full] -> [batch or 1, C]: the entries of the channels each row's sub-batch kept."""
        if index is None:
            return vec.unsqueeze(0)
        rows = torch.arange(batch, device=vec.device) // SUB_BATCH
        return vec[_global_index(index, vec.numel())[rows]]

    def extra_repr(self):
        return "{}, affine={}".format(self.out_channels, self.affine)


class NormDist(nn.Module):
    """Fully connected norm-distance layer y_j = ||x - w_j||_p (+ mean shift, + bias).

    `dropout` is the *keep* rate q of the sort neuron this layer estimates during training
    (None or 1.0 = plain l-p / l-inf distance).  Inputs and outputs are 2-D (B, C)."""

    def __init__(self, in_features, out_features, p=float("inf"), bias=True, std=1.0, mean_shift=True,
                 dropout=None, identity_val=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.p = p
        self.dropout = dropout
        self.weight = nn.Parameter(torch.randn(out_features, in_features) * std)
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.mean_shift = MeanShiftDropout(out_features, affine=False) if mean_shift else None
        if identity_val is not None and in_features <= out_features:
            with torch.no_grad():
                rows = torch.arange(out_features)
                self.weight[rows, rows % in_features] = -identity_val

    @property
    def keep_rate(self):
        return 1.0 if self.dropout is None else self.dropout

    def forward(self, x=None, lower=None, upper=None, mask_in=None, mask_out=None, sort_eval=False):
        """With masks (training): x is compact over `mask_in`, the result compact over `mask_out`;
        every index list must be ascending, as `sample_mask` returns it (the l-inf forward then reads
        W along whole rows; lists in another order would still give exact distances, but ties for
        the maximum could resolve to another tied position than the reference's).
        Without masks: the l-p / l-inf distance of the point value and, when a box
        (lower, upper) is given, its interval bounds (p must be inf).  `sort_eval=True` replaces
        the distance by the deterministic sort neuron with q = `dropout` (the expectation of
        the masked training-time neuron), as the reference does outside training.

        Two cases run as one library call per layer (distance + mean shift + bias together, see
        ops.NormDistLayerF and snb_layer_bound_forward): the training-mode forward of the point
        value, and the evaluation-mode l-inf pass without gradients.  Everything else takes the
        operators one by one."""
        masked = mask_in is not None or mask_out is not None
        box = lower is not None and upper is not None
        if FUSED_LAYERS and x is not None and x.is_cuda and not sort_eval:
            if self.training and not box:
                rm = self.mean_shift.running_mean if self.mean_shift is not None else None
                mom = self.mean_shift.momentum if self.mean_shift is not None else 0.0
                y = ops.norm_dist_layer(x, self.weight, self.bias, self.p, _as_index32(mask_in),
                                        _as_index32(mask_out), rm, mom)
                return y, None, None
            if (not self.training and not masked and math.isinf(self.p)
                    and not (torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad
                                                          or (box and (lower.requires_grad or upper.requires_grad))))):
                return self._eval_linf(x, lower if box else None, upper if box else None)
        x3, l3, u3 = (None if z is None else z.unsqueeze(-1).contiguous() for z in (x, lower, upper))
        if masked:
            x3 = ops.norm_dist_dropout_ascending(x3, self.weight, mask_in, mask_out, self.p)
        elif not sort_eval:
            if x3 is not None:
                x3 = ops.norm_dist(x3, self.weight, self.p)
            if l3 is not None and u3 is not None:
                assert math.isinf(self.p)
                l3, u3 = ops.bound_inf_dist(l3, u3, self.weight)
        else:
            x3 = ops.sort_neuron(x3, self.weight, q=self.dropout)
            if l3 is not None and u3 is not None:
                l3, u3 = ops.bound_sort_neuron(l3, u3, self.weight, q=self.dropout)
        if self.mean_shift is not None:
            x3, l3, u3 = self.mean_shift(x3, l3, u3, index=mask_out)
        if self.bias is not None:
            b = MeanShiftDropout._gathered(self.bias, mask_out, x3.size(0) if x3 is not None else l3.size(0))
            x3, l3, u3 = (None if z is None else z + b.unsqueeze(-1) for z in (x3, l3, u3))
        return tuple(None if z is None else z.squeeze(-1) for z in (x3, l3, u3))

    def _eval_linf(self, x, lower, upper):
        """Evaluation-mode l-inf layer without gradients: point value, interval bounds, running
        mean and bias in one library call."""
        x = x.contiguous()
        B, dev = x.size(0), x.device
        y = torch.empty(B, self.out_features, device=dev, dtype=torch.float32)
        yl = yu = None
        if lower is not None:
            lower, upper = lower.contiguous(), upper.contiguous()
            yl, yu = torch.empty_like(y), torch.empty_like(y)
        rm = self.mean_shift.running_mean if self.mean_shift is not None else None
        _C.layer_bound_forward(x, lower, upper, self.weight, rm, self.bias, y, yl, yu)
        return y, yl, yu

    def extra_repr(self):
        return "in_features={}, out_features={}, bias={}, keep={}".format(
            self.in_features, self.out_features, self.bias is not None, self.dropout)


class NormDistConv(nn.Module):
    """Convolutional norm-distance layer (core/models/norm_dist.py:130-164): every output pixel
    is the distance between the unfolded input patch and a weight row, per channel group.

    Parameters as in the reference: `weight` [out_channels, in_channels / groups * kh * kw],
    optional `bias` [out_channels], `mean_shift.running_mean`.  Inputs and outputs are 4-D
    (B, C, H, W).  With masks (training of the sort-neuron estimate) the input must already be
    compact over `mask_in` [S, groups, kept]; that is the case between 1x1 layers, whose compact
    output over `mask_out` is the next layer's compact input."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 p=float("inf"), bias=True, std=1.0, mean_shift=True, dropout=None, identity_val=None):
        super().__init__()
        if not isinstance(kernel_size, (tuple, list)):
            kernel_size = (kernel_size, kernel_size)
        kernel_size = tuple(kernel_size)
        assert in_channels % groups == 0 and out_channels % groups == 0
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.dilation = kernel_size, stride, padding, dilation
        self.groups, self.p, self.dropout = groups, p, dropout
        fan_in = in_channels // groups * kernel_size[0] * kernel_size[1]
        self.weight = nn.Parameter(torch.randn(out_channels, fan_in) * std)
        self.bias = nn.Parameter(torch.zeros(out_channels)) if bias else None
        self.mean_shift = MeanShiftDropout(out_channels, affine=False) if mean_shift else None
        if identity_val is not None and in_channels <= out_channels:
            with torch.no_grad():
                w4 = self.weight.view(out_channels, -1, *kernel_size)
                rows = torch.arange(out_channels)
                w4[rows, rows % (in_channels // groups), kernel_size[0] // 2, kernel_size[1] // 2] = -identity_val

    @property
    def keep_rate(self):
        return 1.0 if self.dropout is None else self.dropout

    def _unfold(self, z):
        if z is None:
            return None
        if self.kernel_size == (1, 1) and self.stride == 1 and self.padding == 0:
            return z.reshape(z.size(0), z.size(1), -1).contiguous()
        return F.unfold(z, self.kernel_size, self.dilation, self.padding, self.stride).contiguous()

    def forward(self, x=None, lower=None, upper=None, mask_in=None, mask_out=None, sort_eval=False):
        some = x if x is not None else lower
        h, w = ((n + 2 * self.padding - self.dilation * (k - 1) - 1) // self.stride + 1
                for n, k in zip(some.shape[2:], self.kernel_size))
        x3, l3, u3 = self._unfold(x), self._unfold(lower), self._unfold(upper)
        if mask_in is not None or mask_out is not None:
            x3 = ops.norm_dist_dropout(x3, self.weight, mask_in, mask_out, self.p, self.groups)
        elif not sort_eval:
            if x3 is not None:
                x3 = ops.norm_dist(x3, self.weight, self.p, self.groups)
            if l3 is not None and u3 is not None:
                assert math.isinf(self.p)
                l3, u3 = ops.bound_inf_dist(l3, u3, self.weight, self.groups)
        else:
            x3 = ops.sort_neuron(x3, self.weight, self.groups, q=self.dropout)
            if l3 is not None and u3 is not None:
                l3, u3 = ops.bound_sort_neuron(l3, u3, self.weight, self.groups, q=self.dropout)
        if self.mean_shift is not None:
            x3, l3, u3 = self.mean_shift(x3, l3, u3, index=mask_out)
        if self.bias is not None:
            b = MeanShiftDropout._gathered(self.bias, mask_out, some.size(0)).unsqueeze(-1)
            x3, l3, u3 = (None if z is None else z + b for z in (x3, l3, u3))
        return tuple(None if z is None else z.view(z.size(0), -1, h, w) for z in (x3, l3, u3))

    def extra_repr(self):
        return "{}, {}, kernel_size={}, stride={}, groups={}, bias={}, keep={}".format(
            self.in_channels, self.out_channels, self.kernel_size, self.stride, self.groups,
            self.bias is not None, self.dropout)


class SortMLPModel(nn.Module):
    """depth norm-distance layers: pixels -> width -> ... -> width -> num_classes.

    Layers 2..depth estimate the sort neuron with keep rate `dropout` on their inputs, so the
    outputs of layers 1..depth-1 are sub-sampled; the head has a bias and no mean shift."""

    def __init__(self, depth, width, input_dim, num_classes=10, dropout=0.7, std=1.0, identity_val=None,
                 scalar=False):
        super().__init__()
        pixels = input_dim[0] * input_dim[1] * input_dim[2]
        kw = dict(std=std, identity_val=identity_val)
        layers = [NormDist(pixels, width, bias=False, mean_shift=True, **kw)]
        for _ in range(depth - 2):
            layers.append(NormDist(width, width, bias=False, mean_shift=True, dropout=dropout, **kw))
        layers.append(NormDist(width, num_classes, bias=True, mean_shift=False, dropout=dropout, **kw))
        self.fc_dist = nn.ModuleList(layers)
        if isinstance(scalar, float):
            self.scalar = scalar
        else:
            self.scalar = nn.Parameter(torch.ones(1)) if scalar else 1

    def set_p(self, p):
        for layer in self.fc_dist:
            layer.p = p

    def _certifying(self):
        return all(math.isinf(l.p) and not l.training for l in self.fc_dist)

    def draw_masks(self, batch, device):
        """One kept-channel list per hidden activation (None where the next layer keeps all)."""
        sub = (batch - 1) // SUB_BATCH + 1
        todo = [(k, l) for k, l in enumerate(self.fc_dist[1:]) if l.keep_rate != 1.0]
        masks = [None] * (len(self.fc_dist) - 1)
        if not todo:
            return masks
        # The Binomial(in_features, keep) counts fix tensor shapes, so the host must know them: they
        # are drawn from the host generator (a few thousand uniforms) instead of on the device, which
        # would cost a device synchronisation per step and stop the host from queueing kernels
        # ahead of the GPU.
        counts = [int((torch.rand(l.in_features) < l.keep_rate).sum()) for _, l in todo]
        device = torch.device(device)
        if device.type == "cuda" and 1 < len(todo) <= 16:
            # all layers' lists in one launch; counts, seeds and lists are those of the per-layer calls
            outs, seeds = [], []
            for (k, l), c in zip(todo, counts):
                c = min(max(int(c), 1), l.in_features)
                seeds.append(int(torch.randint(0, 2 ** 62, (1,))))
                outs.append(torch.empty(sub, 1, c, dtype=torch.int32, device=device))
                masks[k] = outs[-1]
            _C.sample_masks_into(outs, [l.in_features for _, l in todo], seeds)
            return masks
        for (k, l), c in zip(todo, counts):
            masks[k] = sample_mask(sub, 1, l.in_features, l.keep_rate, device, count=max(int(c), 1))
        return masks

    @torch.no_grad()
    def certified_margin(self, x, targets, eps, up, down, sort_eval=None, after_layer=None):
        """Evaluation-mode interval-bound pass over the box [x - eps, x + eps] clipped to
        [down, up], running means subtracted.  Returns the fraction of rows whose worst-case
        margin is negative for every wrong class.

        sort_eval=None (default) propagates what `forward()` propagates in evaluation mode: the
        sort neuron and its bounds for layers with a keep rate below 1, the plain l-inf distance
        and `bound_inf_dist` otherwise -- the returned fraction is then the certified accuracy of
        the network that is actually evaluated (main.py:205-240 does the same through the model's
        forward).  sort_eval=False forces the plain l-inf distance and its interval bounds in
        every layer, whatever the keep rates: that is the l-inf interval-bound workload
        (bound_inf_dist_cuda.cu), and a certificate only for a network whose keep rates are all 1;
        for a sort-neuron network the number it returns is NOT a certified accuracy, because the
        sort neuron's output lies below the l-inf distance.

        after_layer: optional callable(k), called after layer k has been queued; a caller that
        overlaps other work with this pass (optim.FlatAdamW.apply_update) uses it to place that
        work between two layers."""
        was_training = self.training
        self.eval()
        if sort_eval is None:
            sort_eval = any(l.keep_rate != 1.0 for l in self.fc_dist)
        try:
            x = x.reshape(x.size(0), -1)
            scalars = isinstance(up, (int, float)) and isinstance(down, (int, float))
            if FUSED_LAYERS and scalars and x.is_cuda:
                x = x.contiguous()
                lower, upper = torch.empty_like(x), torch.empty_like(x)
                _C.input_box(x, eps, down, up, lower, upper)
            else:
                lower = torch.maximum(x - eps, torch.as_tensor(down, device=x.device))
                upper = torch.minimum(x + eps, torch.as_tensor(up, device=x.device))
            for k, layer in enumerate(self.fc_dist):
                assert math.isinf(layer.p)
                x, lower, upper = layer(x, lower, upper, sort_eval=sort_eval and layer.keep_rate != 1.0)
                if after_layer is not None:
                    after_layer(k)
            if FUSED_LAYERS and x.is_cuda:
                frac = torch.empty((), device=x.device, dtype=torch.float32)
                rows = torch.empty(x.size(0), device=x.device, dtype=torch.float32)
                _C.certified_fraction(lower.contiguous(), upper.contiguous(), targets.contiguous(), rows, frac)
                return frac
            score_lo, score_hi = -upper, -lower
            margin = score_hi - torch.gather(score_lo, 1, targets.view(-1, 1))
            margin = margin.scatter(1, targets.view(-1, 1), float("-inf"))
            return (margin.max(dim=1)[0] < 0).float().mean()
        finally:
            self.train(was_training)

    def mixture_loss(self, x, targets, eps, lam=0.1, clip=1.0, masks=None):
        """Training forward followed by the reference's `mixture` loss (main.py:357-364) on the
        margin of ell_inf_models.py:45-50: mean_b max_c clamp(margin, 0, clip) + lam * cross_entropy.
        Same value and gradients as `forward(x, targets, eps)` followed by that loss in PyTorch
        ops; the head (margin, loss and its gradient) runs as one kernel."""
        d = self._distances(x, masks)
        if FUSED_LAYERS and d.is_cuda and not isinstance(self.scalar, torch.Tensor):
            return ops.margin_loss(d, targets, eps, clip, lam, float(self.scalar))
        score, margin = self._scores(d, None, None, targets, eps)
        return margin.clamp(min=0, max=clip).max(dim=1)[0].mean() + lam * F.cross_entropy(score, targets)

    def _distances(self, x, masks=None, lower=None, upper=None):
        """Runs the layer stack; returns the head's outputs (and bounds when a box is given)."""
        has_dropout = any(l.keep_rate != 1.0 for l in self.fc_dist)
        use_masks = has_dropout and self.training and torch.is_grad_enabled()
        if use_masks and masks is None:
            masks = self.draw_masks(x.size(0), x.device)
        x = x.reshape(x.size(0), -1)
        mask_in = None
        for k, layer in enumerate(self.fc_dist):
            mask_out = masks[k] if (use_masks and k < len(masks)) else None
            x, lower, upper = layer(x, lower, upper, mask_in=mask_in, mask_out=mask_out,
                                    sort_eval=has_dropout and not use_masks)
            mask_in = mask_out
        if lower is None:
            return x
        return x, lower, upper

    def _scores(self, x, lower, upper, targets, eps):
        lo = x - eps if lower is None else lower
        hi = x + eps if upper is None else upper
        # distances -> scores: negate, so the roles of the bounds swap
        score, score_lo, score_hi = -x, -hi, -lo
        margin = score_hi - torch.gather(score_lo, 1, targets.view(-1, 1))
        margin = margin.scatter(1, targets.view(-1, 1), 0)
        return score * self.scalar, margin / (2 * eps)

    def forward(self, x=None, targets=None, eps=0, up=None, down=None, masks=None):
        x = x.reshape(x.size(0), -1)
        lower = upper = None
        if up is not None and down is not None and self._certifying():
            up, down = (torch.as_tensor(z, device=x.device, dtype=x.dtype) for z in (up, down))
            lower = torch.maximum(x - eps, down.reshape(1, -1) if down.dim() else down)
            upper = torch.minimum(x + eps, up.reshape(1, -1) if up.dim() else up)
        out = self._distances(x, masks, lower, upper)
        if lower is not None:
            x, lower, upper = out
        else:
            x = out
        if targets is None:
            return -x * self.scalar
        return self._scores(x, lower, upper, targets, eps)


@torch.no_grad()
def update_running_means(model, batches, process_group=None):
    """Re-estimates every mean-shift layer's running mean before certification, as the
    reference's `update_bn` does (main.py:184-202): one pass over `batches` (an iterable of input
    tensors) in training mode at p = inf with momentum 1 / (k + 1) for the k-th batch, i.e. a
    plain average of the batch means, then the mean over ranks.  Layer p values, momenta and the
    training flag are restored."""
    from .dist import all_reduce_mean_
    shifts = [m for m in model.modules() if isinstance(m, MeanShiftDropout)]
    layers = [m for m in model.modules() if isinstance(m, NormDist)]
    saved_p = [l.p for l in layers]
    saved_momentum = [m.momentum for m in shifts]
    was_training = model.training
    model.train()
    for l in layers:
        l.p = float("inf")
    try:
        for k, x in enumerate(batches):
            for m in shifts:
                m.momentum = 1.0 / (k + 1)
            model(x)
        for m in shifts:
            all_reduce_mean_(m.running_mean, process_group)
    finally:
        for m, mom in zip(shifts, saved_momentum):
            m.momentum = mom
        for l, p_val in zip(layers, saved_p):
            l.p = p_val
        model.train(was_training)
