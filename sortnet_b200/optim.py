"""Flat-buffer training state: parameters, gradients and AdamW moments in four flat fp32 buffers.

Why: (1) the data-parallel gradient exchange becomes ONE all-reduce of one buffer instead of one
per parameter; (2) the optimiser is one fused kernel (`snb_adamw_step`, 28 bytes of HBM traffic
per parameter); (3) the backward kernels write `grad_weight` straight into their slice of the
flat gradient buffer, so no gradient is copied or accumulated by autograd.

The reference uses torch.optim.AdamW on ordinary parameters behind DistributedDataParallel
(main.py:402,429-432); parameter names, shapes and values are unchanged here (each parameter
becomes a view into the flat buffer), so state_dicts stay interchangeable.
"""
import torch
import torch.distributed as dist

from . import _lib
from . import norm_dist_cuda as _C


def _pad4(n):
    return (n + 3) // 4 * 4


class FlatAdamW:
    """AdamW over all parameters of `module` held in flat buffers.

    After construction every parameter's `.data` is a view into `self.flat_param` and every
    parameter carries `grad_sink`, a view into `self.flat_grad`: the operators of
    `sortnet_b200.ops` write the weight gradient there during backward and hand `None` to autograd
    (see ops._dist_backward); parameters of other modules get ordinary `.grad` tensors, which
    `gather_grads()` copies into the flat buffer.  One weight-decay value for all parameters
    (the reference uses 0 for every norm-distance weight).
    """

    def __init__(self, module, lr=0.02, betas=(0.9, 0.99), eps=1e-10, weight_decay=0.0, process_group=None):
        self.params = [p for p in module.parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters")
        dev = self.params[0].device
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.step_count = 0
        offsets, total = [], 0
        for p in self.params:
            offsets.append(total)
            total += _pad4(p.numel())          # every slice starts 16-byte aligned
        self.numel = total
        self.flat_param = torch.zeros(total, device=dev, dtype=torch.float32)
        self.flat_grad = torch.zeros(total, device=dev, dtype=torch.float32)
        self.exp_avg = torch.zeros(total, device=dev, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(total, device=dev, dtype=torch.float32)
        self._slices = []
        for p, off in zip(self.params, offsets):
            view = self.flat_param[off:off + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view
            sink = self.flat_grad[off:off + p.numel()].view_as(p)
            p.grad_sink = sink
            self._slices.append((p, sink))

    def zero_grad(self):
        """Only autograd-owned gradients need clearing; sinks are overwritten by the backward."""
        for p in self.params:
            p.grad = None

    def gather_grads(self):
        """Copies gradients that autograd produced itself (parameters whose operator does not
        write into the sink) into the flat buffer."""
        for p, sink in self._slices:
            if p.grad is not None:
                sink.copy_(p.grad)
                p.grad = None

    def all_reduce(self, async_op=False):
        """Sums the flat gradient over ranks (one collective); the mean is taken inside step()."""
        if self.world == 1:
            return None
        return dist.all_reduce(self.flat_grad, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)

    def step(self):
        self.step_count += 1
        dev = self.flat_param.device
        with torch.cuda.device(dev):
            rc = _lib.load().snb_adamw_step(
                self.flat_param.data_ptr(), self.flat_grad.data_ptr(), self.exp_avg.data_ptr(),
                self.exp_avg_sq.data_ptr(), self.numel, float(self.lr), float(self.betas[0]),
                float(self.betas[1]), float(self.eps), float(self.weight_decay), self.step_count,
                1.0 / self.world, torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(rc, "adamw_step")
        _C.launch_count += 1
