"""Data-parallel gradient exchange: one process per GPU, batch sharded, weights replicated.

The reference wraps its model in torch DistributedDataParallel (main.py:402), i.e. a bucketed
all-reduce(mean) of every parameter gradient per step.  Here each parameter's gradient is
all-reduced as soon as autograd has finished accumulating it (a post-accumulate hook), on
NCCL's own stream, so the exchange of layer k overlaps the backward kernels of layers
k-1 ... 1; the wide layers' gradients are 60-400 MB each, large enough to run at NVLink
bandwidth without bucketing.  `finish()` waits for the outstanding reductions and turns the
sums into means.  Ranks only ever touch their own memory; NCCL does the transport.
"""
import torch
import torch.distributed as dist


class GradientAllReduce:
    def __init__(self, params, process_group=None):
        self.params = [p for p in params if p.requires_grad]
        if any(getattr(p, "grad_sink", None) is not None for p in self.params):
            # optim.FlatAdamW has taken these parameters over: their gradients are written into its flat
            # buffer and never reach .grad, so the hooks below would never fire
            raise ValueError("parameters managed by FlatAdamW exchange their gradients through it "
                             "(FlatAdamW.all_reduce or its peer-memory step), not through GradientAllReduce")
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self._pending = []
        self._handles = []
        if self.world > 1:
            for p in self.params:
                self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))

    def _on_grad(self, p):
        work = dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._pending.append((work, p))

    def finish(self):
        """Call after backward, before the optimizer step."""
        for work, p in self._pending:
            work.wait()
            p.grad.div_(self.world)
        self._pending.clear()

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles.clear()


def broadcast_parameters(module, src=0, process_group=None):
    """Makes every rank start from rank `src`'s parameters and buffers."""
    if not dist.is_initialized() or dist.get_world_size(process_group) == 1:
        return
    for t in list(module.parameters()) + list(module.buffers()):
        dist.broadcast(t.data, src=src, group=process_group)


def all_reduce_mean_(tensor, process_group=None):
    """In-place mean over ranks (used for the running means before certification, main.py:197-199)."""
    if dist.is_initialized() and dist.get_world_size(process_group) > 1:
        dist.all_reduce(tensor, group=process_group)
        tensor.div_(dist.get_world_size(process_group))
    return tensor
