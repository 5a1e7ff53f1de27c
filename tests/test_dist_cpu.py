"""World-size-2 gloo test (CPU) of the data-parallel gradient exchange: every rank ends with the
mean of the per-rank gradients, i.e. the gradient of the concatenated batch."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sortnet_b200.dist import GradientAllReduce, all_reduce_mean_, broadcast_parameters
    torch.manual_seed(rank)                       # ranks start different ...
    model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
    broadcast_parameters(model)                   # ... and are made identical
    sync = GradientAllReduce(model.parameters())
    g = torch.Generator().manual_seed(7)
    x_all = torch.randn(8, 6, generator=g)
    y_all = torch.randn(8, 3, generator=g)
    shard = slice(rank * 4, rank * 4 + 4)
    for _ in range(2):                            # twice: hooks must survive zero_grad
        model.zero_grad(set_to_none=True)
        loss = ((model(x_all[shard]) - y_all[shard]) ** 2).mean()
        loss.backward()
        sync.finish()
    grads = [p.grad.clone() for p in model.parameters()]
    # single-process reference on the whole batch
    ref = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
    ref.load_state_dict(model.state_dict())
    ((ref(x_all) - y_all) ** 2).mean().backward()
    ok = all(torch.allclose(a, p.grad, atol=1e-6) for a, p in zip(grads, ref.parameters()))
    rm = torch.full((4,), float(rank))
    all_reduce_mean_(rm)
    ok = ok and torch.allclose(rm, torch.full((4,), 0.5))
    out[rank] = bool(ok)
    dist.destroy_process_group()


def test_gradient_all_reduce_world2():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_single_process_is_a_no_op():
    sys.path.insert(0, ROOT)
    from sortnet_b200.dist import GradientAllReduce
    lin = torch.nn.Linear(3, 2)
    sync = GradientAllReduce(lin.parameters())
    lin(torch.randn(4, 3)).sum().backward()
    before = lin.weight.grad.clone()
    sync.finish()
    assert torch.equal(before, lin.weight.grad)
