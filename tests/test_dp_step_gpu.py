"""Two ranks on two GPUs: the fused peer-memory step (reduce-scatter + AdamW + all-gather in one
kernel over NVLink peer pointers) against the NCCL all-reduce + local AdamW path on the same model
and data.  Needs two GPUs; skipped otherwise."""
import copy
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out, overlap=False):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import torch.nn.functional as F
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from sortnet_b200.layers import SortMLPModel
        from sortnet_b200.optim import FlatAdamW
        torch.manual_seed(0)
        a = SortMLPModel(depth=4, width=96, input_dim=(3, 4, 4), num_classes=10, dropout=0.8).to(dev)
        b = copy.deepcopy(a)
        kw = dict(lr=0.02, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.01)
        opt_a = FlatAdamW(a, peer_memory=True, overlap=overlap, **kw)
        opt_b = FlatAdamW(b, peer_memory=False, **kw)
        assert opt_a.peer and opt_a.exp_avg.numel() < opt_b.exp_avg.numel()
        gen = torch.Generator(device=dev).manual_seed(100 + rank)      # different data per rank
        ok = True
        for step in range(3):
            x = torch.rand(64, 3, 4, 4, device=dev, generator=gen)
            t = torch.randint(0, 10, (64,), device=dev, generator=gen)
            masks = a.draw_masks(64, dev)
            a.train()
            logits, margin = a(x, targets=t, eps=0.03, masks=masks)
            loss = margin.clamp(min=0, max=1).max(dim=1)[0].mean() + 0.1 * F.cross_entropy(logits, t)
            opt_a.zero_grad()
            loss.backward()
            opt_a.gather_grads()
            # both optimisers get the very same local gradients (Adam amplifies the run-to-run
            # rounding differences of atomically accumulated gradients where they cancel to ~0)
            opt_b.set_flat_grad(opt_a.flat_grad)
            opt_b.all_reduce()
            opt_b.step()
            if overlap:
                before = [p.detach().clone() for p in a.parameters()]
                opt_a.begin_exchange()
                # work queued between begin and end still sees the old values
                # the shard's update runs on this stream: between two layers of the pass on odd steps
                # (apply_update), at end_exchange() otherwise
                hook = (lambda k: opt_a.start_pulls() if k == 0 else opt_a.apply_update() if k == 1 else None) \
                    if step % 2 else None
                with torch.no_grad():
                    cert = a.certified_margin(x, t, 0.03, torch.ones(1, device=dev), torch.zeros(1, device=dev),
                                              after_layer=hook)
                ok = ok and all(torch.equal(p, q) for p, q in zip(a.parameters(), before)) and bool(cert >= 0)
                opt_a.end_exchange()
            else:
                opt_a.step()
            torch.cuda.synchronize()
            for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
                good = bool((p - q).abs().max() <= 1e-5 * max(q.abs().max().item(), 1.0))
                if not good:
                    print('rank', rank, 'step', step, n, float((p - q).abs().max()), flush=True)
                ok = ok and good
        # replicas identical across ranks
        flat = opt_a.flat_param.clone()
        other = flat.clone()
        dist.broadcast(other, src=0)
        ok = ok and bool(torch.equal(flat, other))
        out[rank] = ok
    finally:
        dist.destroy_process_group()


def test_peer_memory_step_matches_all_reduce_path():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
        assert dict(out) == {0: True, 1: True}


def test_copy_exchange_beside_other_work_matches_all_reduce_path():
    """overlap=True: reduce-scatter and all-gather as device-to-device copies on a side stream, the
    parameters double-buffered; same values as the all-reduce path after every step."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), out, True), nprocs=2, join=True)
        assert dict(out) == {0: True, 1: True}
