"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def col3(a, dtype=None):
    """[B, C] numpy -> [B, C, 1] CUDA tensor (the layout the operators take)."""
    return dev(a, dtype).unsqueeze(-1).contiguous()


def idx3(a):
    """[S, C] numpy int -> [S, 1, C] int32 CUDA tensor."""
    return None if a is None else dev(a, torch.int32).unsqueeze(1).contiguous()


def host(t):
    return t.detach().squeeze(-1).cpu().numpy()


def rel(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)


def make_masks(rng, B, C_full, keep):
    """Index lists in the reference's format: one count for all sub-batches, a random sorted
    subset per 32-row sub-batch (core/models/norm_dist.py:14-17)."""
    S = (B + 31) // 32
    count = int((rng.random(C_full) < keep).sum())
    count = max(count, 1)
    out = np.stack([np.sort(rng.permutation(C_full)[:count]) for _ in range(S)]).astype(np.int32)
    return out
