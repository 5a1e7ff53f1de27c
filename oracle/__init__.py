"""CPU oracle for the norm-distance neuron path (TEST INFRASTRUCTURE ONLY).

numpy front-end of norm_dist_oracle.c plus a numpy restatement of the mean-shift module.
Only the tests, the smoke check and the benchmark's CPU-baseline leg import this package;
the product (`sortnet_b200`) never does and has no CPU fallback.

Parity pin: the reference ships no golden vectors or known-answer tests.  The restatement
is pinned against outputs of the reference's own pure-PyTorch branches
(core/norm_dist.py:180-185, 194-213, 250-259; bound_basic_module.py:123-157) and their
autograd gradients, stored under tests/golden/ by tests/golden/make_golden.py.  Items the
PyTorch branches do not define (argmax words on exact ties, the 1e-10 floors, posL =
0xffffffff) follow the CUDA sources cited in norm_dist_oracle.c and are additionally
compared on the GPU with the reference extension when oracle/_ref holds a build of it.
"""
import ctypes
import os

import numpy as np

from . import build as _build

_lib = None

_F = ctypes.POINTER(ctypes.c_float)
_D = ctypes.POINTER(ctypes.c_double)
_I = ctypes.POINTER(ctypes.c_int32)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build())
    return _lib


def _f(a):
    return None if a is None else a.ctypes.data_as(_F)


def _d(a):
    return None if a is None else a.ctypes.data_as(_D)


def _i(a):
    return None if a is None else a.ctypes.data_as(_I)


def _c32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _ci32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def inf_dist_forward(x, w, ci=None, co=None, want_pos=True):
    """x [B, CI'], w [W_CO, W_CI], ci [S, CI'] / co [S, CO'] int32 or None -> y, pos."""
    x, w, ci, co = _c32(x), _c32(w), _ci32(ci), _ci32(co)
    B, CI = x.shape
    CO = co.shape[-1] if co is not None else w.shape[0]
    y = np.empty((B, CO), np.float32)
    pos = np.empty((B, CO), np.int32) if want_pos else None
    lib().oracle_inf_dist_forward(_f(x), _f(w), B, CO, CI, _f(y), _i(pos), _i(ci), _i(co),
                                  w.shape[1])
    return y, pos


def inf_dist_backward(g, pos, CI, w_shape, ci=None, co=None, want_gw=True):
    g, pos, ci, co = _c32(g), _ci32(pos), _ci32(ci), _ci32(co)
    B, CO = g.shape
    gx = np.empty((B, CI), np.float32)
    gw = np.empty(w_shape, np.float32) if want_gw else None
    lib().oracle_inf_dist_backward(_f(g), _i(pos), B, CO, CI, _f(gx), _f(gw), _i(ci), _i(co),
                                   w_shape[0], w_shape[1])
    return gx, gw


def bound_inf_dist_forward(xl, xu, w, want_pos=True):
    xl, xu, w = _c32(xl), _c32(xu), _c32(w)
    B, CI = xl.shape
    CO = w.shape[0]
    yl = np.empty((B, CO), np.float32)
    yu = np.empty((B, CO), np.float32)
    pl = np.empty((B, CO), np.int32) if want_pos else None
    pu = np.empty((B, CO), np.int32) if want_pos else None
    lib().oracle_bound_inf_dist_forward(_f(xl), _f(xu), _f(w), B, CO, CI, _f(yl), _f(yu),
                                        _i(pl), _i(pu))
    return yl, yu, pl, pu


def bound_inf_dist_backward(gl, gu, pl, pu, CI, want_gw=True):
    gl, gu, pl, pu = _c32(gl), _c32(gu), _ci32(pl), _ci32(pu)
    B, CO = gl.shape
    gxl = np.empty((B, CI), np.float32)
    gxu = np.empty((B, CI), np.float32)
    gw = np.empty((CO, CI), np.float32) if want_gw else None
    lib().oracle_bound_inf_dist_backward(_f(gl), _f(gu), _i(pl), _i(pu), B, CO, CI,
                                         _f(gxl), _f(gxu), _f(gw))
    return gxl, gxu, gw


def norm_dist_forward(x, w, p, ci=None, co=None):
    """Exact-math (float64) l-p distance of the fp32 differences."""
    x, w, ci, co = _c32(x), _c32(w), _ci32(ci), _ci32(co)
    B, CI = x.shape
    CO = co.shape[-1] if co is not None else w.shape[0]
    y = np.empty((B, CO), np.float64)
    lib().oracle_norm_dist_forward(_f(x), _f(w), B, CO, CI, ctypes.c_double(p), _d(y),
                                   _i(ci), _i(co), w.shape[1])
    return y


def norm_dist_backward(g, x, w, y, p, ci=None, co=None, want_gw=True):
    g, x, w, y, ci, co = _c32(g), _c32(x), _c32(w), _c32(y), _ci32(ci), _ci32(co)
    B, CI = x.shape
    CO = g.shape[1]
    gx = np.empty((B, CI), np.float64)
    gw = np.empty(w.shape, np.float64) if want_gw else None
    lib().oracle_norm_dist_backward(_f(g), _f(x), _f(w), _f(y), B, CO, CI, ctypes.c_double(p),
                                    _d(gx), _d(gw), _i(ci), _i(co), w.shape[0], w.shape[1])
    return gx, gw


SUB_BATCH = 32


def mean_shift_train(x, index, out_channels):
    """Training-mode mean-shift (bound_basic_module.py:123-157), float64 numpy.

    x [B, C'] compact activations, index [S, C'] kept channels per 32-row sub-batch or None.
    Returns (y, mean[out_channels]).  mean[c] = sum of x over rows whose sub-batch kept c,
    divided by (1e-10 + rows in those sub-batches); never-kept channels get 0.
    """
    x = np.asarray(x, np.float64)
    B = x.shape[0]
    if index is None:
        mean = x.mean(axis=0)
        return x - mean[None, :], mean
    S = index.shape[0]
    ssum = np.zeros(out_channels)
    cnt = np.full(out_channels, 1e-10)
    for s in range(S):
        rows = x[s * SUB_BATCH:min(B, (s + 1) * SUB_BATCH)]
        np.add.at(ssum, index[s], rows.sum(axis=0))
        np.add.at(cnt, index[s], float(rows.shape[0]))
    mean = ssum / cnt
    y = np.empty_like(x)
    for s in range(S):
        sl = slice(s * SUB_BATCH, min(B, (s + 1) * SUB_BATCH))
        y[sl] = x[sl] - mean[index[s]][None, :]
    return y, mean


def mean_shift_train_backward(gy, index, out_channels):
    """Gradient of mean_shift_train w.r.t. x (the mean is differentiated through)."""
    gy = np.asarray(gy, np.float64)
    B = gy.shape[0]
    if index is None:
        return gy - gy.mean(axis=0)[None, :]
    S = index.shape[0]
    gsum = np.zeros(out_channels)
    cnt = np.full(out_channels, 1e-10)
    for s in range(S):
        rows = gy[s * SUB_BATCH:min(B, (s + 1) * SUB_BATCH)]
        np.add.at(gsum, index[s], rows.sum(axis=0))
        np.add.at(cnt, index[s], float(rows.shape[0]))
    gmean = gsum / cnt
    gx = np.empty_like(gy)
    for s in range(S):
        sl = slice(s * SUB_BATCH, min(B, (s + 1) * SUB_BATCH))
        gx[sl] = gy[sl] - gmean[index[s]][None, :]
    return gx


def sort_forward(x, w, q, K, want_pos=True):
    """Sort neuron: y [B, CO], pos [K, B, CO] (rank 0 = largest) or None."""
    x, w = _c32(x), _c32(w)
    B, CI = x.shape
    CO = w.shape[0]
    y = np.empty((B, CO), np.float32)
    pos = np.empty((K, B, CO), np.int32) if want_pos else None
    lib().oracle_sort_forward(_f(x), _f(w), B, CO, CI, ctypes.c_float(q), K, _f(y), _i(pos))
    return y, pos


def sort_bound_forward(xl, xu, w, q, K):
    xl, xu, w = _c32(xl), _c32(xu), _c32(w)
    B, CI = xl.shape
    CO = w.shape[0]
    yl = np.empty((B, CO), np.float32)
    yu = np.empty((B, CO), np.float32)
    lib().oracle_sort_bound_forward(_f(xl), _f(xu), _f(w), B, CO, CI, ctypes.c_float(q), K, _f(yl), _f(yu))
    return yl, yu


def sort_backward(g, pos, CI, q, K, want_gw=True):
    g, pos = _c32(g), _ci32(pos)
    B, CO = g.shape
    gx = np.empty((B, CI), np.float32)
    gw = np.empty((CO, CI), np.float32) if want_gw else None
    lib().oracle_sort_backward(_f(g), _i(pos), B, CO, CI, ctypes.c_float(q), K, _f(gx), _f(gw))
    return gx, gw
