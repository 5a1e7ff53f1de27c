"""A CPU stand-in for the reference's `norm_dist_cuda` extension, built on the oracle.

TEST INFRASTRUCTURE ONLY.  With `install()` the reference's unmodified Python code
(core/norm_dist.py, core/models/*, ell_inf_models.py) imports and runs on CPU tensors; it is
used to generate model-level fixtures and never by the product.  Names and argument order
follow core/cuda/norm_dist.cpp:294-318; only G = 1, HW = 1 is handled.
"""
import sys
import types

import numpy as np
import torch

import oracle as _o


def _np(t):
    return t.detach().cpu().numpy()


def _sq(t):
    return _np(t).reshape(t.shape[0], t.shape[1])


def _idx(t):
    return None if t is None else _np(t).reshape(t.shape[0], t.shape[2])


def _put(dst, arr):
    dst.copy_(torch.from_numpy(np.ascontiguousarray(arr)).reshape(dst.shape).to(dst.dtype))


def inf_dist_forward(x, w, out, pos, G, ci=None, co=None):
    y, p = _o.inf_dist_forward(_sq(x), _np(w), _idx(ci), _idx(co))
    _put(out, y)
    _put(pos, p)


def inf_dist_forward_nograd(x, w, out, G):
    y, _ = _o.inf_dist_forward(_sq(x), _np(w), want_pos=False)
    _put(out, y)


def inf_dist_backward_input(g, pos, gx, G):
    a, _ = _o.inf_dist_backward(_sq(g), _sq(pos), gx.shape[1], (1, 1), want_gw=False)
    _put(gx, a)


def inf_dist_backward_input_weight(g, pos, gx, gw, G, ci=None, co=None):
    a, b = _o.inf_dist_backward(_sq(g), _sq(pos), gx.shape[1], tuple(gw.shape), _idx(ci), _idx(co))
    _put(gx, a)
    _put(gw, b)


def norm_dist_forward(x, w, out, G, p, ci=None, co=None):
    _put(out, _o.norm_dist_forward(_sq(x), _np(w), p, _idx(ci), _idx(co)))


def norm_dist_backward_input(g, x, w, y, gx, G, p, ci=None, co=None):
    a, _ = _o.norm_dist_backward(_sq(g), _sq(x), _np(w), _sq(y), p, _idx(ci), _idx(co), want_gw=False)
    _put(gx, a)


def norm_dist_backward_input_weight(g, x, w, y, gx, gw, G, p, ci=None, co=None):
    a, b = _o.norm_dist_backward(_sq(g), _sq(x), _np(w), _sq(y), p, _idx(ci), _idx(co))
    _put(gx, a)
    _put(gw, b)


def bound_inf_dist_forward_nograd(xl, xu, w, yl, yu, G):
    a, b, _, _ = _o.bound_inf_dist_forward(_sq(xl), _sq(xu), _np(w), want_pos=False)
    _put(yl, a)
    _put(yu, b)


def bound_inf_dist_forward(xl, xu, w, yl, yu, pl, pu, G):
    a, b, c, d = _o.bound_inf_dist_forward(_sq(xl), _sq(xu), _np(w))
    _put(yl, a)
    _put(yu, b)
    _put(pl, c)
    _put(pu, d)


def bound_inf_dist_backward_input(gl, gu, pl, pu, gxl, gxu, G):
    a, b, _ = _o.bound_inf_dist_backward(_sq(gl), _sq(gu), _sq(pl), _sq(pu), gxl.shape[1], want_gw=False)
    _put(gxl, a)
    _put(gxu, b)


def bound_inf_dist_backward_input_weight(gl, gu, pl, pu, gxl, gxu, gw, G):
    a, b, c = _o.bound_inf_dist_backward(_sq(gl), _sq(gu), _sq(pl), _sq(pu), gxl.shape[1])
    _put(gxl, a)
    _put(gxu, b)
    _put(gw, c)


def install():
    mod = types.ModuleType("norm_dist_cuda")
    for name, fn in list(globals().items()):
        if callable(fn) and not name.startswith("_") and name not in ("install",):
            setattr(mod, name, fn)
    sys.modules["norm_dist_cuda"] = mod
    return mod
