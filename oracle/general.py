"""Grouped / spatial shapes on top of the 2-D CPU oracle.  TEST INFRASTRUCTURE ONLY.

The reference's operators take x [B, G*CIg, HW], w [G*COg, CIg] and produce y [B, G*COg, HW]
(core/norm_dist.py:8-13: `weight.size(1) * group == x.size(1)`, output `B x CO x HW`): group g
of the outputs sees only group g of the input channels and rows g*COg..(g+1)*COg-1 of w, and
every spatial position hw is an independent sample that shares the row's sub-batch (index
arithmetic at core/cuda/inf_dist_cuda.cu:112-123,152-171,203: input offset
((b*G+g)*CIg + c)*HW + hw, weight offset (g*W_COg + co)*W_CIg + ci, mask row (b/32)*G + g).
Each function below slices one (g, hw) problem out, runs the 2-D oracle on it and writes the
result back, so nothing here shares code or layout tricks with the CUDA path it checks.

Masks: ci [S, G, CI'g], co [S, G, CO'g] (int32) or None; w then has full size [G*W_COg, W_CIg].
"""
import numpy as np

from . import (bound_inf_dist_backward, bound_inf_dist_forward, inf_dist_backward,
               inf_dist_forward, norm_dist_backward, norm_dist_forward, sort_backward,
               sort_bound_forward, sort_forward)


def _x4(x, G):
    x = np.asarray(x)
    B, C, HW = x.shape
    assert C % G == 0
    return x.reshape(B, G, C // G, HW)


def _w3(w, G):
    w = np.asarray(w)
    assert w.shape[0] % G == 0
    return w.reshape(G, w.shape[0] // G, w.shape[1])


def _m(m, g):
    return None if m is None else np.ascontiguousarray(np.asarray(m)[:, g])


def _out_per_group(w3, co):
    return co.shape[-1] if co is not None else w3.shape[1]


def inf_dist_forward_g(x, w, G, ci=None, co=None):
    x4, w3 = _x4(x, G), _w3(w, G)
    B, _, _, HW = x4.shape
    COg = _out_per_group(w3, co)
    y = np.empty((B, G, COg, HW), np.float32)
    pos = np.empty((B, G, COg, HW), np.int32)
    for g in range(G):
        for h in range(HW):
            y[:, g, :, h], pos[:, g, :, h] = inf_dist_forward(x4[:, g, :, h], w3[g], _m(ci, g), _m(co, g))
    return y.reshape(B, G * COg, HW), pos.reshape(B, G * COg, HW)


def inf_dist_backward_g(gy, pos, CI, w_shape, G, ci=None, co=None):
    g4, p4 = _x4(gy, G), _x4(pos, G)
    B, _, _, HW = g4.shape
    CIg = CI // G
    gx = np.zeros((B, G, CIg, HW), np.float32)
    gw = np.zeros((G, w_shape[0] // G, w_shape[1]), np.float64)
    for g in range(G):
        for h in range(HW):
            a, b = inf_dist_backward(g4[:, g, :, h], p4[:, g, :, h], CIg, gw.shape[1:], _m(ci, g), _m(co, g))
            gx[:, g, :, h] = a
            gw[g] += b
    return gx.reshape(B, CI, HW), gw.reshape(w_shape).astype(np.float32)


def bound_inf_dist_forward_g(xl, xu, w, G):
    l4, u4, w3 = _x4(xl, G), _x4(xu, G), _w3(w, G)
    B, _, _, HW = l4.shape
    COg = w3.shape[1]
    outs = [np.empty((B, G, COg, HW), t) for t in (np.float32, np.float32, np.int32, np.int32)]
    for g in range(G):
        for h in range(HW):
            r = bound_inf_dist_forward(l4[:, g, :, h], u4[:, g, :, h], w3[g])
            for o, v in zip(outs, r):
                o[:, g, :, h] = v
    return tuple(o.reshape(B, G * COg, HW) for o in outs)


def bound_inf_dist_backward_g(gl, gu, pl, pu, CI, G):
    gl4, gu4, pl4, pu4 = (_x4(a, G) for a in (gl, gu, pl, pu))
    B, _, COg, HW = gl4.shape
    CIg = CI // G
    gxl = np.zeros((B, G, CIg, HW), np.float32)
    gxu = np.zeros((B, G, CIg, HW), np.float32)
    gw = np.zeros((G, COg, CIg), np.float64)
    for g in range(G):
        for h in range(HW):
            a, b, c = bound_inf_dist_backward(gl4[:, g, :, h], gu4[:, g, :, h], pl4[:, g, :, h],
                                              pu4[:, g, :, h], CIg)
            gxl[:, g, :, h], gxu[:, g, :, h] = a, b
            gw[g] += c
    return gxl.reshape(B, CI, HW), gxu.reshape(B, CI, HW), gw.reshape(G * COg, CIg).astype(np.float32)


def norm_dist_forward_g(x, w, p, G, ci=None, co=None):
    x4, w3 = _x4(x, G), _w3(w, G)
    B, _, _, HW = x4.shape
    COg = _out_per_group(w3, co)
    y = np.empty((B, G, COg, HW), np.float64)
    for g in range(G):
        for h in range(HW):
            y[:, g, :, h] = norm_dist_forward(x4[:, g, :, h], w3[g], p, _m(ci, g), _m(co, g))
    return y.reshape(B, G * COg, HW)


def norm_dist_backward_g(gy, x, w, y, p, G, ci=None, co=None):
    g4, x4, y4, w3 = _x4(gy, G), _x4(x, G), _x4(y, G), _w3(w, G)
    B, _, CIg, HW = x4.shape
    gx = np.zeros((B, G, CIg, HW), np.float64)
    gw = np.zeros(w3.shape, np.float64)
    for g in range(G):
        for h in range(HW):
            a, b = norm_dist_backward(g4[:, g, :, h], x4[:, g, :, h], w3[g], y4[:, g, :, h], p,
                                      _m(ci, g), _m(co, g))
            gx[:, g, :, h] = a
            gw[g] += b
    return gx.reshape(B, G * CIg, HW), gw.reshape(np.asarray(w).shape)


def sort_forward_g(x, w, q, K, G):
    x4, w3 = _x4(x, G), _w3(w, G)
    B, _, _, HW = x4.shape
    COg = w3.shape[1]
    y = np.empty((B, G, COg, HW), np.float32)
    pos = np.empty((K, B, G, COg, HW), np.int32)
    for g in range(G):
        for h in range(HW):
            y[:, g, :, h], pos[:, :, g, :, h] = sort_forward(x4[:, g, :, h], w3[g], q, K)
    return y.reshape(B, G * COg, HW), pos.reshape(K, B, G * COg, HW)


def sort_bound_forward_g(xl, xu, w, q, K, G):
    l4, u4, w3 = _x4(xl, G), _x4(xu, G), _w3(w, G)
    B, _, _, HW = l4.shape
    COg = w3.shape[1]
    yl = np.empty((B, G, COg, HW), np.float32)
    yu = np.empty((B, G, COg, HW), np.float32)
    for g in range(G):
        for h in range(HW):
            yl[:, g, :, h], yu[:, g, :, h] = sort_bound_forward(l4[:, g, :, h], u4[:, g, :, h], w3[g], q, K)
    return yl.reshape(B, G * COg, HW), yu.reshape(B, G * COg, HW)


def sort_backward_g(gy, pos, CI, q, K, G):
    g4 = _x4(gy, G)
    B, _, COg, HW = g4.shape
    p5 = np.asarray(pos).reshape(K, B, G, COg, HW)
    CIg = CI // G
    gx = np.zeros((B, G, CIg, HW), np.float32)
    gw = np.zeros((G, COg, CIg), np.float64)
    for g in range(G):
        for h in range(HW):
            a, b = sort_backward(g4[:, g, :, h], p5[:, :, g, :, h], CIg, q, K)
            gx[:, g, :, h] = a
            gw[g] += b
    return gx.reshape(B, CI, HW), gw.reshape(G * COg, CIg).astype(np.float32)
