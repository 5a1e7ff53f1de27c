"""Tensor-level entry points with the names and argument order of the reference's
`norm_dist_cuda` extension module (core/cuda/norm_dist.cpp:294-318).

Every function writes into caller-allocated tensors and returns None, like the reference.
Differences: work is enqueued on PyTorch's *current* stream of the tensors' device (the
reference always uses the legacy default stream, forward.cuh:31), the device of the inputs is
made current for the call, and shapes / dtypes that the reference leaves unchecked raise
RuntimeError instead of corrupting memory.  The *values* of index lists are not looked at on the
normal path (the kernels read w through them unchecked, like the reference's); with
SORTNET_B200_DEBUG=1 in the environment every index list is validated on the device before use
(`snb_check_index_lists`: one small kernel and a stream synchronisation per list) and an entry
outside [0, channels) raises.

`install()` registers this module as `norm_dist_cuda` in sys.modules so that the reference's
unmodified `core/norm_dist.py` (`import norm_dist_cuda as _C`) runs on these kernels.
"""
import ctypes
import os
import sys

import torch

from . import _lib

_SUB_BATCH = 32
DEBUG_INDEX_CHECKS = os.environ.get("SORTNET_B200_DEBUG", "0") == "1"


def _check(t, name, dtype=torch.float32):
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)
    if t.dtype != dtype:
        raise RuntimeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))


def _check_opt_index(t, name, n_sub, width, groups=1, channels=None):
    """Index lists are [sub-batches, groups, kept channels per group]; `width` is the total over
    groups; `channels` (when the caller knows it) is the size of the axis of w the entries index,
    per group, used by the optional value check."""
    if t is None:
        return
    _check(t, name, torch.int32)
    if t.dim() != 3 or t.size(0) != n_sub or t.size(1) != groups or t.size(2) * groups != width:
        raise RuntimeError("%s must have shape [%d, %d, %d], got %s"
                           % (name, n_sub, groups, width // max(groups, 1), tuple(t.shape)))
    if DEBUG_INDEX_CHECKS and channels is not None:
        check_index_lists(t, channels, name)


def check_index_lists(index, channels, name="index"):
    """Validates the values of an index tensor [S, G, count] on its device: raises when an entry lies
    outside [0, channels); returns True when every list is strictly ascending.  Synchronises."""
    import ctypes
    _check(index, name, torch.int32)
    flags = ctypes.c_int(0)
    with torch.cuda.device(index.device):
        rc = _lib.load().snb_check_index_lists(index.data_ptr(), index.size(0) * index.size(1), index.size(2),
                                               int(channels), ctypes.byref(flags),
                                               torch.cuda.current_stream(index.device).cuda_stream)
    if rc == 8:
        raise RuntimeError("%s holds an entry outside [0, %d)" % (name, channels))
    _lib.check(rc, "check_index_lists")
    return not (flags.value & 2)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _dims(x, out):
    return x.size(0), out.size(1), x.size(1), x.size(2)


# Kernels launched by each C entry point (memsets are not counted).
_KERNELS = {
    "snb_inf_dist_forward": 2, "snb_inf_dist_forward_ws": 2, "snb_inf_dist_forward_sorted_ws": 3, "snb_inf_dist_forward_nograd": 1, "snb_inf_dist_backward_input": 1,
    "snb_inf_dist_backward_input_weight": 1, "snb_norm_dist_forward": 1, "snb_norm_dist_forward_ws": 2, "snb_norm_dist_backward_input": 1,
    "snb_norm_dist_backward_input_weight": 1, "snb_bound_inf_dist_forward_nograd": 1,
    "snb_bound_inf_dist_forward": 1, "snb_bound_inf_dist_backward_input": 1,
    "snb_bound_inf_dist_backward_input_weight": 1, "snb_mean_shift_stats": 1, "snb_mean_shift_apply": 1, "snb_sample_mask": 1, "snb_sample_mask_batch": 1,
    "snb_sort_neuron_forward_nograd": 1, "snb_sort_neuron_forward": 1, "snb_bound_sort_neuron_forward": 1,
    "snb_sort_neuron_backward_input": 1, "snb_sort_neuron_backward_input_weight": 1,
}

launch_count = 0          # kernels launched through this module since import / reset_counters()
_timeline = None          # when profiling: list of (entry point, work tag, start event, end event)


def reset_counters():
    global launch_count
    launch_count = 0


def start_profile():
    """Record a CUDA event pair around every entry-point call (on the stream it launches on)."""
    global _timeline
    _timeline = []


def stop_profile():
    """Returns {(entry point, work tag): [milliseconds per call]}; synchronises the device."""
    global _timeline
    tl, _timeline = _timeline or [], None
    torch.cuda.synchronize()
    out = {}
    for name, tag, e0, e1 in tl:
        out.setdefault((name, tag), []).append(e0.elapsed_time(e1))
    return out


def _call(dev, ref_tensor, entry, tag, *args):
    """Runs C entry point `entry` with `dev` current, on the current stream of that device."""
    global launch_count
    lib = _lib.load()
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev)
        if _timeline is not None:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record(stream)
        rc = getattr(lib, entry)(*args, stream.cuda_stream)
        if _timeline is not None:
            e1.record(stream)
            _timeline.append((entry, tag, e0, e1))
    _lib.check(rc, entry[4:])
    launch_count += _KERNELS[entry]
    if entry in ("snb_norm_dist_forward", "snb_norm_dist_forward_ws") and args[8] > 10.0:
        launch_count += 1      # the l-inf pass that supplies the normaliser


def _same_device(*ts):
    dev = ts[0].device
    for t in ts[1:]:
        if t is not None and t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
    return dev


def inf_dist_forward(input, weight, output, pos, G, w_index_ci=None, w_index_co=None):
    """core/cuda/norm_dist.cpp:131-147."""
    _check(input, "input"); _check(weight, "weight"); _check(output, "output")
    _check(pos, "pos", torch.int32)
    B, CO, CI, HW = _dims(input, output)
    S = (B + _SUB_BATCH - 1) // _SUB_BATCH
    _check_opt_index(w_index_ci, "w_index_ci", S, CI, G, weight.size(1))
    _check_opt_index(w_index_co, "w_index_co", S, CO, G, weight.size(0) // G)
    if output.size(0) != B or pos.shape != output.shape:
        raise RuntimeError("output / pos shape mismatch")
    dev = _same_device(input, weight, output, pos, w_index_ci, w_index_co)
    # scratch for the k-split merge of (value, position) pairs: 8 bytes per output, taken from
    # PyTorch's caching allocator (stream-ordered, no device synchronisation)
    ws = torch.empty(B * CO, dtype=torch.int64, device=dev)
    _call(dev, input, "snb_inf_dist_forward_ws", (B, CO, CI),
          _ptr(input), _ptr(weight), B, CO, CI, G, HW, _ptr(output), _ptr(pos), _ptr(w_index_ci),
          _ptr(w_index_co), weight.size(0), weight.size(1) * G, ws.data_ptr(), ws.numel() * 8)


def inf_dist_forward_sorted(input, weight, output, pos, w_index_ci=None, w_index_co=None):
    """inf_dist_forward (G = 1) for index lists in ascending order, as sample_mask and the reference's
    sampler (core/models/norm_dist.py:14-17) produce them: same results, W read along whole rows
    (snb_inf_dist_forward_sorted_ws).  No counterpart in the reference's extension."""
    _check(input, "input"); _check(weight, "weight"); _check(output, "output")
    _check(pos, "pos", torch.int32)
    B, CO, CI, HW = _dims(input, output)
    S = (B + _SUB_BATCH - 1) // _SUB_BATCH
    _check_opt_index(w_index_ci, "w_index_ci", S, CI, 1, weight.size(1))
    _check_opt_index(w_index_co, "w_index_co", S, CO, 1, weight.size(0))
    if output.size(0) != B or pos.shape != output.shape:
        raise RuntimeError("output / pos shape mismatch")
    dev = _same_device(input, weight, output, pos, w_index_ci, w_index_co)
    if DEBUG_INDEX_CHECKS:        # the promise itself: every list strictly ascending
        for t, name, channels in ((w_index_ci, "w_index_ci", weight.size(1)), (w_index_co, "w_index_co", weight.size(0))):
            if t is not None and not check_index_lists(t, channels, name):
                raise RuntimeError("%s is not in ascending order: use inf_dist_forward" % name)
    nbytes = _lib.load().snb_inf_dist_forward_sorted_workspace_bytes(B, CO, weight.size(1))
    ws = torch.empty((nbytes + 7) // 8, dtype=torch.int64, device=dev)
    _call(dev, input, "snb_inf_dist_forward_sorted_ws", (B, CO, CI),
          _ptr(input), _ptr(weight), B, CO, CI, 1, HW, _ptr(output), _ptr(pos), _ptr(w_index_ci),
          _ptr(w_index_co), weight.size(0), weight.size(1), ws.data_ptr(), ws.numel() * 8)


def inf_dist_forward_nograd(input, weight, output, G):
    """core/cuda/norm_dist.cpp:149-156."""
    _check(input, "input"); _check(weight, "weight"); _check(output, "output")
    B, CO, CI, HW = _dims(input, output)
    if weight.size(0) != CO or weight.size(1) * G != CI or output.size(0) != B:
        raise RuntimeError("shape mismatch between input, weight and output")
    dev = _same_device(input, weight, output)
    _call(dev, input, "snb_inf_dist_forward_nograd", (B, CO, CI),
          _ptr(input), _ptr(weight), B, CO, CI, G, HW, _ptr(output))


def inf_dist_backward_input(grad_output, pos, grad_input, G):
    """core/cuda/norm_dist.cpp:158-165."""
    _check(grad_output, "grad_output"); _check(pos, "pos", torch.int32); _check(grad_input, "grad_input")
    B, CO, CI, HW = grad_output.size(0), grad_output.size(1), grad_input.size(1), grad_input.size(2)
    if pos.shape != grad_output.shape or grad_input.size(0) != B:
        raise RuntimeError("shape mismatch between grad_output, pos and grad_input")
    dev = _same_device(grad_output, pos, grad_input)
    _call(dev, grad_output, "snb_inf_dist_backward_input", (B, CO, CI),
          _ptr(grad_output), _ptr(pos), B, CO, CI, G, HW, _ptr(grad_input))


def inf_dist_backward_input_weight(grad_output, pos, grad_input, grad_weight, G,
                                   w_index_ci=None, w_index_co=None):
    """core/cuda/norm_dist.cpp:167-184."""
    _check(grad_output, "grad_output"); _check(pos, "pos", torch.int32)
    _check(grad_input, "grad_input"); _check(grad_weight, "grad_weight")
    B, CO, CI, HW = grad_output.size(0), grad_output.size(1), grad_input.size(1), grad_output.size(2)
    S = (B + _SUB_BATCH - 1) // _SUB_BATCH
    _check_opt_index(w_index_ci, "w_index_ci", S, CI, G, grad_weight.size(1))
    _check_opt_index(w_index_co, "w_index_co", S, CO, G, grad_weight.size(0) // G)
    if pos.shape != grad_output.shape or grad_input.size(0) != B:
        raise RuntimeError("shape mismatch between grad_output, pos and grad_input")
    dev = _same_device(grad_output, pos, grad_input, grad_weight, w_index_ci, w_index_co)
    _call(dev, grad_output, "snb_inf_dist_backward_input_weight", (B, CO, CI),
          _ptr(grad_output), _ptr(pos), B, CO, CI, G, HW, _ptr(grad_input), _ptr(grad_weight),
          _ptr(w_index_ci), _ptr(w_index_co), grad_weight.size(0), grad_weight.size(1) * G)


def _lp_common(input, weight, output, w_index_ci, w_index_co, G):
    B, CO, CI, HW = _dims(input, output)
    S = (B + _SUB_BATCH - 1) // _SUB_BATCH
    _check_opt_index(w_index_ci, "w_index_ci", S, CI, G, weight.size(1))
    _check_opt_index(w_index_co, "w_index_co", S, CO, G, weight.size(0) // G)
    return B, CO, CI, HW


def norm_dist_forward(input, weight, output, G, p, w_index_ci=None, w_index_co=None):
    """core/cuda/norm_dist.cpp:43-65 (p <= 10 plain sum, p > 10 max-normalised)."""
    _check(input, "input"); _check(weight, "weight"); _check(output, "output")
    B, CO, CI, HW = _lp_common(input, weight, output, w_index_ci, w_index_co, G)
    dev = _same_device(input, weight, output, w_index_ci, w_index_co)
    # p > 10: scratch for the maxima (4 bytes per output) from PyTorch's caching allocator, so that
    # the kernel may share output tiles between thread blocks
    ws = torch.empty(B * CO * HW if p > 10 else 0, dtype=torch.float32, device=dev)
    _call(dev, input, "snb_norm_dist_forward_ws", (B, CO, CI),
          _ptr(input), _ptr(weight), B, CO, CI, G, HW, _ptr(output), float(p), _ptr(w_index_ci),
          _ptr(w_index_co), weight.size(0), weight.size(1) * G, ws.data_ptr() if ws.numel() else None,
          ws.numel() * 4)


def norm_dist_forward_with_max(input, weight, max_output, output, G, p, w_index_ci=None, w_index_co=None):
    """core/cuda/norm_dist.cpp:67-85.  Never called by the reference's Python code; provided for
    completeness.  The supplied maximum is not needed: the result equals norm_dist_forward's."""
    _check(max_output, "max_output")
    if max_output.shape != output.shape:
        raise RuntimeError("max_output must have the shape of output")
    norm_dist_forward(input, weight, output, G, p, w_index_ci, w_index_co)


def norm_dist_backward_input(grad_output, input, weight, output, grad_input, G, p,
                             w_index_ci=None, w_index_co=None):
    """core/cuda/norm_dist.cpp:87-106."""
    for t, n in ((grad_output, "grad_output"), (input, "input"), (weight, "weight"), (output, "output"),
                 (grad_input, "grad_input")):
        _check(t, n)
    B, CO, CI, HW = _lp_common(input, weight, output, w_index_ci, w_index_co, G)
    dev = _same_device(grad_output, input, weight, output, grad_input, w_index_ci, w_index_co)
    _call(dev, input, "snb_norm_dist_backward_input", (B, CO, CI),
          _ptr(grad_output), _ptr(input), _ptr(weight), _ptr(output), B, CO, CI, G, HW, _ptr(grad_input),
          float(p), _ptr(w_index_ci), _ptr(w_index_co), weight.size(0), weight.size(1) * G)


def norm_dist_backward_input_weight(grad_output, input, weight, output, grad_input, grad_weight, G, p,
                                    w_index_ci=None, w_index_co=None):
    """core/cuda/norm_dist.cpp:108-129."""
    for t, n in ((grad_output, "grad_output"), (input, "input"), (weight, "weight"), (output, "output"),
                 (grad_input, "grad_input"), (grad_weight, "grad_weight")):
        _check(t, n)
    B, CO, CI, HW = _lp_common(input, weight, output, w_index_ci, w_index_co, G)
    if grad_weight.shape != weight.shape:
        raise RuntimeError("grad_weight must have the shape of weight")
    dev = _same_device(grad_output, input, weight, output, grad_input, grad_weight, w_index_ci, w_index_co)
    _call(dev, input, "snb_norm_dist_backward_input_weight", (B, CO, CI),
          _ptr(grad_output), _ptr(input), _ptr(weight), _ptr(output), B, CO, CI, G, HW, _ptr(grad_input),
          _ptr(grad_weight), float(p), _ptr(w_index_ci), _ptr(w_index_co), weight.size(0),
          weight.size(1) * G)


def bound_inf_dist_forward_nograd(inputL, inputU, weight, outputL, outputU, G):
    """core/cuda/norm_dist.cpp:186-196."""
    for t, n in ((inputL, "inputL"), (inputU, "inputU"), (weight, "weight"), (outputL, "outputL"),
                 (outputU, "outputU")):
        _check(t, n)
    B, CO, CI, HW = _dims(inputL, outputL)
    if inputU.shape != inputL.shape or outputU.shape != outputL.shape or weight.size(0) != CO \
            or weight.size(1) * G != CI:
        raise RuntimeError("shape mismatch")
    dev = _same_device(inputL, inputU, weight, outputL, outputU)
    _call(dev, inputL, "snb_bound_inf_dist_forward_nograd", (B, CO, CI),
          _ptr(inputL), _ptr(inputU), _ptr(weight), B, CO, CI, G, HW, _ptr(outputL), _ptr(outputU))


def bound_inf_dist_forward(inputL, inputU, weight, outputL, outputU, posL, posU, G):
    """core/cuda/norm_dist.cpp:198-211."""
    for t, n in ((inputL, "inputL"), (inputU, "inputU"), (weight, "weight"), (outputL, "outputL"),
                 (outputU, "outputU")):
        _check(t, n)
    _check(posL, "posL", torch.int32); _check(posU, "posU", torch.int32)
    B, CO, CI, HW = _dims(inputL, outputL)
    if inputU.shape != inputL.shape or outputU.shape != outputL.shape or weight.size(0) != CO \
            or weight.size(1) * G != CI or posL.shape != outputL.shape or posU.shape != outputL.shape:
        raise RuntimeError("shape mismatch")
    dev = _same_device(inputL, inputU, weight, outputL, outputU, posL, posU)
    _call(dev, inputL, "snb_bound_inf_dist_forward", (B, CO, CI),
          _ptr(inputL), _ptr(inputU), _ptr(weight), B, CO, CI, G, HW, _ptr(outputL), _ptr(outputU),
          _ptr(posL), _ptr(posU))


def bound_inf_dist_backward_input(grad_outputL, grad_outputU, posL, posU, grad_inputL, grad_inputU, G):
    """core/cuda/norm_dist.cpp:213-226."""
    for t, n in ((grad_outputL, "grad_outputL"), (grad_outputU, "grad_outputU"),
                 (grad_inputL, "grad_inputL"), (grad_inputU, "grad_inputU")):
        _check(t, n)
    _check(posL, "posL", torch.int32); _check(posU, "posU", torch.int32)
    B, CO, CI, HW = grad_outputL.size(0), grad_outputL.size(1), grad_inputL.size(1), grad_inputL.size(2)
    dev = _same_device(grad_outputL, grad_outputU, posL, posU, grad_inputL, grad_inputU)
    _call(dev, grad_outputL, "snb_bound_inf_dist_backward_input", (B, CO, CI),
          _ptr(grad_outputL), _ptr(grad_outputU), _ptr(posL), _ptr(posU), B, CO, CI, G, HW,
          _ptr(grad_inputL), _ptr(grad_inputU))


def bound_inf_dist_backward_input_weight(grad_outputL, grad_outputU, posL, posU, grad_inputL, grad_inputU,
                                         grad_weight, G):
    """core/cuda/norm_dist.cpp:228-241."""
    for t, n in ((grad_outputL, "grad_outputL"), (grad_outputU, "grad_outputU"),
                 (grad_inputL, "grad_inputL"), (grad_inputU, "grad_inputU"), (grad_weight, "grad_weight")):
        _check(t, n)
    _check(posL, "posL", torch.int32); _check(posU, "posU", torch.int32)
    B, CO, CI, HW = grad_outputL.size(0), grad_outputL.size(1), grad_weight.size(1) * G, grad_outputL.size(2)
    if grad_inputL.size(1) != CI or grad_weight.size(0) != CO:
        raise RuntimeError("shape mismatch")
    dev = _same_device(grad_outputL, grad_outputU, posL, posU, grad_inputL, grad_inputU, grad_weight)
    _call(dev, grad_outputL, "snb_bound_inf_dist_backward_input_weight", (B, CO, CI),
          _ptr(grad_outputL), _ptr(grad_outputU), _ptr(posL), _ptr(posU), B, CO, CI, G, HW,
          _ptr(grad_inputL), _ptr(grad_inputU), _ptr(grad_weight))


def sort_neuron_forward(input, weight, output, pos, G, q, K):
    """core/cuda/norm_dist.cpp:243-251.  pos: int32 [K, B, CO, HW]."""
    _check(input, "input"); _check(weight, "weight"); _check(output, "output"); _check(pos, "pos", torch.int32)
    B, CO, CI, HW = _dims(input, output)
    if weight.size(0) != CO or weight.size(1) * G != CI or tuple(pos.shape) != (K, B, CO, HW):
        raise RuntimeError("shape mismatch")
    dev = _same_device(input, weight, output, pos)
    _call(dev, input, "snb_sort_neuron_forward", (B, CO, CI),
          _ptr(input), _ptr(weight), B, CO, CI, G, HW, _ptr(output), _ptr(pos), float(q), int(K))


def bound_sort_neuron_forward(inputL, inputU, weight, outputL, outputU, G, q, K):
    """core/cuda/norm_dist.cpp:253-263."""
    for t, n in ((inputL, "inputL"), (inputU, "inputU"), (weight, "weight"), (outputL, "outputL"),
                 (outputU, "outputU")):
        _check(t, n)
    B, CO, CI, HW = _dims(inputL, outputL)
    if inputU.shape != inputL.shape or outputU.shape != outputL.shape or weight.size(0) != CO \
            or weight.size(1) * G != CI:
        raise RuntimeError("shape mismatch")
    dev = _same_device(inputL, inputU, weight, outputL, outputU)
    _call(dev, inputL, "snb_bound_sort_neuron_forward", (B, CO, CI),
          _ptr(inputL), _ptr(inputU), _ptr(weight), B, CO, CI, G, HW, _ptr(outputL), _ptr(outputU),
          float(q), int(K))


def sort_neuron_forward_nograd(input, weight, output, G, q, K):
    """core/cuda/norm_dist.cpp:265-272."""
    _check(input, "input"); _check(weight, "weight"); _check(output, "output")
    B, CO, CI, HW = _dims(input, output)
    if weight.size(0) != CO or weight.size(1) * G != CI:
        raise RuntimeError("shape mismatch")
    dev = _same_device(input, weight, output)
    _call(dev, input, "snb_sort_neuron_forward_nograd", (B, CO, CI),
          _ptr(input), _ptr(weight), B, CO, CI, G, HW, _ptr(output), float(q), int(K))


def sort_neuron_backward_input(grad_output, pos, grad_input, G, q, K):
    """core/cuda/norm_dist.cpp:274-281."""
    _check(grad_output, "grad_output"); _check(pos, "pos", torch.int32); _check(grad_input, "grad_input")
    B, CO, CI, HW = grad_output.size(0), grad_output.size(1), grad_input.size(1), grad_input.size(2)
    if tuple(pos.shape) != (K, B, CO, HW):
        raise RuntimeError("pos must have shape [K, B, CO, HW]")
    dev = _same_device(grad_output, pos, grad_input)
    _call(dev, grad_output, "snb_sort_neuron_backward_input", (B, CO, CI),
          _ptr(grad_output), _ptr(pos), B, CO, CI, G, HW, _ptr(grad_input), float(q), int(K))


def sort_neuron_backward_input_weight(grad_output, pos, grad_input, grad_weight, G, q, K):
    """core/cuda/norm_dist.cpp:283-292."""
    _check(grad_output, "grad_output"); _check(pos, "pos", torch.int32)
    _check(grad_input, "grad_input"); _check(grad_weight, "grad_weight")
    B, CO, CI, HW = grad_output.size(0), grad_output.size(1), grad_input.size(1), grad_output.size(2)
    if tuple(pos.shape) != (K, B, CO, HW) or grad_weight.size(0) != CO or grad_weight.size(1) * G != CI:
        raise RuntimeError("shape mismatch")
    dev = _same_device(grad_output, pos, grad_input, grad_weight)
    _call(dev, grad_output, "snb_sort_neuron_backward_input_weight", (B, CO, CI),
          _ptr(grad_output), _ptr(pos), B, CO, CI, G, HW, _ptr(grad_input), _ptr(grad_weight), float(q), int(K))


def mean_shift_stats(x, index, mean, running_mean=None, momentum=0.1):
    """mean[c] over the rows whose sub-batch kept channel c; optional running-mean update.
    x [B, C, 1], index [S, 1, C] int32 or None, mean [C_full] (output)."""
    _check(x, "x"); _check(mean, "mean")
    B, C = x.size(0), x.size(1)
    if x.dim() != 3 or x.size(2) != 1:
        raise RuntimeError("x must have shape [B, C, 1]")
    S = (B + _SUB_BATCH - 1) // _SUB_BATCH
    _check_opt_index(index, "index", S, C)
    if running_mean is not None:
        _check(running_mean, "running_mean")
        if running_mean.numel() != mean.numel():
            raise RuntimeError("running_mean / mean size mismatch")
    dev = _same_device(x, index, mean, running_mean)
    _call(dev, x, "snb_mean_shift_stats", (B, C),
          _ptr(x), _ptr(index), B, C, mean.numel(), _ptr(mean), _ptr(running_mean), float(momentum))


def mean_shift_apply(x, mean, index, y):
    """y[b, j] = x[b, j] - mean[index[s_b][j]]; y may be x."""
    _check(x, "x"); _check(mean, "mean"); _check(y, "y")
    B, C = x.size(0), x.size(1)
    if x.dim() != 3 or x.size(2) != 1 or y.shape != x.shape:
        raise RuntimeError("x and y must have shape [B, C, 1]")
    S = (B + _SUB_BATCH - 1) // _SUB_BATCH
    _check_opt_index(index, "index", S, C)
    if index is None and mean.numel() != C:
        raise RuntimeError("mean must have C entries when there is no index")
    dev = _same_device(x, mean, index, y)
    _call(dev, x, "snb_mean_shift_apply", (B, C),
          _ptr(x), _ptr(mean), _ptr(index), B, C, _ptr(y))


def sample_mask_into(out, channels, seed):
    """out [S, G, count] int32 CUDA tensor -> S * G independent sorted subsets of range(channels)."""
    _check(out, "out", torch.int32)
    if out.dim() != 3:
        raise RuntimeError("out must have shape [sub-batches, groups, count]")
    lists, count = out.size(0) * out.size(1), out.size(2)
    _call(out.device, out, "snb_sample_mask", (lists, channels, count),
          _ptr(out), lists, int(channels), count, int(seed) & 0xFFFFFFFFFFFFFFFF)


def sample_masks_into(outs, channels, seeds):
    """sample_mask_into for several tensors in one launch: outs[j] [S, G, count_j] int32 (the same
    S * G for all), channels[j], seeds[j].  Same lists as separate sample_mask_into calls."""
    if not outs or len(outs) != len(channels) or len(outs) != len(seeds):
        raise RuntimeError("outs, channels and seeds must be non-empty and of equal length")
    lists = outs[0].size(0) * outs[0].size(1)
    for out in outs:
        _check(out, "out", torch.int32)
        if out.dim() != 3 or out.size(0) * out.size(1) != lists or out.device != outs[0].device:
            raise RuntimeError("every out must be [sub-batches, groups, count] with the same number of lists on one device")
    n = len(outs)
    ptrs = (ctypes.c_void_p * n)(*[o.data_ptr() for o in outs])
    chans = (ctypes.c_int * n)(*[int(c) for c in channels])
    counts = (ctypes.c_int * n)(*[o.size(2) for o in outs])
    seed_arr = (ctypes.c_ulonglong * n)(*[int(s) & 0xFFFFFFFFFFFFFFFF for s in seeds])
    _call(outs[0].device, outs[0], "snb_sample_mask_batch", (n, lists, max(int(c) for c in channels)),
          n, ptrs, chans, counts, seed_arr, lists)


# ---- whole layers and the model head (one C call each; G = 1, HW = 1, 2-D tensors) ---------------

_LAYER_KERNELS = {"snb_layer_forward": 4, "snb_layer_backward": 4, "snb_layer_bound_forward": 3, "snb_input_box": 1,
                  "snb_margin_loss": 2, "snb_certified_fraction": 2}


def _layer_call(entry, tag, ref, *args):
    """Lean variant of _call for the layer-level entry points: the callers in ops.py / layers.py own
    every tensor they pass (fresh allocations of the right shape and dtype), so only the device is
    looked after here."""
    global launch_count
    if _timeline is not None:
        return _call(ref.device, ref, entry, tag, *args)
    dev = ref.device
    fn = getattr(_lib.load(), entry)
    if torch.cuda.current_device() == dev.index:
        rc = fn(*args, torch.cuda.current_stream(dev).cuda_stream)
    else:
        with torch.cuda.device(dev):
            rc = fn(*args, torch.cuda.current_stream(dev).cuda_stream)
    if rc:
        _lib.check(rc, entry[4:])
    launch_count += _LAYER_KERNELS[entry]


_KERNELS.update(_LAYER_KERNELS)


def layer_forward(x, weight, p, w_index_ci, w_index_co, y_dist, pos, workspace, running_mean, momentum, mean, bias,
                  out):
    """snb_layer_forward on 2-D tensors: x [B, CI'], weight [W_CO, W_CI], y_dist / out [B, CO'],
    pos int32 [B, CO'] or None, workspace any tensor or None, mean [W_CO] or None (None = no mean
    shift), running_mean [W_CO] or None, bias [W_CO] or None."""
    B, CI = x.shape
    CO = y_dist.size(1)
    nbytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    _layer_call("snb_layer_forward", (B, CO, CI), x,
                x.data_ptr(), weight.data_ptr(), B, CO, CI, float(p), _ptr(w_index_ci), _ptr(w_index_co),
                weight.size(0), weight.size(1), y_dist.data_ptr(), _ptr(pos), _ptr(workspace), nbytes,
                _ptr(running_mean), float(momentum), _ptr(mean), _ptr(bias), out.data_ptr())


def layer_backward(grad_out, x, weight, y_dist, pos, p, w_index_ci, w_index_co, mean_shift, mean, grad_centred,
                   grad_bias, grad_x, grad_w):
    """snb_layer_backward on 2-D tensors (see layer_forward); grad_x [B, CI'] or None, grad_w like
    weight or None, grad_bias [W_CO] or None; mean [W_CO] and grad_centred [B, CO'] are scratch for
    the mean-shift part."""
    B, CO = grad_out.shape
    CI = x.size(1)
    _layer_call("snb_layer_backward", (B, CO, CI), grad_out,
                grad_out.data_ptr(), x.data_ptr(), weight.data_ptr(), _ptr(y_dist), _ptr(pos), B, CO, CI, float(p),
                _ptr(w_index_ci), _ptr(w_index_co), weight.size(0), weight.size(1), 1 if mean_shift else 0,
                _ptr(mean), _ptr(grad_centred), _ptr(grad_bias), _ptr(grad_x), _ptr(grad_w))


def layer_bound_forward(x, xl, xu, weight, running_mean, bias, y, yl, yu):
    """snb_layer_bound_forward on 2-D tensors; x / y or xl, xu / yl, yu may be None."""
    some = x if x is not None else xl
    B, CI = some.shape
    CO = weight.size(0)
    _layer_call("snb_layer_bound_forward", (B, CO, CI), some,
                _ptr(x), _ptr(xl), _ptr(xu), weight.data_ptr(), B, CO, CI, _ptr(running_mean), _ptr(bias), _ptr(y),
                _ptr(yl), _ptr(yu))


def input_box(x, eps, down, up, xl, xu):
    """xl = max(x - eps, down), xu = min(x + eps, up) with Python-number bounds."""
    _layer_call("snb_input_box", (x.numel(),), x, x.data_ptr(), float(eps), float(down), float(up), x.numel(),
                xl.data_ptr(), xu.data_ptr())


def margin_loss(d, targets, eps, clip, lam, scale, margin, row_loss, loss, grad_d):
    """snb_margin_loss: d [B, K] fp32, targets [B] int64; margin [B, K] / grad_d [B, K] optional."""
    B, K = d.shape
    _layer_call("snb_margin_loss", (B, K), d, d.data_ptr(), targets.data_ptr(), B, K, float(eps), float(clip),
                float(lam), float(scale), _ptr(margin), row_loss.data_ptr(), loss.data_ptr(), _ptr(grad_d))


def certified_fraction(yl, yu, targets, row_flag, fraction):
    """snb_certified_fraction: bounds [B, K] fp32, targets [B] int64 -> fraction (0-d / 1-element)."""
    B, K = yl.shape
    _layer_call("snb_certified_fraction", (B, K), yl, yl.data_ptr(), yu.data_ptr(), targets.data_ptr(), B, K,
                row_flag.data_ptr(), fraction.data_ptr())


def install():
    """Registers this module under the name the reference's operator layer imports."""
    sys.modules["norm_dist_cuda"] = sys.modules[__name__]
    return sys.modules[__name__]
