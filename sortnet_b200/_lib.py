"""ctypes loader for libsortnet_b200.so (the C ABI declared in include/sortnet_b200.h)."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# SORTNET_B200_LIB lets a caller point at a library built elsewhere (e.g. an experimental build).
LIB_PATH = os.environ.get("SORTNET_B200_LIB") or os.path.join(HERE, "libsortnet_b200.so")

_lib = None

_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float

# name -> argument types (every function returns int status)
SIGNATURES = {
    "snb_inf_dist_forward": [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _I, _I, _P],
    "snb_inf_dist_forward_ws": [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _I, _I, _P, ctypes.c_size_t, _P],
    "snb_inf_dist_forward_sorted_ws": [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _I, _I, _P, ctypes.c_size_t, _P],
    "snb_inf_dist_forward_noalloc": [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P],
    "snb_inf_dist_forward_nograd": [_P, _P, _I, _I, _I, _I, _I, _P, _P],
    "snb_inf_dist_backward_input": [_P, _P, _I, _I, _I, _I, _I, _P, _P],
    "snb_inf_dist_backward_input_weight": [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _I, _I, _P],
    "snb_norm_dist_forward": [_P, _P, _I, _I, _I, _I, _I, _P, _F, _P, _P, _I, _I, _P],
    "snb_norm_dist_forward_ws": [_P, _P, _I, _I, _I, _I, _I, _P, _F, _P, _P, _I, _I, _P, ctypes.c_size_t, _P],
    "snb_norm_dist_backward_input": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _F, _P, _P, _I, _I, _P],
    "snb_norm_dist_backward_input_weight": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _F, _P, _P, _I, _I, _P],
    "snb_bound_inf_dist_forward_nograd": [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P],
    "snb_bound_inf_dist_forward": [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P],
    "snb_bound_inf_dist_backward_input": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P],
    "snb_bound_inf_dist_backward_input_weight": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P],
    "snb_sort_neuron_forward_nograd": [_P, _P, _I, _I, _I, _I, _I, _P, _F, _I, _P],
    "snb_sort_neuron_forward": [_P, _P, _I, _I, _I, _I, _I, _P, _P, _F, _I, _P],
    "snb_bound_sort_neuron_forward": [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _F, _I, _P],
    "snb_sort_neuron_backward_input": [_P, _P, _I, _I, _I, _I, _I, _P, _F, _I, _P],
    "snb_sort_neuron_backward_input_weight": [_P, _P, _I, _I, _I, _I, _I, _P, _P, _F, _I, _P],
    "snb_mean_shift_stats": [_P, _P, _I, _I, _I, _P, _P, _F, _P],
    "snb_mean_shift_apply": [_P, _P, _P, _I, _I, _P, _P],
    "snb_sample_mask": [_P, _I, _I, _I, ctypes.c_ulonglong, _P],
    "snb_sample_mask_batch": [_I, _P, _P, _P, _P, _I, _P],
    "snb_adamw_step": [_P, _P, _P, _P, ctypes.c_longlong, _F, _F, _F, _F, _F, _I, _F, _P],
    "snb_adamw_reduce_step": [_P, _P, _P, _I, _P, _P, ctypes.c_longlong, _F, _F, _F, _F, _F, _I, _F, _P],
    "snb_dp_adamw_step": [_P, _P, _P, _P, _I, _I, ctypes.c_longlong, ctypes.c_longlong, _F, _F, _F, _F, _F, _I, _P],
    "snb_layer_forward": [_P, _P, _I, _I, _I, _F, _P, _P, _I, _I, _P, _P, _P, ctypes.c_size_t, _P, _F, _P, _P, _P, _P],
    "snb_layer_backward": [_P, _P, _P, _P, _P, _I, _I, _I, _F, _P, _P, _I, _I, _I, _P, _P, _P, _P, _P, _P],
    "snb_layer_bound_forward": [_P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P, _P, _P],
    "snb_input_box": [_P, _F, _F, _F, ctypes.c_longlong, _P, _P, _P],
    "snb_margin_loss": [_P, _P, _I, _I, _F, _F, _F, _F, _P, _P, _P, _P, _P],
    "snb_certified_fraction": [_P, _P, _P, _I, _I, _P, _P, _P],
    "snb_peer_barrier": [_P, _I, _I, ctypes.c_uint, ctypes.c_ulonglong, _P, _P],
    "snb_peer_signal": [_P, _I, _I, ctypes.c_uint, _P],
    "snb_peer_wait": [_P, _I, _I, ctypes.c_uint, ctypes.c_ulonglong, _P, _P],
    "snb_check_index_lists": [_P, _I, _I, _I, ctypes.POINTER(ctypes.c_int), _P],
    "snb_probe_fp32": [_P, _I, ctypes.POINTER(ctypes.c_double), _P],
}


class SortnetB200Error(RuntimeError):
    pass


def load(build_if_missing: bool = False):
    """Loads the shared library once and declares the prototypes; raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if build_if_missing:
            from . import build as _build
            _build.build()
        else:
            raise SortnetB200Error(
                "libsortnet_b200.so is not built (run `python -m sortnet_b200.build`); "
                "there is no CPU or PyTorch fallback for these operators")
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int
    lib.snb_status_string.argtypes = [ctypes.c_int]
    lib.snb_status_string.restype = ctypes.c_char_p
    lib.snb_last_cuda_error.argtypes = []
    lib.snb_last_cuda_error.restype = ctypes.c_char_p
    lib.snb_version.argtypes = []
    lib.snb_version.restype = ctypes.c_int
    lib.snb_trim_scratch.argtypes = []
    lib.snb_trim_scratch.restype = ctypes.c_int
    lib.snb_device_wait_failed.argtypes = []
    lib.snb_device_wait_failed.restype = ctypes.c_int
    lib.snb_inf_dist_forward_noalloc_max_outputs.argtypes = []
    lib.snb_inf_dist_forward_noalloc_max_outputs.restype = ctypes.c_int
    lib.snb_inf_dist_forward_workspace_bytes.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.snb_inf_dist_forward_workspace_bytes.restype = ctypes.c_size_t
    lib.snb_inf_dist_forward_sorted_workspace_bytes.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.snb_inf_dist_forward_sorted_workspace_bytes.restype = ctypes.c_size_t
    lib.snb_norm_dist_forward_workspace_bytes.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_float]
    lib.snb_norm_dist_forward_workspace_bytes.restype = ctypes.c_size_t
    _lib = lib
    return lib


def check(status: int, what: str):
    if status == 0:
        return
    lib = load()
    msg = lib.snb_status_string(status).decode()
    if status == 5:
        msg += ": " + lib.snb_last_cuda_error().decode()
    raise SortnetB200Error("%s failed: %s (status %d)" % (what, msg, status))
