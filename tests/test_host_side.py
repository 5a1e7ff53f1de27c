"""CPU-only checks of the host side: the C-ABI library exports what the header declares, the
tensor-level module offers the reference extension's names, and argument validation works
without touching a GPU."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "sortnet_b200.h")).read()
    return sorted(set(re.findall(r"\b(snb_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def built_lib():
    from sortnet_b200 import build
    return ctypes.CDLL(build.build())


def test_library_exports_every_declared_symbol(built_lib):
    names = declared_symbols()
    assert len(names) >= 16
    for n in names:
        assert hasattr(built_lib, n), n


def test_loader_signatures_cover_the_header(built_lib):
    from sortnet_b200 import _lib
    utility = {"snb_status_string", "snb_last_cuda_error", "snb_version", "snb_inf_dist_forward_workspace_bytes",
               "snb_inf_dist_forward_noalloc_max_outputs", "snb_device_wait_failed", "snb_trim_scratch",
               "snb_norm_dist_forward_workspace_bytes", "snb_inf_dist_forward_sorted_workspace_bytes"}
    assert set(_lib.SIGNATURES) | utility == set(declared_symbols())
    lib = _lib.load()
    assert lib.snb_version() >= 100
    assert lib.snb_status_string(0) == b"ok" and b"null" in lib.snb_status_string(1)
    assert lib.snb_inf_dist_forward_workspace_bytes(512, 5120) == 8 * 512 * 5120
    # merge keys + full-width input + one inverse list per 32-row sub-batch
    assert lib.snb_inf_dist_forward_sorted_workspace_bytes(512, 4600, 5120) == 8 * 512 * 4600 + 4 * 512 * 5120 + 4 * 16 * 5120
    assert lib.snb_inf_dist_forward_sorted_workspace_bytes(33, 3, 8) == 800 + 4 * 33 * 8 + 4 * 2 * 8   # 792 rounded up to 16


def test_status_codes_without_gpu(built_lib):
    # argument checks run before any CUDA call
    from sortnet_b200 import _lib
    lib = _lib.load()
    assert lib.snb_inf_dist_forward_nograd(None, None, 1, 1, 1, 1, 1, None, None) == 1
    one = ctypes.c_void_p(16)
    assert lib.snb_inf_dist_forward_nograd(one, one, 1, 1, 1, 2, 1, one, None) == 2      # 1 channel, 2 groups
    assert lib.snb_inf_dist_forward_noalloc(one, one, 2, 2, 2, 2, 1, one, one, None) == 3   # groups need scratch
    assert lib.snb_inf_dist_forward_nograd(one, one, 0, 1, 1, 1, 1, one, None) == 2      # empty batch
    assert lib.snb_inf_dist_forward(one, one, 4, 4, 4, 1, 1, one, one, None, None, 5, 4, None) == 2
    assert lib.snb_norm_dist_forward(one, one, 4, 4, 4, 1, 1, one, ctypes.c_float(-1.0), None, None, 4, 4, None) == 3
    assert lib.snb_bound_inf_dist_forward_nograd(one, one, one, 70000, 70000, 4, 1, 1, one, one, None) == 4
    with pytest.raises(_lib.SortnetB200Error):
        _lib.check(2, "probe")


REFERENCE_NAMES = [
    "norm_dist_forward", "norm_dist_forward_with_max", "norm_dist_backward_input",
    "norm_dist_backward_input_weight", "inf_dist_forward", "inf_dist_forward_nograd",
    "inf_dist_backward_input", "inf_dist_backward_input_weight", "bound_inf_dist_forward",
    "bound_inf_dist_forward_nograd", "bound_inf_dist_backward_input", "bound_inf_dist_backward_input_weight",
    "sort_neuron_forward", "bound_sort_neuron_forward", "sort_neuron_forward_nograd",
    "sort_neuron_backward_input", "sort_neuron_backward_input_weight",
]


def test_tensor_level_module_has_the_reference_names():
    from sortnet_b200 import norm_dist_cuda as C
    for n in REFERENCE_NAMES:
        assert callable(getattr(C, n)), n


def test_tensor_checks_raise_on_cpu_tensors():
    from sortnet_b200 import norm_dist_cuda as C
    x = torch.rand(4, 8, 1)
    w = torch.rand(3, 8)
    y = torch.empty(4, 3, 1)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        C.inf_dist_forward_nograd(x, w, y, 1)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        C.bound_inf_dist_forward_nograd(x, x, w, y, y, 1)


def test_operator_layer_signatures_match_the_reference():
    import inspect
    from sortnet_b200 import ops
    want = {
        "norm_dist": ["input", "weight", "p", "groups", "use_custom_cuda_func", "tag"],
        "norm_dist_dropout": ["input", "weight", "w_index_ci", "w_index_co", "p", "groups",
                              "use_custom_cuda_func", "tag"],
        "sort_neuron": ["input", "weight", "groups", "q", "truncate", "use_custom_cuda_func", "tag"],
        "bound_sort_neuron": ["x_lower", "x_upper", "weight", "groups", "q", "truncate", "tag"],
        "bound_inf_dist": ["x_lower", "x_upper", "weight", "groups", "use_custom_cuda_func", "tag"],
    }
    for name, params in want.items():
        assert list(inspect.signature(getattr(ops, name)).parameters) == params, name
    for cls in ("NormDistF", "NormDistDropoutF", "SortNeuronF", "BoundInfDistF"):
        assert issubclass(getattr(ops, cls), torch.autograd.Function)


def test_sample_mask_format():
    from sortnet_b200.layers import sample_mask
    torch.manual_seed(0)
    m = sample_mask(3, 1, 50, 0.8, device="cpu")
    assert m.dtype == torch.int32 and m.dim() == 3 and m.size(0) == 3 and m.size(1) == 1
    assert bool((m[..., 1:] > m[..., :-1]).all()) and int(m.max()) < 50 and int(m.min()) >= 0


def test_model_state_dict_keys_match_the_reference_layout():
    from sortnet_b200.layers import SortMLPModel
    model = SortMLPModel(depth=4, width=16, input_dim=(1, 2, 2), num_classes=3, dropout=0.9)
    keys = set(model.state_dict().keys())
    assert keys == {"fc_dist.0.weight", "fc_dist.0.mean_shift.running_mean", "fc_dist.1.weight",
                    "fc_dist.1.mean_shift.running_mean", "fc_dist.2.weight",
                    "fc_dist.2.mean_shift.running_mean", "fc_dist.3.weight", "fc_dist.3.bias"}


def test_shard_bounds_tile_the_flat_buffer():
    from sortnet_b200.optim import shard_bounds
    for numel in (4, 8, 120, 4096, 120644 // 4 * 4):
        for world in (1, 2, 3, 4, 8):
            edges = [shard_bounds(numel, world, r) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == numel
            for (lo, hi), (lo2, _) in zip(edges, edges[1:]):
                assert hi == lo2 and lo <= hi
            assert all(lo % 4 == 0 and hi % 4 == 0 for lo, hi in edges)
