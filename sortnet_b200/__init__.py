"""sortnet_b200: B200 (sm_100a) kernels for the norm-distance neuron of SortNet.

Layout
    csrc/                 CUDA kernels and the extern "C" entry points (include/sortnet_b200.h)
    build.py              in-tree nvcc build of libsortnet_b200.so
    _lib.py               ctypes loader for the C ABI
    norm_dist_cuda.py     tensor-level functions with the names and argument order of the
                          reference's `norm_dist_cuda` extension module
    ops.py                operator / autograd layer with the signatures of core/norm_dist.py
    layers.py             NormDist / MeanShiftDropout modules and the SortNet-MLP harness

There is no CPU implementation: every operator raises if the CUDA library cannot be loaded.
"""
__all__ = ["norm_dist_cuda", "ops", "layers"]
