"""Builds the reference's own CUDA extension for sm_100a into oracle/_ref/ (TEST INFRASTRUCTURE).

    python -m oracle.build_ref            # needs the reference checkout, see REF below

The sources are compiled where they lie (core/cuda/norm_dist.cpp and the four .cu files of
zbh2047/SortNet); nothing is copied into this repository and the output directory is
git-ignored.  The resulting module is imported by the GPU tests as a second checker (the real
reference kernels on the same inputs) and by the benchmark as the GPU comparator.  It is never
on the product path.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# checkout of zbh2047/SortNet: $SORTNET_REFERENCE, else a directory "reference" beside this repository
REF = os.environ.get("SORTNET_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
SOURCES = ["norm_dist.cpp", "inf_dist_cuda.cu", "norm_dist_cuda.cu", "bound_inf_dist_cuda.cu", "sort_neuron.cu"]


def built_path():
    return os.path.join(OUT, "norm_dist_cuda.so")


def build(force: bool = False):
    """Returns the path of the built module, or None when the reference checkout is absent."""
    if os.path.exists(built_path()) and not force:
        return built_path()
    src_dir = os.path.join(REF, "core", "cuda")
    if not os.path.isdir(src_dir):
        return None
    os.makedirs(OUT, exist_ok=True)
    from torch.utils import cpp_extension
    cpp_extension.load(
        name="norm_dist_cuda",
        sources=[os.path.join(src_dir, s) for s in SOURCES],
        build_directory=OUT,
        extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-O3"],
        extra_cflags=["-O2"],
        is_python_module=False,     # compile and link only: there is no GPU on the build machine
        verbose=False,
    )
    if not os.path.exists(built_path()):
        return None
    for f in os.listdir(OUT):            # keep only the module: the directory travels with the tree
        if f.endswith(".o") or f.endswith(".d") or f in ("build.ninja", "lock", ".ninja_log", ".ninja_deps"):
            os.remove(os.path.join(OUT, f))
    return built_path()


def load():
    """Imports the built reference extension, or returns None if it is not there."""
    if not os.path.exists(built_path()):
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location("norm_dist_cuda", built_path())
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
