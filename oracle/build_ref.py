"""Builds the reference's own CUDA extension for sm_100a into oracle/_ref/ and stages the
reference's operator / layer / model Python beside it (TEST INFRASTRUCTURE).

    python -m oracle.build_ref            # needs the reference checkout, see REF below

The CUDA sources are compiled where they lie (core/cuda/norm_dist.cpp and the four .cu files of
zbh2047/SortNet).  The Python files the drop-in claim is about (core/norm_dist.py,
core/models/*.py, ell_inf_models.py) are placed, byte for byte, under oracle/_ref/py/ so that a
machine without the checkout can still import the *unmodified* reference code.  The whole
output directory is git-ignored: nothing of the reference enters this repository's history.

Users: the GPU tests (the real reference kernels and the real reference model as second
checkers), the benchmark's GPU comparator and its CPU arm.  Never the product path.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# checkout of zbh2047/SortNet: $SORTNET_REFERENCE, else a directory "reference" beside this repository
REF = os.environ.get("SORTNET_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
SOURCES = ["norm_dist.cpp", "inf_dist_cuda.cu", "norm_dist_cuda.cu", "bound_inf_dist_cuda.cu", "sort_neuron.cu"]
PY_OUT = os.path.join(OUT, "py")
PY_FILES = ["ell_inf_models.py", "core/norm_dist.py", "core/models/__init__.py", "core/models/norm_dist.py",
            "core/models/bound_basic_module.py"]


def built_path():
    return os.path.join(OUT, "norm_dist_cuda.so")


def staged_python():
    """Directory holding the staged reference Python (to put on sys.path), or None."""
    ok = all(os.path.exists(os.path.join(PY_OUT, f)) for f in PY_FILES)
    return PY_OUT if ok else None


def stage_python(force: bool = False):
    """Copies the reference's Python files of this path into oracle/_ref/py/ unchanged."""
    if staged_python() and not force:
        return PY_OUT
    if not all(os.path.exists(os.path.join(REF, f)) for f in PY_FILES):
        return None
    for f in PY_FILES:
        dst = os.path.join(PY_OUT, f)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(REF, f), dst)
    return PY_OUT


def build(force: bool = False):
    """Returns the path of the built module, or None when the reference checkout is absent."""
    stage_python(force)
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


def import_reference_python(extension_module):
    """Imports the staged, unmodified reference Python with `extension_module` standing where its
    `import norm_dist_cuda as _C` looks.  Returns (core.norm_dist, core.models, ell_inf_models) or
    None when nothing is staged.  Later calls rebind the operator layer's `_C` to the module given,
    which is how one process runs the same reference code over two different extensions."""
    path = staged_python()
    if path is None:
        return None
    import importlib
    if path not in sys.path:
        sys.path.insert(0, path)
    sys.modules["norm_dist_cuda"] = extension_module
    ops = importlib.import_module("core.norm_dist")
    ops._C = extension_module
    models = importlib.import_module("core.models")
    nets = importlib.import_module("ell_inf_models")
    return ops, models, nets


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
