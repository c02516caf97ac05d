r"""Builds the reference's own single-GPU operators into oracle/_ref.  TEST INFRASTRUCTURE.

The reference's native operators (cuda/local_exchange.cu, cuda/balancing.cu,
cuda/parallel_linear.cu, with cuda/stream_manager.cpp and the pybind file
cuda/fmoe_cuda.cpp) are compiled where they lie, unmodified and without NCCL
(``FMOE_USE_NCCL`` undefined), by ``torch.utils.cpp_extension.load`` -- not by the
reference's setup.py.  Nothing is copied; only the built module
``oracle/_ref/fmoe_cuda_ref*.so`` is written (git-ignored, shipped to the GPU box).

The module is used by tests/test_vs_reference_ext.py (when present) to run the
reference's kernels next to this library's on the same GPU inputs, and by
tests/golden/make_routing_golden.py to record their outputs.
"""
import glob
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "fmoe_cuda_ref"
SOURCES = ["fmoe_cuda.cpp", "stream_manager.cpp", "balanced_assignment.cpp", "local_exchange.cu", "balancing.cu",
           "parallel_linear.cu"]


def default_reference():
    """The reference checkout: $FASTERMOE_REFERENCE, else the directory `reference` beside this repository."""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return os.environ.get("FASTERMOE_REFERENCE") or os.path.join(os.path.dirname(here), "reference")


def built_path():
    hits = glob.glob(os.path.join(OUT, NAME + "*.so"))
    return hits[0] if hits else None


def build(reference=None, verbose=False):
    reference = reference or default_reference()
    from torch.utils import cpp_extension
    cuda_dir = os.path.join(reference, "cuda")
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    cpp_extension.load(
        name=NAME, sources=[os.path.join(cuda_dir, s) for s in SOURCES], build_directory=OUT,
        extra_include_paths=[cuda_dir],
        extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-O3"],
        extra_ldflags=["-lcublas"], verbose=verbose, is_python_module=False)
    return built_path()


def build_if_possible(reference=None):
    """Builds when the reference checkout is mounted and nothing is built yet."""
    reference = reference or default_reference()
    if built_path() or not os.path.isdir(os.path.join(reference, "cuda")):
        return built_path()
    try:
        return build(reference)
    except Exception as e:  # the checker is optional; the product does not depend on it
        sys.stderr.write(f"[oracle/build_ref] reference operators not built: {e}\n")
        return None


def load():
    """Imports the built module (None if absent).  Needs a CUDA device to be useful."""
    path = built_path()
    if not path:
        return None
    import importlib.util
    import torch  # noqa: F401  (the module links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(verbose=True))
