"""Build recipe for the reference's own CUDA kernels (test infrastructure: the GPU oracle and GPU baseline).

    python oracle/build_ref.py /path/to/reference        # writes oracle/_ref/haste_ref_C.so

Compiles the reference's four extension sources (shared_ffi/ffi_forward_kernels.cu, ffi_backward_features.cu,
ffi_backward_weights.cu, ffi_wrapper.cpp — the list of its setup.py:10-15) for sm_100a exactly where they lie in
the reference checkout: nothing is copied into this repository and nothing of the reference is modified.  The
reference's setup.py is not run; the module is linked against the PyTorch headers and libraries of the current
interpreter, under the module name ``haste_ref_C`` so that it cannot shadow anything.  Its wmma kernels then run as
legacy (non-tcgen05) code on a B200.

The product never loads this library: only tests and the benchmark's baseline legs do (see ``load``).
"""
import glob
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "haste_ref_C"
SOURCES = ["ffi_forward_kernels.cu", "ffi_backward_features.cu", "ffi_backward_weights.cu", "ffi_wrapper.cpp"]


def lib_path():
    hits = glob.glob(os.path.join(OUT, NAME + "*.so"))
    return hits[0] if hits else None


def build(reference_root, verbose=False):
    from torch.utils import cpp_extension
    src = [os.path.join(reference_root, "shared_ffi", s) for s in SOURCES]
    missing = [s for s in src if not os.path.exists(s)]
    if missing:
        raise FileNotFoundError(f"reference sources not found: {missing}")
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    cpp_extension.load(name=NAME, sources=src, build_directory=OUT, verbose=verbose, is_python_module=True,
                       extra_cflags=["-O3"],
                       extra_cuda_cflags=["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a"])
    return lib_path()


def load():
    """Import the built module (None when it was never built).  Functions, as bound at shared_ffi/ffi_wrapper.cpp:28-44:
    ffi_forward_cuda(locations, features_t, weights, bias, B, H, FANIN, L, gsize),
    ffi_backward_features_cuda(features_t, weights, locations, grad_outputs, B, H, FANIN, L, gsize),
    ffi_backward_weights_cuda(same)."""
    path = lib_path()
    if path is None:
        return None
    import importlib.util
    import torch  # noqa: F401  (the module links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    print(build(sys.argv[1], verbose="-v" in sys.argv))
