"""Compiles the REFERENCE's own CUDA extension (fused_decode.cpp + decode_kernel.cu of
Anay21013/Spherical-KV) from the sources where they lie, into oracle/_ref/.

    python oracle/build_ref.py            # needs the reference tree and nvcc; no GPU needed

Test infrastructure only: the built module is the same-box comparison kernel for the
LayerPool-format operators (tests/test_gpu_ref_cuda.py, bench.py --workload pool).  Nothing of
the reference is copied into this repository: the sources are compiled in place and only the
binary lands in oracle/_ref/ (git-ignored).  The extension is built under another name than the
reference's `fused_decode_cuda` so that it cannot collide with a build cache of the reference.
"""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "sphkv_ref_fused_decode"
# the reference checkout: $SPHKV_REFERENCE, else a directory named "reference" beside this repository
REF = os.environ.get("SPHKV_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


def built_path() -> str:
    return os.path.join(OUT, NAME + ".so")


def build(verbose: bool = False) -> str | None:
    """Returns the path of the built module, or None when the reference tree is absent."""
    srcs = [os.path.join(REF, "fused_decode.cpp"), os.path.join(REF, "decode_kernel.cu")]
    if not all(os.path.exists(s) for s in srcs):
        return built_path() if os.path.exists(built_path()) else None
    if os.path.exists(built_path()) and all(os.path.getmtime(built_path()) >= os.path.getmtime(s) for s in srcs):
        return built_path()
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    load(NAME, sources=srcs, build_directory=OUT, verbose=verbose, is_python_module=False,
         extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"])
    return built_path()


def load_module():
    """Imports the built extension (pybind module with `forward` and `encode_append`,
    fused_decode.cpp:16-19); None when it has not been built."""
    path = built_path()
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv)
    print(p if p else "reference tree not found: nothing built")
