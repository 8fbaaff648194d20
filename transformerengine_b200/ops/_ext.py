"""Loader for the in-tree CUDA extension ``transformerengine_b200/_C*.so``.

The extension is compiled for ``sm_100a`` by :func:`build` (called from the
repository's ``__graft_entry__.build``) and placed inside the package so that
the binary is found next to the Python sources without any install step.
Ops on CUDA tensors require it and raise if it is absent: there is no silent
PyTorch fallback on a GPU.  Ops on CPU tensors use the pure-PyTorch reference
path and never touch it.
"""
from __future__ import annotations

import glob
import importlib.machinery
import importlib.util
import os
import sys
from typing import Optional

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_CSRC = os.path.join(_PKG_DIR, "csrc")
_NAME = "_teb200_C"
_mod = None
_err: Optional[BaseException] = None


def sources():
    cu = sorted(glob.glob(os.path.join(_CSRC, "**", "*.cu"), recursive=True))
    cpp = sorted(glob.glob(os.path.join(_CSRC, "**", "*.cpp"), recursive=True))
    return cpp + cu


def so_path() -> Optional[str]:
    hits = sorted(glob.glob(os.path.join(_PKG_DIR, _NAME + "*.so")))
    return hits[0] if hits else None


def cuda_flags():
    return [
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "--expt-relaxed-constexpr", "--use_fast_math", "-Xptxas", "-v",
        "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
        "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
    ]


def build(verbose: bool = False) -> str:
    """Compile every source under ``csrc/`` into ``_teb200_C.so`` inside the package."""
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(max(2, (os.cpu_count() or 4))))
    from torch.utils import cpp_extension

    build_dir = os.path.join(_PKG_DIR, "build")
    os.makedirs(build_dir, exist_ok=True)
    cpp_extension.load(
        name=_NAME,
        sources=sources(),
        extra_include_paths=[os.path.join(_CSRC, "include")],
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=cuda_flags(),
        extra_ldflags=["-lcuda"] if os.path.exists("/usr/local/cuda/lib64/stubs/libcuda.so") and False else [],
        build_directory=build_dir,
        verbose=verbose,
        is_python_module=True,
    )
    built = os.path.join(build_dir, _NAME + ".so")
    dst = os.path.join(_PKG_DIR, _NAME + ".so")
    import shutil

    shutil.copy2(built, dst)
    global _mod, _err
    _mod, _err = None, None
    return dst


def _import(path: str):
    import torch  # noqa: F401  (the extension links against libtorch)

    loader = importlib.machinery.ExtensionFileLoader(_NAME, path)
    spec = importlib.util.spec_from_file_location(_NAME, path, loader=loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    sys.modules[_NAME] = mod
    return mod


def available() -> bool:
    return so_path() is not None


def get():
    """Return the extension module, importing it on first use."""
    global _mod, _err
    if _mod is not None:
        return _mod
    if _err is not None:
        raise RuntimeError(f"CUDA extension failed to load: {_err}") from _err
    p = so_path()
    if p is None:
        raise RuntimeError(
            "transformerengine_b200 CUDA extension is not built; run "
            "`python -c 'import __graft_entry__ as g; g.build()'` from the repository root"
        )
    try:
        _mod = _import(p)
    except BaseException as e:  # noqa: BLE001
        _err = e
        raise
    return _mod


def use_cuda(*tensors) -> bool:
    """True when the op must run on the GPU extension (any CUDA tensor given, not exporting)."""
    from ..export import is_in_onnx_export_mode

    if is_in_onnx_export_mode():
        return False
    for t in tensors:
        if t is not None and getattr(t, "is_cuda", False):
            return True
    return False
