"""Export mode switch (reference: ``pytorch/export.py``).  Inside ``onnx_export(True)`` modules
take their pure-PyTorch path (``ops.ref``), which traces to standard ATen operators; the custom
sm_100a kernels are opaque to exporters."""
from contextlib import contextmanager

_IN_EXPORT = False


def is_in_onnx_export_mode() -> bool:
    return _IN_EXPORT


@contextmanager
def onnx_export(enabled: bool = False):
    global _IN_EXPORT
    prev, _IN_EXPORT = _IN_EXPORT, bool(enabled)
    try:
        yield
    finally:
        _IN_EXPORT = prev
