"""The allocation-free norm backward, called through its exported C symbol.

Some callers of this library may not allocate device memory (a step whose memory
plan is frozen, a C host without a tensor library).  For them the library exports
``teb200_norm_bwd_noalloc``, which keeps its reduction scratch in a fixed array
inside the library.  This test calls it twice in a row and compares with the
regular entry point, which takes an allocated workspace.
"""
import ctypes

import pytest
import torch

from transformerengine_b200 import ops
from transformerengine_b200.ops import _ext

pytestmark = pytest.mark.gpu


def _lib():
    _ext.get()  # makes sure libtorch and the extension are loaded
    lib = ctypes.CDLL(_ext.so_path())
    fn = lib.teb200_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int] * 6 + [ctypes.c_void_p] * 10
    need = lib.teb200_norm_bwd_noalloc_scratch_floats
    need.restype = ctypes.c_longlong
    need.argtypes = [ctypes.c_int, ctypes.c_int]
    return fn, need


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


@pytest.mark.parametrize("layernorm", [False, True])
def test_noalloc_matches_regular_twice(layernorm):
    fn, need = _lib()
    R, C = 1024, 2048
    assert need(R, C) <= 4 * 1024 * 1024
    dev = "cuda"
    for trial in range(2):  # the shared scratch keeps the previous call's contents
        torch.manual_seed(trial)
        x = torch.randn(R, C, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(R, C, device=dev, dtype=torch.bfloat16)
        g = (torch.randn(C, device=dev) * 0.1 + 1).to(torch.bfloat16)
        b = torch.zeros(C, device=dev, dtype=torch.bfloat16) if layernorm else None
        _, _, mu, rs = ops.norm_fwd(x, g, b, 1e-5, False, layernorm)
        dx_ref, dg_ref, db_ref = ops.norm_bwd(dy, x, mu, rs, g, False, layernorm)
        dx, dg = torch.empty_like(x), torch.empty_like(g)
        db = torch.empty_like(g) if layernorm else None
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = fn(int(layernorm), R, C, 2, 2, 0, _p(dy), _p(x), _p(mu), _p(rs), _p(g), _p(None), _p(dx), _p(dg),
                _p(db), stream)
        assert rc == 0
        torch.cuda.synchronize()
        # same kernels, same reduction order: results agree exactly; keep the usual tolerance anyway
        assert torch.allclose(dx.float(), dx_ref.float(), rtol=5e-3, atol=5e-3)
        assert torch.allclose(dg.float(), dg_ref.float(), rtol=1e-2, atol=1e-2)
        if layernorm:
            assert torch.allclose(db.float(), db_ref.float(), rtol=1e-2, atol=1e-2)


def test_noalloc_rejects_oversize():
    fn, need = _lib()
    R, C = 8192, 16384
    assert need(R, C) > 4 * 1024 * 1024
    z = ctypes.c_void_p(0)
    rc = fn(0, R, C, 2, 2, 0, z, z, z, z, z, z, z, z, z, z)
    assert rc != 0  # refused before any launch, pointers never touched
