"""The framework-agnostic C interface (``csrc/include/teb200/c_api.h``) driven through ctypes: handle
life cycle and argument validation on CPU, GEMM / quantize / norm numerics on a GPU."""
import ctypes as C
import os

import pytest
import torch

_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "transformerengine_b200", "_teb200_C.so")
pytestmark = pytest.mark.skipif(not os.path.exists(_SO), reason="extension not built")

OK, INVALID, UNSUPPORTED = 0, 1, 2
F32, F16, BF16, BYTE, E4M3, E5M2 = 0, 1, 2, 3, 4, 5
NONE, TENSOR, MXFP8, NVFP4 = 0, 1, 2, 3
ROW, COL, SCALE, AMAX, ROW_SINV, COL_SINV = 0, 1, 2, 3, 4, 5


@pytest.fixture(scope="module")
def lib():
    l = C.CDLL(_SO)
    l.teb200_last_error.restype = C.c_char_p
    l.teb200_version.restype = C.c_char_p
    l.teb200_scale_inv_bytes.restype = C.c_int64
    l.teb200_scale_inv_bytes.argtypes = [C.c_int, C.c_int64, C.c_int64, C.c_int]
    l.teb200_tensor_set_param.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_int64), C.c_int]
    l.teb200_tensor_destroy.argtypes = [C.c_void_p]
    l.teb200_gemm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
    l.teb200_quantize.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    l.teb200_dequantize.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    l.teb200_norm_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p]
    return l


def _tensor(lib, scaling):
    h = C.c_void_p()
    assert lib.teb200_tensor_create(scaling, C.byref(h)) == OK
    return h


def _set(lib, h, which, ptr, dtype, shape):
    arr = (C.c_int64 * len(shape))(*shape)
    return lib.teb200_tensor_set_param(h, which, C.c_void_p(ptr), dtype, arr, len(shape))


def test_handles_and_validation(lib):
    assert b"teb200" in lib.teb200_version()
    h = _tensor(lib, NONE)
    # an unscaled tensor cannot hold FP8 data; misaligned data is refused
    assert _set(lib, h, ROW, 4096, E4M3, [4, 8]) == INVALID
    assert b"unscaled" in lib.teb200_last_error()
    assert _set(lib, h, ROW, 4100, BF16, [4, 8]) == INVALID
    assert _set(lib, h, ROW, 4096, BF16, [2, 3, 8]) == OK
    rows, cols = C.c_int64(), C.c_int64()
    assert lib.teb200_tensor_matrix_shape(h, C.byref(rows), C.byref(cols)) == OK
    assert (rows.value, cols.value) == (6, 8)
    ptr, dt, nd = C.c_void_p(), C.c_int(), C.c_int()
    shape = (C.c_int64 * 8)()
    assert lib.teb200_tensor_get_param(h, ROW, C.byref(ptr), C.byref(dt), shape, C.byref(nd)) == OK
    assert ptr.value == 4096 and dt.value == BF16 and list(shape[:nd.value]) == [2, 3, 8]
    assert lib.teb200_tensor_destroy(h) == OK
    bad = C.c_void_p()
    assert lib.teb200_tensor_create(99, C.byref(bad)) == INVALID
    # scale buffer sizes: swizzled 128 x 4 tiles for MXFP8 / NVFP4, fp32 blocks for block scaling
    assert lib.teb200_scale_inv_bytes(MXFP8, 256, 1024, 0) == 256 * 32
    assert lib.teb200_scale_inv_bytes(MXFP8, 200, 96, 0) == 256 * 4
    assert lib.teb200_scale_inv_bytes(MXFP8, 256, 1024, 1) == 1024 * 8
    assert lib.teb200_scale_inv_bytes(NVFP4, 128, 64, 0) == 128 * 4
    assert lib.teb200_scale_inv_bytes(4, 64, 256, 0) == 64 * 2 * 4
    assert lib.teb200_scale_inv_bytes(5, 256, 256, 0) == 2 * 2 * 4


def test_quant_config(lib):
    c = C.c_void_p()
    assert lib.teb200_quant_config_create(C.byref(c)) == OK
    v = C.c_int(1)
    assert lib.teb200_quant_config_set(c, 2, C.byref(v), C.sizeof(v)) == OK
    out = C.c_int(0)
    assert lib.teb200_quant_config_get(c, 2, C.byref(out), C.sizeof(out)) == OK and out.value == 1
    seed = C.c_uint64(1234567890123)
    assert lib.teb200_quant_config_set(c, 5, C.byref(seed), 8) == OK
    assert lib.teb200_quant_config_set(c, 5, C.byref(v), 4) == INVALID      # wrong size for a uint64 attribute
    assert lib.teb200_quant_config_set(c, 42, C.byref(v), 4) == INVALID
    assert lib.teb200_quant_config_destroy(c) == OK


def test_gemm_argument_checks_launch_nothing(lib):
    a, b, d = _tensor(lib, NONE), _tensor(lib, NONE), _tensor(lib, NONE)
    _set(lib, a, ROW, 4096, BF16, [128, 64])
    _set(lib, b, ROW, 8192, BF16, [256, 32])
    _set(lib, d, ROW, 16384, BF16, [128, 256])
    status = C.c_void_p(65536)
    assert lib.teb200_gemm(a, b, d, None, 0, 1.0, status, None) == INVALID     # K mismatch
    assert b"contraction" in lib.teb200_last_error()
    _set(lib, b, ROW, 8192, BF16, [256, 64])
    assert lib.teb200_gemm(a, b, d, None, 0, 1.0, None, None) == INVALID       # no status word
    m = _tensor(lib, MXFP8)
    _set(lib, m, ROW, 4096, E4M3, [128, 64])
    assert lib.teb200_gemm(m, b, d, None, 0, 1.0, status, None) == INVALID     # mixed scaling modes
    t1, t2 = _tensor(lib, TENSOR), _tensor(lib, TENSOR)
    _set(lib, t1, ROW, 4096, E4M3, [128, 64])
    _set(lib, t2, ROW, 8192, E4M3, [256, 64])
    assert lib.teb200_gemm(t1, t2, d, None, 0, 1.0, status, None) == UNSUPPORTED
    for h in (a, b, d, m, t1, t2):
        assert lib.teb200_tensor_destroy(h) == OK


@pytest.mark.gpu
def test_gemm_quantize_norm_on_gpu(lib):
    torch.manual_seed(0)
    dev = "cuda"
    M, N, K = 256, 384, 512
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    hx, hw, hb, ho = (_tensor(lib, NONE) for _ in range(4))
    assert _set(lib, hx, ROW, x.data_ptr(), BF16, [M, K]) == OK
    assert _set(lib, hw, ROW, w.data_ptr(), BF16, [N, K]) == OK
    assert _set(lib, hb, ROW, bias.data_ptr(), BF16, [N]) == OK
    assert _set(lib, ho, ROW, out.data_ptr(), BF16, [M, N]) == OK
    assert lib.teb200_gemm(hx, hw, ho, hb, 0, 1.0, C.c_void_p(status.data_ptr()), stream) == OK, lib.teb200_last_error()
    ref = x.float() @ w.float().t() + bias.float()
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-1)
    # MXFP8: quantize both operands through the C interface, multiply, compare with the fp32 product
    def mx(t, rows, cols):
        h = _tensor(lib, MXFP8)
        data = torch.empty(rows, cols, device=dev, dtype=torch.uint8)
        sinv = torch.zeros(lib.teb200_scale_inv_bytes(MXFP8, rows, cols, 0), device=dev, dtype=torch.uint8)
        assert _set(lib, h, ROW, data.data_ptr(), E4M3, [rows, cols]) == OK
        assert _set(lib, h, ROW_SINV, sinv.data_ptr(), BYTE, [sinv.numel()]) == OK
        return h, data, sinv
    qx, dx, sx = mx(x, M, K)
    qw, dw, sw = mx(w, N, K)
    assert lib.teb200_quantize(hx, qx, None, stream) == OK, lib.teb200_last_error()
    assert lib.teb200_quantize(hw, qw, None, stream) == OK, lib.teb200_last_error()
    out2 = torch.empty_like(out)
    ho2 = _tensor(lib, NONE)
    _set(lib, ho2, ROW, out2.data_ptr(), BF16, [M, N])
    assert lib.teb200_gemm(qx, qw, ho2, None, 0, 1.0, C.c_void_p(status.data_ptr()), stream) == OK, lib.teb200_last_error()
    ref2 = x.float() @ w.float().t()
    err = (out2.float() - ref2).norm() / ref2.norm()
    assert err < 0.06, err
    # dequantize returns the quantized values: close to the input
    back = torch.empty_like(x)
    hback = _tensor(lib, NONE)
    _set(lib, hback, ROW, back.data_ptr(), BF16, [M, K])
    assert lib.teb200_dequantize(qx, hback, stream) == OK, lib.teb200_last_error()
    assert ((back.float() - x.float()).norm() / x.float().norm()) < 0.05
    # RMSNorm
    g = torch.rand(K, device=dev, dtype=torch.bfloat16) + 0.5
    y = torch.empty_like(x)
    rs = torch.empty(M, device=dev, dtype=torch.float32)
    hg, hy = _tensor(lib, NONE), _tensor(lib, NONE)
    _set(lib, hg, ROW, g.data_ptr(), BF16, [K])
    _set(lib, hy, ROW, y.data_ptr(), BF16, [M, K])
    assert lib.teb200_norm_forward(hx, hg, None, 1e-5, 0, hy, None, C.c_void_p(rs.data_ptr()), stream) == OK, lib.teb200_last_error()
    xf = x.float()
    refn = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()
    torch.testing.assert_close(y.float(), refn, rtol=2e-2, atol=2e-2)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for h in (hx, hw, hb, ho, ho2, qx, qw, hback, hg, hy):
        assert lib.teb200_tensor_destroy(h) == OK
