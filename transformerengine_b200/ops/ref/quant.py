"""Pure-PyTorch quantization math (runs on CPU or GPU).

These functions are the numerical oracle for the CUDA kernels in ``csrc/quant``
and the execution path of the library on CPU tensors.  Formulas follow the
reference: per-tensor FP8 scale rule ``common/recipe/recipe_common.cuh:14-49``,
MXFP8 ``common/cast/mxfp8/quantize_mxfp8.cuh:268-300`` with the E8M0 rounding of
``common/util/ptx_arch_spec.cuh:72-104``, NVFP4
``pytorch/custom_recipes/reference_nvfp4.py:651-778``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

FP8_E4M3 = torch.float8_e4m3fn
FP8_E5M2 = torch.float8_e5m2
FP32_MAX = torch.finfo(torch.float32).max


def fp8_max(dtype: torch.dtype) -> float:
    return 448.0 if dtype == FP8_E4M3 else 57344.0


def round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


# ----------------------------------------------------------------------------
# per-tensor FP8
# ----------------------------------------------------------------------------
def compute_scale_from_amax(
    amax: torch.Tensor,
    fp8_max_val: float,
    margin: int = 0,
    force_pow_2: bool = False,
    epsilon: float = 0.0,
    prev_scale: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """scale = (fp8_max / amax) / 2^margin with the reference's guards.

    amax == 0 or non-finite keeps ``prev_scale`` (1.0 if none); an infinite
    scale saturates at fp32 max; ``force_pow_2`` floors to a power of two.
    """
    amax = amax.float()
    if epsilon > 0.0:
        amax = torch.clamp(amax, min=epsilon)
    sf = (fp8_max_val / amax) / (2.0**margin)
    keep = (amax <= 0.0) | ~torch.isfinite(amax)
    sf = torch.where(torch.isinf(sf), torch.full_like(sf, FP32_MAX), sf)
    if force_pow_2:
        # floor to power of two: clear the mantissa bits
        bits = sf.view(torch.int32) & 0x7F800000
        sf = bits.view(torch.float32)
    fallback = prev_scale.float() if prev_scale is not None else torch.ones_like(sf)
    return torch.where(keep, fallback, sf)


def quantize_fp8_tensor(x: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Saturating cast of ``x * scale`` to FP8; returns the FP8 tensor."""
    m = fp8_max(dtype)
    y = x.float() * scale.float()
    y = torch.clamp(y, -m, m)
    return y.to(dtype)


def dequantize_fp8_tensor(q: torch.Tensor, scale_inv: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return (q.float() * scale_inv.float()).to(dtype)


# ----------------------------------------------------------------------------
# E8M0 helpers
# ----------------------------------------------------------------------------
def float_to_e8m0(val: torch.Tensor) -> torch.Tensor:
    """Round a non-negative fp32 value UP to a power of two, biased uint8.

    NaN -> 0xFF, inf -> 0xFE, 0 -> 0.  Sub-normal inputs at or below 2^-127 map
    to exponent 0 (``cvt.rp.satfinite.ue8m0x2.f32``).
    """
    val = val.float().contiguous()
    bits = val.view(torch.int32)
    exponent = (bits >> 23) & 0xFF
    mantissa = bits & 0x7FFFFF
    bump = (mantissa > 0) & (exponent != 0xFE) & ~((exponent == 0) & (mantissa <= 0x400000))
    exponent = exponent + bump.to(torch.int32)
    exponent = torch.where(torch.isnan(val), torch.full_like(exponent, 0xFF), exponent)
    exponent = torch.where(torch.isinf(val), torch.full_like(exponent, 0xFE), exponent)
    exponent = torch.where(val == 0, torch.zeros_like(exponent), exponent)
    return exponent.to(torch.uint8)


def e8m0_to_float(e: torch.Tensor) -> torch.Tensor:
    """2^(e-127) as fp32 (e == 0 gives the sub-normal 2^-127, 255 gives NaN)."""
    e32 = e.to(torch.int32)
    bits = e32 << 23
    bits = torch.where(e32 == 0, torch.full_like(bits, 0x00400000), bits)
    bits = torch.where(e32 == 255, torch.full_like(bits, 0x7FFFFFFF), bits)
    return bits.view(torch.float32)


def e8m0_rcp(e: torch.Tensor) -> torch.Tensor:
    """2^(127-e) as fp32, the factor applied to values before the FP8 cast."""
    e32 = e.to(torch.int32)
    bits = (254 - e32) << 23
    bits = torch.where(e32 == 254, torch.full_like(bits, 0x00400000), bits)
    bits = torch.where(e32 == 255, torch.full_like(bits, 0x7FFFFFFF), bits)
    return bits.view(torch.float32)


# ----------------------------------------------------------------------------
# MXFP8
# ----------------------------------------------------------------------------
MX_BLOCK = 32


def quantize_mxfp8_rowwise(x2d: torch.Tensor, dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantize along the last dim.  Returns (fp8 data [R,C], e8m0 scales [R,C/32])."""
    R, C = x2d.shape
    assert C % MX_BLOCK == 0, f"MXFP8 needs the quantized dim to be a multiple of 32, got {C}"
    xb = x2d.float().reshape(R, C // MX_BLOCK, MX_BLOCK)
    amax = xb.abs().amax(dim=-1)
    e = float_to_e8m0(amax * (1.0 / fp8_max(dtype)))
    rcp = e8m0_rcp(e).unsqueeze(-1)
    m = fp8_max(dtype)
    q = torch.clamp(xb * rcp, -m, m).to(dtype).reshape(R, C)
    return q, e


def quantize_mxfp8_2d(x2d: torch.Tensor, dtype: torch.dtype, rowwise: bool = True, columnwise: bool = True):
    """MXFP8 with one scale per 32 x 32 block (weights): the row-wise scales repeat over the 32 rows of a block,
    the column-wise ones over its 32 columns, so both copies hold the SAME values (the column-wise data is the
    transpose of the row-wise data) in the ordinary MXFP8 layout.  Returns the tuple of ``quantize_mxfp8``.
    (Reference: ``MXFP8Quantizer(with_2d_quantization=True)``, ``MXFP8BlockScaling(enable_2d_quantization=True)``.)"""
    R, C = x2d.shape
    assert R % MX_BLOCK == 0 and C % MX_BLOCK == 0, f"2-D MXFP8 blocks need both dims to be multiples of 32, got {R}x{C}"
    m = fp8_max(dtype)
    xb = x2d.float().reshape(R // MX_BLOCK, MX_BLOCK, C // MX_BLOCK, MX_BLOCK)
    e = float_to_e8m0(xb.abs().amax(dim=(1, 3)) * (1.0 / m))                   # [R/32, C/32]
    q = torch.clamp(xb * e8m0_rcp(e)[:, None, :, None], -m, m).to(dtype).reshape(R, C)
    rd = rs = cd = cs = None
    if rowwise:
        rd, rs = q, e.repeat_interleave(MX_BLOCK, dim=0)                         # [R, C/32]
    if columnwise:
        cd, cs = q.t().contiguous(), e.t().contiguous().repeat_interleave(MX_BLOCK, dim=0)   # [C, R], [C, R/32]
    return rd, rs, cd, cs


def quantize_mxfp8(
    x2d: torch.Tensor, dtype: torch.dtype, rowwise: bool = True, columnwise: bool = True
):
    """MXFP8 quantization of a matrix in one or both directions.

    Returns ``(row_data [R,C], row_scale [R,C/32], col_data_t [C,R], col_scale_t
    [C,R/32])``.  The column-direction copy (blocks of 32 along dim 0) is stored
    TRANSPOSED so that every GEMM operand has its contraction dim contiguous.
    """
    rd = rs = cd = cs = None
    if rowwise:
        rd, rs = quantize_mxfp8_rowwise(x2d, dtype)
    if columnwise:
        cd, cs = quantize_mxfp8_rowwise(x2d.t().contiguous(), dtype)
    return rd, rs, cd, cs


def dequantize_mxfp8_rowwise(q: torch.Tensor, e: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    R, C = q.shape
    nb = C // MX_BLOCK
    s = e8m0_to_float(e[:R, :nb]).unsqueeze(-1)
    return (q.float().reshape(R, nb, MX_BLOCK) * s).reshape(R, C).to(out_dtype)


def pad_scales(e: torch.Tensor, row_mult: int = 128, col_mult: int = 4) -> torch.Tensor:
    """Zero-pad a compact scale matrix to [roundup(R,128), roundup(K,4)]."""
    R, K = e.shape
    Rp, Kp = round_up(R, row_mult), round_up(K, col_mult)
    if (Rp, Kp) == (R, K):
        return e.contiguous()
    out = torch.zeros(Rp, Kp, dtype=e.dtype, device=e.device)
    out[:R, :K] = e
    return out


def swizzle_scales(e: torch.Tensor) -> torch.Tensor:
    """Compact [R,K] scale bytes -> the 128x4-tile layout the tensor core reads.

    Element (i, j) lands at ``((i/128)*ceil(K/4) + j/4)*512 + (i%32)*16 +
    ((i%128)/32)*4 + j%4``.  The result is 1-D of padded size.
    """
    e = pad_scales(e)
    Rp, Kp = e.shape
    t = e.reshape(Rp // 128, 4, 32, Kp // 4, 4)  # [tile, q, r, kt, j]
    return t.permute(0, 3, 2, 1, 4).contiguous().reshape(-1)


def unswizzle_scales(s: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Inverse of :func:`swizzle_scales`; returns the compact [rows, cols] matrix."""
    Rp, Kp = round_up(rows, 128), round_up(cols, 4)
    t = s.reshape(Rp // 128, Kp // 4, 32, 4, 4)  # [tile, kt, r, q, j]
    return t.permute(0, 3, 2, 1, 4).contiguous().reshape(Rp, Kp)[:rows, :cols].contiguous()


# ----------------------------------------------------------------------------
# NVFP4
# ----------------------------------------------------------------------------
NVFP4_BLOCK = 16
_E2M1_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
# decision boundaries for round-to-nearest-even on the E2M1 grid
_E2M1_BOUNDS = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
# at a tie, the code with an even mantissa bit wins: 0.25->0, 0.75->1.0, 1.25->1.0,
# 1.75->2.0, 2.5->2.0, 3.5->4.0, 5.0->4.0
_E2M1_TIE_UP = [False, True, False, True, False, True, False]

RHT_SIGNS = [1, 1, 1, -1, 1, -1, -1, -1, -1, -1, -1, 1, -1, 1, -1, -1]


def cast_to_e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even onto the E2M1 grid; returns 4-bit codes (uint8)."""
    a = x.abs()
    code = torch.zeros_like(a, dtype=torch.uint8)
    for b, tie_up in zip(_E2M1_BOUNDS, _E2M1_TIE_UP):
        code += ((a >= b) if tie_up else (a > b)).to(torch.uint8)
    sign = (torch.signbit(x) & (x != 0)).to(torch.uint8) << 3
    # the reference keeps -0.0 as code 8 only for values in [-0.25, -0.0)
    sign = torch.where((x < 0), torch.full_like(sign, 8), sign)
    return code | sign


def stochastic_round_e2m1_codes(x: torch.Tensor, rand: torch.Tensor) -> torch.Tensor:
    """Stochastic rounding onto the E2M1 grid.  ``rand`` is uniform in [0,1)."""
    grid = torch.tensor(_E2M1_VALUES, dtype=torch.float32, device=x.device)
    a = x.abs().clamp(max=6.0)
    hi_idx = torch.bucketize(a, grid, right=False).clamp(max=7)
    lo_idx = (hi_idx - 1).clamp(min=0)
    lo, hi = grid[lo_idx], grid[hi_idx]
    span = (hi - lo).clamp(min=1e-30)
    p_up = torch.where(hi > lo, (a - lo) / span, torch.zeros_like(a))
    idx = torch.where(rand < p_up, hi_idx, lo_idx)
    idx = torch.where(a == hi, hi_idx, idx)
    return idx.to(torch.uint8) | ((x < 0).to(torch.uint8) << 3)


def pack_fp4(codes: torch.Tensor) -> torch.Tensor:
    """[R, C] 4-bit codes -> [R, C/2] bytes, element 2i in the low nibble."""
    return codes[..., 0::2] | (codes[..., 1::2] << 4)


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    lo = packed & 0xF
    hi = packed >> 4
    return torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def e2m1_codes_to_float(codes: torch.Tensor) -> torch.Tensor:
    grid = torch.tensor(_E2M1_VALUES + [-v for v in _E2M1_VALUES], dtype=torch.float32, device=codes.device)
    return grid[codes.long()]


def hadamard_matrix_16(device=None, dtype=torch.float32, with_signs: bool = True) -> torch.Tensor:
    """16x16 Sylvester Hadamard / 4, rows pre-multiplied by the fixed sign vector."""
    h = torch.ones(1, 1, dtype=torch.float32)
    for _ in range(4):
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    h = h / 4.0
    if with_signs:
        h = torch.diag(torch.tensor(RHT_SIGNS, dtype=torch.float32)) @ h
    return h.to(device=device, dtype=dtype)


def apply_rht(x2d: torch.Tensor) -> torch.Tensor:
    """Random Hadamard transform over blocks of 16 along the last dim."""
    R, C = x2d.shape
    h = hadamard_matrix_16(x2d.device, torch.float32)
    y = x2d.float().reshape(R, C // 16, 16) @ h
    return y.reshape(R, C).to(x2d.dtype)


def nvfp4_global_encode_scale(amax: torch.Tensor) -> torch.Tensor:
    """S_enc = 448*6/amax, clamped to fp32 max; 1 where amax == 0."""
    a = amax.float()
    s = torch.full_like(a, 448.0 * 6.0) / a  # tensor / tensor: "scalar / tensor" is reciprocal-then-multiply on CPU
    s = torch.clamp(s, max=FP32_MAX)
    return torch.where((amax == 0) | (s == 0), torch.ones_like(s), s)


def quantize_nvfp4_1d(
    x2d: torch.Tensor,
    global_amax: torch.Tensor,
    stochastic: bool = False,
    generator: Optional[torch.Generator] = None,
    four_over_six: Optional[str] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """1x16 block NVFP4 quantization along the last dim.

    Returns (packed data [R, C/2] uint8, per-block decode scales [R, C/16] as
    E4M3 bytes).
    """
    R, C = x2d.shape
    assert C % NVFP4_BLOCK == 0
    xb = x2d.float().reshape(R, C // NVFP4_BLOCK, NVFP4_BLOCK)
    vec_max = xb.abs().amax(dim=-1, keepdim=True)
    if four_over_six:
        assert not stochastic, "4-over-6 selection compares deterministic candidates"
        return _nvfp4_encode_4over6(xb, vec_max, global_amax, R, C, four_over_six, rows_per_tile=1)
    return _nvfp4_encode(xb, vec_max, global_amax, stochastic, generator, R, C)


def quantize_nvfp4_2d(x2d: torch.Tensor, global_amax: torch.Tensor,
                      four_over_six: Optional[str] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """16x16 block NVFP4 quantization (weights): one scale shared by 16 rows."""
    R, C = x2d.shape
    assert C % NVFP4_BLOCK == 0 and R % NVFP4_BLOCK == 0
    blocks = x2d.float().reshape(R // 16, 16, C // 16, 16)
    bmax = blocks.abs().amax(dim=(1, 3))  # [R/16, C/16]
    vec_max = bmax.repeat_interleave(16, dim=0).unsqueeze(-1)  # [R, C/16, 1]
    xb = x2d.float().reshape(R, C // 16, 16)
    if four_over_six:
        return _nvfp4_encode_4over6(xb, vec_max, global_amax, R, C, four_over_six, rows_per_tile=16)
    return _nvfp4_encode(xb, vec_max, global_amax, False, None, R, C)


def _nvfp4_encode_4over6(xb, vec_max, global_amax, R, C, err_mode: str, rows_per_tile: int):
    """Adaptive block scaling ("4 over 6"): every block is quantized twice, with its amax mapped to 6 (the largest
    E2M1 value, the standard choice) and mapped to 4 (a block scale 1.5 times larger, which puts the values on a
    grid with a finer top end), and keeps whichever reconstructs the block with the smaller error (``"MAE"``: sum
    of absolute errors, ``"MSE"``: of squared errors, measured on the original values; ties keep 6).  A 16 x 16
    tile (``rows_per_tile == 16``) chooses once for the whole tile.  The caller passes a ``global_amax`` scaled so
    that 1.5 x the block scale still fits E4M3 (global bound 256 instead of 448).
    (Reference: ``pytorch/custom_recipes/reference_nvfp4.py``, the 4over6 path; restated here.)"""
    assert err_mode in ("MAE", "MSE")
    s_enc = nvfp4_global_encode_scale(global_amax.float().reshape(-1)[:1])
    s_dec_global = torch.ones_like(s_enc) / s_enc
    base = torch.clamp(vec_max * (s_enc * torch.full_like(s_enc, 1.0 / 6.0)), max=FP32_MAX)
    cands = []
    for factor in (1.0, 1.5):                                   # map to 6, map to 4
        dec = torch.clamp(base * factor, -448.0, 448.0).to(FP8_E4M3)
        enc = torch.clamp(torch.ones_like(s_enc) / (dec.float() * s_dec_global), max=FP32_MAX)
        codes = cast_to_e2m1_codes(torch.clamp(xb * enc, -6.0, 6.0).reshape(R, C))
        recon = e2m1_codes_to_float(codes).reshape(xb.shape) * (dec.float() * s_dec_global)
        diff = (xb - recon).abs() if err_mode == "MAE" else (xb - recon).square()
        err = diff.sum(dim=-1)                                   # [R, C/16]
        if rows_per_tile > 1:
            err = err.reshape(R // rows_per_tile, rows_per_tile, -1).sum(dim=1).repeat_interleave(rows_per_tile, dim=0)
        cands.append((codes, dec.squeeze(-1), err))
    (c6, d6, e6), (c4, d4, e4) = cands
    use4 = e4 < e6                                               # [R, C/16]
    codes = torch.where(use4.repeat_interleave(NVFP4_BLOCK, dim=1), c4, c6)
    dec = torch.where(use4, d4.float(), d6.float()).to(FP8_E4M3)
    return pack_fp4(codes), dec.view(torch.uint8)


def _nvfp4_encode(xb, vec_max, global_amax, stochastic, generator, R, C):
    # 1-element tensors, not 0-dim ones: CPU kernels promote a 0-dim operand to a double scalar,
    # which changes products such as dec * s_dec_global in the last bit
    s_enc = nvfp4_global_encode_scale(global_amax.float().reshape(-1)[:1])
    s_dec_global = torch.ones_like(s_enc) / s_enc
    dec = vec_max * (s_enc * torch.full_like(s_enc, 1.0 / 6.0))
    dec = torch.clamp(dec, max=FP32_MAX)
    dec = torch.clamp(dec, -448.0, 448.0).to(FP8_E4M3)
    enc = torch.clamp(torch.ones_like(s_enc) / (dec.float() * s_dec_global), max=FP32_MAX)
    scaled = torch.clamp(xb * enc, -6.0, 6.0).reshape(R, C)
    if stochastic:
        rand = torch.rand(scaled.shape, generator=generator, device=scaled.device)
        codes = stochastic_round_e2m1_codes(scaled, rand)
    else:
        codes = cast_to_e2m1_codes(scaled)
    return pack_fp4(codes), dec.squeeze(-1).view(torch.uint8)


def dequantize_nvfp4(
    packed: torch.Tensor, scales_e4m3: torch.Tensor, global_amax: torch.Tensor, out_dtype: torch.dtype
) -> torch.Tensor:
    R, Ch = packed.shape
    C = Ch * 2
    vals = e2m1_codes_to_float(unpack_fp4(packed))
    s_enc = nvfp4_global_encode_scale(global_amax.float().reshape(-1)[:1])
    sd = scales_e4m3[:R, : C // 16].contiguous().view(FP8_E4M3).float() * (torch.ones_like(s_enc) / s_enc)
    return (vals.reshape(R, C // 16, 16) * sd.unsqueeze(-1)).reshape(R, C).to(out_dtype)


# ----------------------------------------------------------------------------
# FP8 block scaling (1x128 and 128x128, fp32 scales)
# ----------------------------------------------------------------------------
def quantize_fp8_blockwise(
    x2d: torch.Tensor, dtype: torch.dtype, block_dims: Tuple[int, int], pow2: bool = True, eps: float = 0.0
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Block-scaled FP8.  ``block_dims`` is (1,128) or (128,128).

    Returns (data [R,C], scale_inv [ceil(R/br), ceil(C/bc)] fp32).
    """
    R, C = x2d.shape
    br, bc = block_dims
    Rp, Cp = round_up(R, br), round_up(C, bc)
    xp = torch.zeros(Rp, Cp, dtype=torch.float32, device=x2d.device)
    xp[:R, :C] = x2d.float()
    blocks = xp.reshape(Rp // br, br, Cp // bc, bc)
    amax = blocks.abs().amax(dim=(1, 3))
    scale = compute_scale_from_amax(amax, fp8_max(dtype), 0, pow2, eps)
    q = torch.clamp(blocks * scale[:, None, :, None], -fp8_max(dtype), fp8_max(dtype))
    q = q.reshape(Rp, Cp)[:R, :C].to(dtype)
    return q, 1.0 / scale


def dequantize_fp8_blockwise(q, scale_inv, block_dims, out_dtype):
    R, C = q.shape
    br, bc = block_dims
    s = scale_inv.repeat_interleave(br, 0)[:R].repeat_interleave(bc, 1)[:, :C]
    return (q.float() * s).to(out_dtype)


def philox_uniform(shape, seed: int, offset: int, device) -> torch.Tensor:
    """Deterministic uniform [0,1) stream for CPU-side stochastic rounding tests."""
    g = torch.Generator(device="cpu")
    g.manual_seed((seed * 0x9E3779B1 + offset) & 0x7FFFFFFFFFFFFFFF)
    return torch.rand(shape, generator=g).to(device)


def amax_abs(x: torch.Tensor) -> torch.Tensor:
    return x.detach().abs().amax().float().reshape(1) if x.numel() else torch.zeros(1, device=x.device)


def log2_ceil(v: float) -> int:
    return int(math.ceil(math.log2(v))) if v > 0 else 0
