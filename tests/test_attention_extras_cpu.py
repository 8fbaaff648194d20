"""Score-modifier attention and the latent-attention query projection (CPU path)."""
import math

import pytest

import torch

import transformerengine_b200 as te
from transformerengine_b200.attention.fused_mla_q_uproj import FusedMLAQUpProjRopeQuant
from transformerengine_b200.tensor import MXFP8Quantizer


def test_score_mod_edits_scores_before_softmax():
    torch.manual_seed(0)
    b, s, h, d = 2, 16, 2, 8
    attn = te.DotProductAttention(h, d, qkv_format="bshd", attn_mask_type="causal")
    q, k, v = (torch.randn(b, s, h, d, requires_grad=True) for _ in range(3))
    slopes = torch.tensor([0.5, 0.25]).reshape(1, h, 1, 1)
    dist = (torch.arange(s)[None, :] - torch.arange(s)[:, None]).float().reshape(1, 1, s, s)

    def mod(score, tensors):
        return score + tensors["slopes"] * tensors["dist"]

    out = attn(q, k, v, score_mod=mod, score_mod_tensors={"slopes": slopes, "dist": dist})
    out.sum().backward()
    qt, kt, vt = (t.detach().transpose(1, 2) for t in (q, k, v))
    sc = qt @ kt.transpose(-1, -2) / math.sqrt(d) + slopes * dist
    sc = sc.masked_fill(torch.triu(torch.ones(s, s, dtype=torch.bool), 1), float("-inf"))
    ref = (sc.softmax(-1) @ vt).transpose(1, 2).reshape(b, s, h * d)
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    assert q.grad is not None and q.grad.abs().sum() > 0


def test_fused_mla_query_projection_matches_composed_math():
    torch.manual_seed(0)
    s, b, k_dim, nh, d, d_rot = 32, 2, 64, 2, 64, 32
    assert FusedMLAQUpProjRopeQuant.is_supported()
    x = torch.randn(s * b, k_dim)
    w = torch.randn(nh * d, k_dim) * 0.1
    ang = torch.rand(s, d_rot // 2) * 6.28
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    q, saved = FusedMLAQUpProjRopeQuant.run(x, w, cos, sin, s, b, head_dim=d)
    assert saved is x and tuple(q.logical_shape) == (s, b, nh, d)
    ref = (x @ w.t()).reshape(s, b, nh, d)
    rot = ref[..., d - d_rot:]
    r1, r2 = rot[..., :d_rot // 2], rot[..., d_rot // 2:]
    c, sn = cos.reshape(s, 1, 1, d_rot), sin.reshape(s, 1, 1, d_rot)
    ref = torch.cat([ref[..., :d - d_rot], rot * c + torch.cat([-r2, r1], -1) * sn], -1)
    got = q.dequantize(dtype=torch.float32)
    assert (got - ref).abs().max() < 0.08 * ref.abs().max()
    assert q.get_usages() == {"rowwise": True, "columnwise": True}

    # FP8 path: an MXFP8 primary weight keeps the projection in MXFP8 and returns the columnwise activation
    wq = MXFP8Quantizer(torch.float8_e4m3fn)(w)
    q2, saved2 = FusedMLAQUpProjRopeQuant.run(x, wq, cos, sin, s, b, head_dim=d)
    assert saved2.get_usages() == {"rowwise": False, "columnwise": True}
    assert (q2.dequantize(dtype=torch.float32) - ref).abs().max() < 0.15 * ref.abs().max()


def test_fused_qkv_split_and_rope_matches_separate_calls():
    from transformerengine_b200.attention.rope import (RotaryPositionEmbedding, apply_fused_qkv_rotary_pos_emb,
                                                       apply_rotary_pos_emb)

    torch.manual_seed(0)
    s, b, g, d = 16, 2, 2, 32
    qkv = torch.randn(s, b, g, 4 * d + d + d, requires_grad=True)
    freqs = RotaryPositionEmbedding(d)(s)
    q, k, v = apply_fused_qkv_rotary_pos_emb(qkv, freqs, freqs, [4 * d, d, d])
    assert q.shape == (s, b, 4 * g, d) and k.shape == (s, b, g, d) and v.shape == (s, b, g, d)
    torch.testing.assert_close(q, apply_rotary_pos_emb(qkv[..., :4 * d].reshape(s, b, 4 * g, d), freqs))
    torch.testing.assert_close(k, apply_rotary_pos_emb(qkv[..., 4 * d:5 * d], freqs))
    torch.testing.assert_close(v, qkv[..., 5 * d:])
    (q.sum() + k.sum() + v.sum()).backward()
    assert qkv.grad.abs().sum() > 0


def test_causal_cross_attention_is_top_left_aligned():
    """'causal' keeps the diagonal at the top-left corner when sq != sk; only '*_bottom_right' moves it."""
    torch.manual_seed(0)
    b, h, sq, sk, d = 1, 2, 4, 7, 8
    q, k, v = torch.randn(sq, b, h, d), torch.randn(sk, b, h, d), torch.randn(sk, b, h, d)
    dpa = te.DotProductAttention(h, d, attention_dropout=0.0, attention_type="cross", qkv_format="sbhd")
    score = torch.einsum("sbhd,tbhd->bhst", q, k) / d ** 0.5
    i, j = torch.arange(sq)[:, None], torch.arange(sk)[None, :]
    for mask_type, allowed in (("causal", j <= i), ("causal_bottom_right", j <= i + (sk - sq))):
        p = torch.softmax(score.masked_fill(~allowed, float("-inf")), dim=-1)
        want = torch.einsum("bhst,tbhd->sbhd", p, v).reshape(sq, b, h * d)
        got = dpa(q, k, v, attn_mask_type=mask_type)
        assert torch.allclose(got, want, atol=1e-5), mask_type


def test_context_parallel_refuses_what_it_does_not_implement(monkeypatch):
    """With a context-parallel group of more than one rank, arguments outside scale / causal / window
    raise instead of being dropped."""
    from transformerengine_b200.parallel import distributed as D

    dpa = te.DotProductAttention(2, 8, attention_dropout=0.0, qkv_format="sbhd")
    dpa.set_context_parallel_group(object(), [0, 1], None, "p2p")
    monkeypatch.setattr(D, "get_world_size", lambda group=None: 2)
    q = torch.randn(4, 1, 2, 8)
    with pytest.raises(NotImplementedError, match="alibi"):
        dpa(q, q, q, core_attention_bias_type="alibi")
    with pytest.raises(NotImplementedError, match="mask"):
        dpa(q, q, q, attn_mask_type="padding", attention_mask=torch.zeros(1, 1, 1, 4, dtype=torch.bool))
    dpa_drop = te.DotProductAttention(2, 8, attention_dropout=0.1, qkv_format="sbhd")
    dpa_drop.set_context_parallel_group(object(), [0, 1], None, "p2p")
    with pytest.raises(NotImplementedError, match="dropout"):
        dpa_drop(q, q, q)
    cu = torch.tensor([0, 4], dtype=torch.int32)
    with pytest.raises(NotImplementedError, match="sliding window"):
        dpa(q.reshape(4, 2, 8), q.reshape(4, 2, 8), q.reshape(4, 2, 8), qkv_format="thd", cu_seqlens_q=cu,
            attn_mask_type="padding_causal", window_size=(2, 0))


@pytest.mark.parametrize("layout", ["grouped", "blocked"])
@pytest.mark.parametrize("fmt", ["sbhd", "bshd"])
def test_rotate_packed_qkv_in_place_matches_separate_rotations(layout, fmt):
    from transformerengine_b200.attention.rope import (RotaryPositionEmbedding, apply_rotary_pos_emb,
                                                       rotate_packed_qkv_)

    torch.manual_seed(0)
    s, b, hq, hk, d = 6, 2, 4, 2, 16
    g = hq // hk
    freqs = RotaryPositionEmbedding(d)(s)
    base = torch.randn((s, b, (hq + 2 * hk) * d) if fmt == "sbhd" else (b, s, (hq + 2 * hk) * d), dtype=torch.float64)
    lead = base.shape[:2]

    def split(m):
        if layout == "grouped":
            m5 = m.reshape(*lead, hk, g + 2, d)
            q, k, v = torch.split(m5, (g, 1, 1), dim=-2)
            return q.reshape(*lead, hq, d), k.reshape(*lead, hk, d), v.reshape(*lead, hk, d)
        q, k, v = torch.split(m, (hq * d, hk * d, hk * d), dim=-1)
        return q.reshape(*lead, hq, d), k.reshape(*lead, hk, d), v.reshape(*lead, hk, d)

    w = torch.randn_like(base)
    a = base.clone().requires_grad_(True)
    q, k, v = split(a * 1.0)
    ref = torch.cat([apply_rotary_pos_emb(q, freqs, fmt).flatten(2), apply_rotary_pos_emb(k, freqs, fmt).flatten(2),
                     v.flatten(2)], dim=-1)
    bt = base.clone().requires_grad_(True)
    mixed = bt * 1.0                                 # a non-leaf the rotation may overwrite
    out = rotate_packed_qkv_(mixed, freqs, freqs, fmt, layout, hq, hk, d)
    assert out.data_ptr() == mixed.data_ptr()        # in place
    view_in = (bt * 1.0).reshape(-1).reshape(base.shape)   # a view: rotated into a new tensor instead
    out_v = rotate_packed_qkv_(view_in, freqs, freqs, fmt, layout, hq, hk, d)
    assert out_v.data_ptr() != view_in.data_ptr()
    torch.testing.assert_close(out_v, out)
    q2, k2, v2 = split(out)
    got = torch.cat([q2.flatten(2), k2.flatten(2), v2.flatten(2)], dim=-1)
    torch.testing.assert_close(got, ref)
    wq = torch.randn_like(ref)
    (ref * wq).sum().backward()
    (got * wq).sum().backward()
    torch.testing.assert_close(bt.grad, a.grad)


def test_bottom_right_diagonal_and_packed_inputs():
    """``bottom_right_diagonal`` picks the corner a sliding window is aligned to when s_q != s_kv (default for
    non-causal masks: bottom right, as in the reference); ``qkv_layer`` / ``kv_layer`` are unpacked as views."""
    torch.manual_seed(0)
    b, h, sq, sk, d = 2, 2, 4, 7, 8
    q, k, v = torch.randn(b, sq, h, d), torch.randn(b, sk, h, d), torch.randn(b, sk, h, d)
    dpa = te.DotProductAttention(h, d, attention_dropout=0.0, qkv_format="bshd", attn_mask_type="no_mask",
                                 attention_type="cross")

    def ref(bottom_right, w):
        s = torch.einsum("bqhd,bkhd->bhqk", q, k) / d ** 0.5
        qi = torch.arange(sq)[:, None] + ((sk - sq) if bottom_right else 0)
        ki = torch.arange(sk)[None]
        p = torch.softmax(s.masked_fill((ki < qi - w[0]) | (ki > qi + w[1]), float("-inf")), -1)
        return torch.einsum("bhqk,bkhd->bqhd", p, v).reshape(b, sq, h * d)

    w = (1, 1)
    torch.testing.assert_close(dpa(q, k, v, window_size=w), ref(True, w))
    torch.testing.assert_close(dpa(q, k, v, window_size=w, bottom_right_diagonal=False), ref(False, w))
    top_left = te.DotProductAttention(h, d, attention_dropout=0.0, qkv_format="bshd", attn_mask_type="no_mask",
                                      attention_type="cross", bottom_right_diagonal=False)
    torch.testing.assert_close(top_left(q, k, v, window_size=w), ref(False, w))
    qkv = torch.randn(b, 5, 3, h, d)
    assert torch.equal(dpa(qkv_layer=qkv, attn_mask_type="causal"),
                       dpa(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], attn_mask_type="causal"))
    kv = torch.randn(b, sk, h, 2, d)
    assert torch.equal(dpa(q, kv_layer=kv, qkv_interleave_dim=-2), dpa(q, kv[..., 0, :], kv[..., 1, :]))
    with pytest.raises(ValueError):
        dpa(q, k, v, kv_layer=kv, qkv_interleave_dim=-2)
    with pytest.raises(ValueError):
        dpa(qkv_layer=qkv, qkv_interleave_dim=-1)
    with pytest.raises(ValueError, match="autocast"):
        dpa(q, k, v, fp8_output=True)


def _fp8_rt(t, dtype):
    """Per-tensor FP8 rounding with the scale of the tensor's own amax (fp32 math)."""
    f = t.float()
    scale = torch.finfo(dtype).max / f.abs().max()
    return ((f * scale).to(dtype).float() / scale).to(t.dtype)


def test_fp8_attention_rounds_the_boundary_tensors():
    """``recipe.fp8_dpa``: Q, K, V (and the output with ``fp8_mha`` / ``fp8_output``) are rounded to the forward FP8
    format, the gradients dO and dQ / dK / dV to the gradient format; without the flags nothing changes."""
    from transformerengine_b200.common import recipe as R
    torch.manual_seed(0)
    dpa = te.DotProductAttention(2, 8, attention_dropout=0.0, qkv_format="bshd", attn_mask_type="causal")
    q, k, v = (torch.randn(2, 6, 2, 8, requires_grad=True) for _ in range(3))
    go = torch.randn(2, 6, 16)
    plain = dpa(q, k, v)
    with te.autocast(enabled=True, recipe=R.DelayedScaling()):
        assert torch.equal(dpa(q, k, v), plain)

    def expected(quantize_out, bwd):
        qq, kk, vv = (t.detach().clone().requires_grad_() for t in (q, k, v))
        e4, e5 = torch.float8_e4m3fn, torch.float8_e5m2
        ste = lambda t: _fp8_rt(t.detach(), e4) + (t - t.detach())  # noqa: E731  (straight-through rounding)
        o = dpa(ste(qq), ste(kk), ste(vv))
        out = _fp8_rt(o.detach(), e4) if quantize_out else o.detach()
        o.backward(_fp8_rt(go, e5) if bwd else go)
        grads = [(_fp8_rt(t.grad, e5) if bwd else t.grad) for t in (qq, kk, vv)]
        return out, grads

    for rec, kw, quantize_out, bwd in ((R.DelayedScaling(fp8_dpa=True), {}, False, True),
                                       (R.Float8CurrentScaling(fp8_dpa=True, fp8_mha=True), {}, True, True),
                                       (R.DelayedScaling(fp8_dpa=True), dict(fp8_output=True, bf16_backward=True),
                                        True, False)):
        for t in (q, k, v):
            t.grad = None
        with te.autocast(enabled=True, recipe=rec):
            o = dpa(q, k, v, **kw)
        o.backward(go)
        want_o, want_g = expected(quantize_out, bwd)
        torch.testing.assert_close(o, want_o, rtol=0, atol=1e-6)
        for t, g in zip((q, k, v), want_g):
            torch.testing.assert_close(t.grad, g, rtol=0, atol=1e-6)
        assert not torch.equal(o, plain)
    # MXFP8 recipes round with 1 x 32 block scales where the shape allows, else with the per-tensor scale
    with te.autocast(enabled=True, recipe=R.MXFP8BlockScaling(fp8_dpa=True)):
        o = dpa(q, k, v)
    assert o.shape == plain.shape and torch.isfinite(o).all() and (o - plain).abs().max() < 0.2
    big = te.DotProductAttention(2, 32, attention_dropout=0.0, qkv_format="bshd")
    x = torch.randn(2, 8, 2, 32)
    with te.autocast(enabled=True, recipe=R.MXFP8BlockScaling(fp8_dpa=True)):
        o = big(x, x, x)
    assert (o - big(x, x, x)).abs().max() < 0.2 and not torch.equal(o, big(x, x, x))


def test_attention_backend_report():
    from transformerengine_b200.attention.utils import AttentionParams, get_attention_backend
    backend, why = get_attention_backend(AttentionParams())
    if not torch.cuda.is_available():
        assert backend == "reference_math" and any("oracle" in w for w in why)
    backend, why = get_attention_backend(AttentionParams(device="cpu", head_dim=64, attention_dropout=0.1))
    assert backend == "reference_math" and why
    assert any("FP8" in w for w in get_attention_backend(AttentionParams(fp8=True))[1])


def test_attention_backend_logging(caplog):
    import logging
    from transformerengine_b200.utils import config as C
    dpa = te.DotProductAttention(2, 8, attention_dropout=0.0, qkv_format="bshd", layer_number=3)
    q = torch.randn(1, 4, 2, 8)
    with C.override(debug=True, debug_level=1), caplog.at_level(logging.DEBUG, logger="DotProductAttention"):
        dpa(q, q, q)
        dpa(q, q, q)                        # the same configuration is reported once
    lines = [r.getMessage() for r in caplog.records if r.name == "DotProductAttention"]
    assert sum("layer 3" in ln for ln in lines) == 1 and any("reference_math" in ln for ln in lines)
    caplog.clear()
    with caplog.at_level(logging.DEBUG, logger="DotProductAttention"):
        dpa(q, q, q)
    assert not [r for r in caplog.records if r.name == "DotProductAttention"]


def test_return_max_logit():
    """``return_max_logit``: per-head maximum of the scaled scores that the mask leaves visible (GQA, causal,
    sliding window, padding mask), computed in blocks of query rows."""
    from transformerengine_b200.ops.attention import max_attention_logit
    torch.manual_seed(0)
    b, sq, h, g, d = 2, 12, 4, 2, 8
    q, k, v = torch.randn(b, sq, h, d), torch.randn(b, sq, g, d), torch.randn(b, sq, g, d)
    scores = torch.einsum("bqhd,bkhd->bhqk", q, k.repeat_interleave(h // g, dim=2)) / d ** 0.5
    qi, ki = torch.arange(sq)[:, None], torch.arange(sq)[None, :]

    def want(masked):
        return scores.masked_fill(masked, float("-inf")).amax(dim=(0, 2, 3))

    dpa = te.DotProductAttention(h, d, num_gqa_groups=g, attention_dropout=0.0, qkv_format="bshd",
                                 attn_mask_type="causal", return_max_logit=True)
    plain = te.DotProductAttention(h, d, num_gqa_groups=g, attention_dropout=0.0, qkv_format="bshd",
                                   attn_mask_type="causal")
    out, mx = dpa(q, k, v)
    assert torch.equal(out, plain(q, k, v)) and mx.shape == (h,) and mx.dtype == torch.float32
    torch.testing.assert_close(mx, want(ki > qi))
    _, mx = dpa(q, k, v, attn_mask_type="no_mask")
    torch.testing.assert_close(mx, want(torch.zeros(sq, sq, dtype=torch.bool)))
    _, mx = dpa(q, k, v, window_size=(3, 0))
    torch.testing.assert_close(mx, want((ki > qi) | (ki < qi - 3)))
    pad = torch.zeros(b, 1, 1, sq, dtype=torch.bool)
    pad[1, ..., 8:] = True
    _, mx = dpa(q, k, v, attn_mask_type="padding", attention_mask=pad)
    full = pad.reshape(b, 1, 1, sq) | pad.reshape(b, 1, sq, 1)
    torch.testing.assert_close(mx, want(full))
    _, mx = dpa(q, k, v, checkpoint_core_attention=True)
    torch.testing.assert_close(mx, want(ki > qi))
    # the blocked pass gives the same maximum whatever the block size
    qb, kb = q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3)
    torch.testing.assert_close(max_attention_logit(qb, kb, causal=True, chunk_bytes=1), want(ki > qi))
    with pytest.raises(NotImplementedError):
        dpa(q.reshape(-1, h, d), k.reshape(-1, g, d), v.reshape(-1, g, d), qkv_format="thd",
            cu_seqlens_q=torch.tensor([0, 12, 24], dtype=torch.int32))
