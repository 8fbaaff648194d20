"""The library's own tcgen05 fused attention kernels versus the fp32 reference math
(test model: reference ``tests/pytorch/attention/test_attention.py``)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, do, causal, bottom_right):
    from transformerengine_b200.ops.attention import attention_ref

    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    o = attention_ref(qf, kf, vf, causal=causal, bottom_right=bottom_right)
    o.backward(do.float())
    return o, qf.grad, kf.grad, vf.grad


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item()
    assert err <= tol * max(ref, 1e-3), (err, ref)


CASES = [
    # b, hq, hk, sq, sk, causal, bottom_right
    (2, 4, 2, 512, 512, True, True),
    (1, 4, 4, 256, 256, False, True),
    (1, 8, 2, 300, 200, False, True),
    (1, 2, 1, 128, 384, True, True),
    (1, 2, 2, 333, 333, True, True),
    (1, 4, 1, 1024, 1024, True, True),
    (1, 2, 2, 200, 456, True, False),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_flash_matches_reference(case, dtype):
    import transformerengine_b200 as te
    from transformerengine_b200.ops import flash

    b, hq, hk, sq, sk, causal, br = case
    torch.manual_seed(0)
    q = torch.randn(b, hq, sq, 128, device="cuda", dtype=dtype, requires_grad=True)
    k = torch.randn(b, hk, sk, 128, device="cuda", dtype=dtype, requires_grad=True)
    v = torch.randn(b, hk, sk, 128, device="cuda", dtype=dtype, requires_grad=True)
    do = torch.randn(b, hq, sq, 128, device="cuda", dtype=dtype)
    assert flash.supported(q, k, v, causal)
    o = flash.flash_attention(q, k, v, None, causal, br)
    o.backward(do)
    te.ops.check_status()
    ro, rdq, rdk, rdv = _ref(q, k, v, do, causal, br)
    _close(o, ro, 2e-2)
    _close(q.grad, rdq, 3e-2)
    _close(k.grad, rdk, 3e-2)
    _close(v.grad, rdv, 3e-2)


def test_flash_sbhd_views_and_lse():
    """Strided [s, b, h, d] projections are consumed in place; LSE matches the reference."""
    import transformerengine_b200 as te
    from transformerengine_b200.ops import flash
    from transformerengine_b200.ops.attention import attention_ref

    torch.manual_seed(1)
    s, b, hq, hk = 384, 2, 4, 2
    qkv = torch.randn(s, b, (hq + 2 * hk) * 128, device="cuda", dtype=torch.bfloat16)
    q = qkv[..., :hq * 128].reshape(s, b, hq, 128).permute(1, 2, 0, 3)
    k = qkv[..., hq * 128:(hq + hk) * 128].reshape(s, b, hk, 128).permute(1, 2, 0, 3)
    v = qkv[..., (hq + hk) * 128:].reshape(s, b, hk, 128).permute(1, 2, 0, 3)
    assert not q.is_contiguous()
    o, lse = flash.flash_forward_lse(q, k, v, None, True)
    te.ops.check_status()
    ro, rlse = attention_ref(q.float(), k.float(), v.float(), causal=True, return_lse=True)
    _close(o, ro, 2e-2)
    assert (lse - rlse).abs().max().item() < 2e-2
    o2 = flash.flash_attention(q, k, v, None, True, True, "sbhd")
    assert o2.permute(2, 0, 1, 3).is_contiguous()
    _close(o2, ro, 2e-2)


def test_dot_product_attention_uses_own_kernel():
    import transformerengine_b200 as te

    torch.manual_seed(2)
    dpa = te.DotProductAttention(4, 128, num_gqa_groups=2, attn_mask_type="causal", qkv_format="sbhd")
    q = torch.randn(256, 2, 4, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(256, 2, 2, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(256, 2, 2, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    C_ = te.ops._ext.get()
    out = dpa(q, k, v)
    out.float().square().mean().backward()
    te.ops.check_status()
    from transformerengine_b200.ops.attention import attention_ref

    ref = attention_ref(q.detach().permute(1, 2, 0, 3).float(), k.detach().permute(1, 2, 0, 3).float(),
                        v.detach().permute(1, 2, 0, 3).float(), causal=True)
    _close(out.reshape(256, 2, 4, 128).permute(1, 2, 0, 3), ref, 2e-2)
    assert q.grad is not None and torch.isfinite(q.grad.float()).all()
    assert hasattr(C_, "flash_fwd")


VARLEN_CASES = [
    # q lengths, kv lengths (None: same), causal, bottom_right, gaps between sequences (padded offsets)
    ([300, 128, 517, 64, 1], None, True, True, None),
    ([300, 128, 517, 64, 1], None, False, True, None),
    ([100, 260], [356, 260], True, True, None),
    ([256, 40, 0, 129], None, True, True, [3, 0, 5, 2]),
]


@pytest.mark.parametrize("case", VARLEN_CASES)
def test_flash_varlen_matches_per_sequence_reference(case):
    """Packed sequences in one launch versus the fp32 reference run sequence by sequence."""
    import transformerengine_b200 as te
    from transformerengine_b200.ops import flash

    lq, lk, causal, br, gaps = case
    lk = lk or lq
    gaps = gaps or [0] * len(lq)
    hq, hk = 4, 2

    def offsets(lens):
        cu, off, pos = [0], [], 0
        for n, g in zip(lens, gaps):
            off.append(pos)
            pos += n + g
            cu.append(cu[-1] + n)
        off.append(pos)
        return cu, off

    cu_q, off_q = offsets(lq)
    cu_k, off_k = offsets(lk)
    torch.manual_seed(0)
    q = torch.randn(off_q[-1], hq, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(off_k[-1], hk, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(off_k[-1], hk, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    do = torch.randn_like(q)
    assert flash.supported_varlen(q, k, v)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    padded = any(gaps)
    o = flash.flash_attention_varlen(q, k, v, t(cu_q), t(cu_k), None, causal, br,
                                     cu_seqlens_q_padded=t(off_q) if padded else None,
                                     cu_seqlens_kv_padded=t(off_k) if padded else None)
    o.backward(do)
    te.ops.check_status()
    ro, rdq, rdk, rdv = (torch.zeros_like(x, dtype=torch.float32) for x in (q, q, k, v))
    for i in range(len(lq)):
        if lq[i] == 0:
            continue
        sq, sk = slice(off_q[i], off_q[i] + lq[i]), slice(off_k[i], off_k[i] + lk[i])
        bh = lambda x: x.detach().permute(1, 0, 2).unsqueeze(0)
        r = _ref(bh(q[sq]), bh(k[sk]), bh(v[sk]), bh(do[sq]), causal, br)
        ro[sq], rdq[sq], rdk[sk], rdv[sk] = (x.squeeze(0).permute(1, 0, 2) for x in r)
    _close(o, ro, 2e-2)
    _close(q.grad, rdq, 3e-2)
    _close(k.grad, rdk, 3e-2)
    _close(v.grad, rdv, 3e-2)


def test_dot_product_attention_thd_uses_varlen_kernel():
    import transformerengine_b200 as te

    lens = [200, 312]
    cu = torch.tensor([0, 200, 512], dtype=torch.int32, device="cuda")
    attn = te.DotProductAttention(4, 128, num_gqa_groups=2, qkv_format="thd", attn_mask_type="padding_causal").cuda()
    torch.manual_seed(1)
    q = torch.randn(512, 4, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(512, 2, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(512, 2, 128, device="cuda", dtype=torch.bfloat16)
    o = attn(q, k, v, cu_seqlens_q=cu, cu_seqlens_kv=cu, max_seqlen_q=312, max_seqlen_kv=312)
    te.ops.check_status()
    assert o.shape == (512, 4 * 128)
    from transformerengine_b200.ops.attention import attention_ref

    pos = 0
    for n in lens:
        bh = lambda x: x[pos:pos + n].float().permute(1, 0, 2).unsqueeze(0)
        r = attention_ref(bh(q), bh(k), bh(v), causal=True).squeeze(0).permute(1, 0, 2).reshape(n, -1)
        _close(o[pos:pos + n], r, 2e-2)
        pos += n


WINDOW_CASES = [
    # b, hq, hk, sq, sk, causal, bottom_right, (left, right)
    (1, 4, 2, 1024, 1024, True, True, (256, 0)),
    (2, 2, 2, 512, 512, True, True, (100, 0)),
    (1, 4, 1, 700, 700, False, True, (64, 32)),
    (1, 2, 2, 300, 556, True, True, (128, 0)),
    (1, 2, 1, 512, 512, False, True, (-1, 17)),
    (1, 4, 1, 8192, 8192, True, True, (1024, 0)),
]


@pytest.mark.parametrize("case", WINDOW_CASES)
def test_flash_sliding_window_matches_reference(case):
    import transformerengine_b200 as te
    from transformerengine_b200.ops import flash
    from transformerengine_b200.ops.attention import attention_ref

    b, hq, hk, sq, sk, causal, br, window = case
    torch.manual_seed(0)
    dtype = torch.bfloat16
    q = torch.randn(b, hq, sq, 128, device="cuda", dtype=dtype, requires_grad=True)
    k = torch.randn(b, hk, sk, 128, device="cuda", dtype=dtype, requires_grad=True)
    v = torch.randn(b, hk, sk, 128, device="cuda", dtype=dtype, requires_grad=True)
    do = torch.randn(b, hq, sq, 128, device="cuda", dtype=dtype)
    o = flash.flash_attention(q, k, v, None, causal, br, window=window)
    o.backward(do)
    te.ops.check_status()
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ro = attention_ref(qf, kf, vf, causal=causal, window=window, bottom_right=br)
    ro.backward(do.float())
    _close(o, ro, 2e-2)
    _close(q.grad, qf.grad, 3e-2)
    _close(k.grad, kf.grad, 3e-2)
    _close(v.grad, vf.grad, 3e-2)


def test_flash_varlen_with_sliding_window():
    import transformerengine_b200 as te
    from transformerengine_b200.ops import flash
    from transformerengine_b200.ops.attention import attention_ref

    lens, window = [400, 130, 700], (96, 0)
    cu = [0, 400, 530, 1230]
    torch.manual_seed(0)
    q = torch.randn(cu[-1], 4, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(cu[-1], 2, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(cu[-1], 2, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    do = torch.randn_like(q)
    cut = torch.tensor(cu, dtype=torch.int32, device="cuda")
    o = flash.flash_attention_varlen(q, k, v, cut, cut, None, True, True, window=window)
    o.backward(do)
    te.ops.check_status()
    bh = lambda x: x.permute(1, 0, 2).unsqueeze(0)  # noqa: E731
    for a, b in zip(cu[:-1], cu[1:]):
        qf, kf, vf = (bh(t[a:b].detach().float()).requires_grad_() for t in (q, k, v))
        ro = attention_ref(qf, kf, vf, causal=True, window=window)
        ro.backward(bh(do[a:b].float()))
        _close(bh(o[a:b]), ro, 2e-2)
        _close(bh(q.grad[a:b]), qf.grad, 3e-2)
        _close(bh(k.grad[a:b]), kf.grad, 3e-2)
        _close(bh(v.grad[a:b]), vf.grad, 3e-2)
