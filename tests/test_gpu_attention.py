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
