"""Packed-sequence kernels (``csrc/misc/thd.cu``) versus the PyTorch path of the same functions."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cu(lens):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    return torch.tensor(cu, dtype=torch.int32)


def test_thd_kernels_match_pytorch_path():
    import transformerengine_b200 as te
    from transformerengine_b200.attention import thd

    torch.manual_seed(0)
    lens = [8, 120, 16, 248]
    cu = _cu(lens)
    t, h, d = int(cu[-1]), 4, 64
    cud = cu.cuda()
    for world in (1, 2, 4):
        for r in range(world):
            assert thd.thd_get_partitioned_indices(cud, t, world, r).cpu().tolist() == \
                thd.thd_get_partitioned_indices(cu, t, world, r).tolist()
    for dt in (torch.bfloat16, torch.float32):
        x = torch.randn(t, h, d).to(dt)
        kv = torch.randn(2, t, h, d).to(dt)
        for half in (0, 1):
            assert torch.equal(thd.thd_read_half_tensor(x.cuda(), cud, half).cpu(), thd.thd_read_half_tensor(x, cu, half))
            assert torch.equal(thd.thd_read_half_tensor(kv.cuda(), cud, half).cpu(), thd.thd_read_half_tensor(kv, cu, half))
        lse, lse_s = torch.randn(h, t) + 3, torch.randn(h, t) + 3
        for second in (False, True):
            step = torch.randn(t // 2 if second else t, h, d).to(dt)
            ls = thd.thd_read_second_half_lse(lse_s, cu) if second else lse_s
            out_c, out_g = x.clone(), x.clone().cuda()
            thd.thd_out_correction(out_c, step, lse, ls, cu, second)
            thd.thd_out_correction(out_g, step.cuda(), lse.cuda(), ls.cuda(), cud, second)
            torch.testing.assert_close(out_g.cpu().float(), out_c.float(), rtol=2e-2, atol=2e-2)
        for modes, ts in ((("add", "copy"), t), (("none", "add"), t // 2), (("copy", "none"), t // 2)):
            g_c = kv.clone()
            g_g = kv.clone().cuda()
            step = torch.randn(2, ts, h, d).to(dt)
            thd.thd_grad_correction(g_c, step, cu, *modes)
            thd.thd_grad_correction(g_g, step.cuda(), cud, *modes)
            torch.testing.assert_close(g_g.cpu().float(), g_c.float(), rtol=1e-2, atol=1e-2)
    a, b = torch.randn(h, t), torch.randn(h, t // 2)
    assert torch.equal(thd.thd_read_second_half_lse(a.cuda(), cud).cpu(), thd.thd_read_second_half_lse(a, cu))
    a_g = a.clone().cuda()
    thd.thd_second_half_lse_correction(a_g, b.cuda(), cud)
    thd.thd_second_half_lse_correction(a, b, cu)
    torch.testing.assert_close(a_g.cpu(), a, rtol=1e-5, atol=1e-5)
    x = torch.randn(t, h, d, dtype=torch.bfloat16)
    pad_g = thd.convert_thd_to_bshd(x.cuda(), cud, 5, 248)
    assert torch.equal(pad_g.cpu(), thd.convert_thd_to_bshd(x, cu, 5, 248))
    assert torch.equal(thd.convert_bshd_to_thd(pad_g, cud, t + 8).cpu()[:t], x)
    te.ops.check_status()


@pytest.mark.parametrize("paged", [False, True])
def test_kv_cache_step_kernel(paged):
    import transformerengine_b200 as te
    from transformerengine_b200.attention import thd

    torch.manual_seed(1)
    h, d = 2, 128
    olds, news = [70, 0, 129], [1, 33, 2]
    if paged:
        ps, pages = 64, 16
        tables, free = [], list(range(pages))[::-1]
        for o, n in zip(olds, news):
            tables.append([free.pop() for _ in range(-(-(o + n) // ps))])
        width = max(len(x) for x in tables)
        pt = torch.tensor([x + [-1] * (width - len(x)) for x in tables], dtype=torch.int32)
    else:
        ps, pages = 256, 4
        pt = torch.tensor([[2], [0], [3]], dtype=torch.int32)
    ck = torch.randn(pages, ps, h, d, dtype=torch.bfloat16)
    cv = torch.randn(pages, ps, h, d, dtype=torch.bfloat16)
    new_k = torch.randn(sum(news), h, d, dtype=torch.bfloat16)
    new_v = torch.randn(sum(news), h, d, dtype=torch.bfloat16)
    cu_new, cu_kv = _cu(news), _cu([o + n for o, n in zip(olds, news)])
    total = int(cu_kv[-1])
    ck_g, cv_g = ck.cuda(), cv.cuda()
    k_g, v_g = thd.kv_cache_step(new_k.cuda(), new_v.cuda(), ck_g, cv_g, pt.cuda(), cu_new.cuda(), cu_kv.cuda(), total)
    k_c, v_c = thd.kv_cache_step(new_k, new_v, ck, cv, pt, cu_new, cu_kv, total)
    te.ops.check_status()
    assert torch.equal(k_g.cpu(), k_c) and torch.equal(v_g.cpu(), v_c)
    assert torch.equal(ck_g.cpu(), ck) and torch.equal(cv_g.cpu(), cv)
