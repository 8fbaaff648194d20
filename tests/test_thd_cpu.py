"""Packed-sequence helpers, PyTorch path: context-parallel partitioning and the merging of partial
attention results must reproduce attention over the whole sequences
(test model: reference ``tests/pytorch/attention/test_attention_with_cp.py`` for the thd format)."""
import torch

from transformerengine_b200.attention import thd
from transformerengine_b200.ops.attention import attention_ref


def test_partition_indices_cover_every_token_once():
    cu = torch.tensor([0, 8, 24, 32], dtype=torch.int32)
    world = 2
    parts = [thd.thd_get_partitioned_indices(cu, 32, world, r) for r in range(world)]
    assert sorted(torch.cat(parts).tolist()) == list(range(32))
    # rank 0 of sequence 0 (8 tokens, chunks of 2): chunks 0 and 3
    assert parts[0][:4].tolist() == [0, 1, 6, 7]
    assert parts[1][:4].tolist() == [2, 3, 4, 5]


def test_half_tensor_lse_and_out_correction_merge_two_partial_attentions():
    """Split the keys in two, attend to each part, merge with the thd helpers == full attention."""
    torch.manual_seed(0)
    cu = torch.tensor([0, 6, 16], dtype=torch.int32)
    t, h, d = 16, 2, 8
    q, k, v = torch.randn(t, h, d), torch.randn(t, h, d), torch.randn(t, h, d)

    def attend(qs, ks, vs):
        bh = lambda x: x.permute(1, 0, 2).unsqueeze(0)  # noqa: E731
        o, lse = attention_ref(bh(qs), bh(ks), bh(vs), return_lse=True)
        return o.squeeze(0).permute(1, 0, 2), lse.squeeze(0)

    full = torch.zeros(t, h, d)
    o1, o2 = torch.zeros(t, h, d), torch.zeros(t, h, d)
    l1, l2 = torch.zeros(h, t), torch.zeros(h, t)
    for a, b in zip(cu[:-1].tolist(), cu[1:].tolist()):
        m = (a + b) // 2
        full[a:b] = attend(q[a:b], k[a:b], v[a:b])[0]
        o1[a:b], l1[:, a:b] = attend(q[a:b], k[a:m], v[a:m])
        o2[a:b], l2[:, a:b] = attend(q[a:b], k[m:b], v[m:b])
    lse = torch.logaddexp(l1, l2)
    out = torch.zeros(t, h, d)
    thd.thd_out_correction(out, o1, lse, l1, cu, False)
    thd.thd_out_correction(out, o2, lse, l2, cu, False)
    torch.testing.assert_close(out, full, rtol=1e-5, atol=1e-5)

    # second-half-only variants
    half_q = thd.thd_read_half_tensor(q, cu, 1)
    assert half_q.shape == (8, h, d)
    torch.testing.assert_close(half_q[:3], q[3:6])
    torch.testing.assert_close(half_q[3:], q[11:16])
    stacked = torch.stack([k, v])
    torch.testing.assert_close(thd.thd_read_half_tensor(stacked, cu, 0)[1, :3], v[0:3])
    lse_b = l1.clone()
    half_l2 = thd.thd_read_second_half_lse(l2, cu)
    thd.thd_second_half_lse_correction(lse_b, half_l2, cu)
    torch.testing.assert_close(lse_b[:, 3:6], lse[:, 3:6])
    torch.testing.assert_close(lse_b[:, 0:3], l1[:, 0:3])
    out_b = torch.zeros(t, h, d)
    thd.thd_out_correction(out_b, thd.thd_read_half_tensor(o2, cu, 1), lse, half_l2, cu, True)
    torch.testing.assert_close(out_b[3:6], o2[3:6] * torch.exp(l2 - lse)[:, 3:6].t().unsqueeze(-1))
    assert out_b[0:3].abs().max() == 0


def test_grad_correction_modes():
    cu = torch.tensor([0, 4, 10], dtype=torch.int32)
    g = torch.ones(10, 3)
    step = torch.full((10, 3), 2.0)
    thd.thd_grad_correction(g, step, cu, "add", "copy")
    assert g[0:2].eq(3).all() and g[2:4].eq(2).all() and g[4:7].eq(3).all() and g[7:10].eq(2).all()
    g = torch.ones(2, 10, 1, 3)
    half = torch.arange(5, dtype=torch.float32).reshape(1, 5, 1, 1).expand(2, 5, 1, 3).contiguous()
    thd.thd_grad_correction(g, half, cu, "none", "add")
    assert g[:, 0:2].eq(1).all() and g[0, 2, 0, 0] == 1 and g[0, 3, 0, 0] == 2 and g[1, 7, 0, 0] == 3 and g[1, 9, 0, 0] == 5


def test_thd_bshd_round_trip_and_kv_cache_step():
    cu = torch.tensor([0, 3, 8], dtype=torch.int32)
    x = torch.randn(8, 2, 4)
    padded = thd.convert_thd_to_bshd(x, cu, 3, 6)
    assert padded.shape == (3, 6, 2, 4) and padded[0, 3:].abs().max() == 0 and padded[2].abs().max() == 0
    torch.testing.assert_close(thd.convert_bshd_to_thd(padded, cu, 8), x)

    # paged cache, page size 4: sequence 0 holds 5 tokens (pages 7, 2) and gets 1; sequence 1 is new with 3
    ck, cv = torch.zeros(8, 4, 2, 4), torch.zeros(8, 4, 2, 4)
    old = torch.randn(5, 2, 4)
    ck[7], ck[2, 0] = old[:4], old[4]
    cv[7], cv[2, 0] = -old[:4], -old[4]
    new_k = torch.randn(4, 2, 4)
    pt = torch.tensor([[7, 2], [5, -1]], dtype=torch.int32)
    k, v = thd.kv_cache_step(new_k, -new_k, ck, cv, pt, torch.tensor([0, 1, 4], dtype=torch.int32),
                             torch.tensor([0, 6, 9], dtype=torch.int32), 9)
    torch.testing.assert_close(k, torch.cat([old, new_k[:1], new_k[1:]]))
    torch.testing.assert_close(v, -k)
    torch.testing.assert_close(ck[2, 1], new_k[0])
    torch.testing.assert_close(ck[5, :3], new_k[1:])


def test_sequence_order_and_cp_rank_order_round_trip():
    cu = torch.tensor([0, 8, 24, 32], dtype=torch.int32)
    x = torch.arange(32, dtype=torch.float32).reshape(32, 1)
    r = thd.thd_sequence_order_to_cp_rank_order(x, cu, 2, 32)
    # the first half is rank 0's shard: chunks 0 and 3 of every sequence
    assert r[:4, 0].tolist() == [0, 1, 6, 7] and r[16:20, 0].tolist() == [2, 3, 4, 5]
    back = thd.thd_reorder_between_sequence_and_cp_rank_order(r, cu, 2, True, 32)
    assert torch.equal(back, x)
