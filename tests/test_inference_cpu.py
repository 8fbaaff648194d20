"""Incremental decoding through the KV cache reproduces full-sequence causal attention
(test model: reference ``tests/pytorch/attention/test_kv_cache.py``)."""
from collections import OrderedDict

import pytest
import torch

import transformerengine_b200 as te


@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("fmt", ["bshd", "sbhd"])
def test_kv_cache_matches_full_attention(paged, fmt):
    torch.manual_seed(0)
    b, h, hk, d, total = 2, 4, 2, 16, 12
    mha = te.MultiheadAttention(h * d, h, num_gqa_groups=hk, attention_dropout=0.0, attn_mask_type="causal",
                                qkv_format=fmt, bias=False, params_dtype=torch.float32, device="cpu")
    mha.eval()
    rope = te.RotaryPositionEmbedding(d)(total)
    x = torch.randn(b, total, h * d)
    xin = x if fmt == "bshd" else x.transpose(0, 1)
    with torch.no_grad():
        full = mha(xin, rotary_pos_emb=rope)
        full = full if fmt == "bshd" else full.transpose(0, 1)
        params = te.InferenceParams(max_batch_size=4, max_sequence_length=32, num_heads_kv=hk, head_dim_k=d,
                                    dtype=torch.float32, is_paged=paged, page_size=4, total_num_pages=16,
                                    qkv_format=fmt, device="cpu")
        # prefill 5 tokens, then 3 tokens, then one token at a time
        outs, pos = [], 0
        for n in (5, 3, 1, 1, 1, 1):
            params.pre_step(OrderedDict((i, n) for i in range(b)))
            chunk = x[:, pos:pos + n]
            chunk = chunk if fmt == "bshd" else chunk.transpose(0, 1)
            y = mha(chunk, rotary_pos_emb=rope, inference_params=params)
            outs.append(y if fmt == "bshd" else y.transpose(0, 1))
            pos += n
        inc = torch.cat(outs, dim=1)
    assert torch.allclose(inc, full, atol=1e-5), (inc - full).abs().max()


def test_paged_cache_releases_pages_of_finished_sequences():
    m = te.PagedKVCacheManager(total_num_pages=4, page_size=2, num_heads_kv=1, head_dim_k=4, dtype=torch.float32,
                               max_batch_size=2, max_sequence_length=8, device="cpu")
    m.pre_step(OrderedDict([(7, 3), (9, 2)]))
    assert len(m.free_pages) == 1
    k = torch.randn(5, 1, 4)
    kf, vf, lens = m.step(1, k, k, [0, 3, 5])
    assert lens == [3, 2] and torch.equal(kf, k)
    m.post_step()
    m.pre_step(OrderedDict([(9, 1)]))          # sequence 7 finished
    assert 7 not in m.page_table and len(m.free_pages) == 2
    assert m.get_page_table().shape == (1, 2)


def test_paged_cache_queries_and_conversion():
    m = te.PagedKVCacheManager(total_num_pages=6, page_size=2, num_heads_kv=1, head_dim_k=4, dtype=torch.float32,
                               max_batch_size=3, max_sequence_length=8, device="cpu")
    m.allocate_sequence(5, 3)
    assert m.get_sequence_count() == 1 and m.get_page_count(5) == 2 and m.has_free_page()
    assert m.get_page_table([5]).tolist() == [m.get_page_list(5)]
    m.deallocate_sequence(5)
    assert m.get_sequence_count() == 0 and len(m.free_pages) == 6
    for _ in range(6):
        m.allocate_page(1)
    with pytest.raises(RuntimeError, match="full"):
        m.allocate_page(2)
    m.reset()
    assert len(m.free_pages) == 6 and m.get_sequence_lengths() == []

    params = te.InferenceParams(max_batch_size=2, max_sequence_length=8, num_heads_kv=1, head_dim_k=4,
                                dtype=torch.float32, is_paged=True, page_size=2, total_num_pages=8, device="cpu")
    params.pre_step(OrderedDict([(0, 3), (1, 2)]))
    k = torch.arange(5 * 4, dtype=torch.float32).reshape(5, 1, 4)
    params.cache_manager.step(1, k, k + 100, [0, 3, 5])
    kc, vc = params.convert_paged_to_nonpaged(1)
    assert kc.shape == (2, 4, 1, 4)
    assert torch.equal(kc[0, :3], k[:3]) and torch.equal(kc[1, :2], k[3:5]) and torch.equal(vc[0, :3], k[:3] + 100)
    assert "paged" in repr(params)
    params.reset()
    assert params.cache_manager.get_sequence_count() == 0
    flat = te.NonPagedKVCacheManager(2, 8, 1, 4, torch.float32, device="cpu")
    flat.pre_step(OrderedDict([(3, 2)]))
    flat.reset()
    assert not flat.slots and len(flat.free_slots) == 2
