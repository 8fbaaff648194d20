"""MoE router, permutation, GroupedLinear, and expert parallelism (gloo) on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import transformerengine_b200 as te
from transformerengine_b200.common import recipe as R
from transformerengine_b200.models import mixtral
from transformerengine_b200.modules.grouped_linear import GroupedLinear
from transformerengine_b200.moe import (fused_compute_score_for_moe_aux_loss, fused_moe_aux_loss,
                                        fused_topk_with_score_function, moe_permute, moe_permute_with_probs,
                                        moe_sort_chunks_by_index, moe_unpermute)


@pytest.mark.parametrize("score", ["softmax", "sigmoid", "sqrtsoftplus"])
@pytest.mark.parametrize("pre", [False, True])
def test_router_topk(score, pre):
    T, E, k = 32, 16, 4
    logits = torch.randn(T, E)
    bias = torch.randn(E) * 0.1 if score != "softmax" else None
    probs, rmap = fused_topk_with_score_function(logits, k, pre, None, None, 2.0, score, bias)
    assert rmap.sum(-1).eq(k).all() and ((probs != 0) == rmap).all()
    if score == "softmax" and not pre:
        ref = torch.softmax(logits.topk(k).values, -1) * 2.0
        assert torch.allclose(probs.gather(1, logits.topk(k).indices), ref, atol=1e-6)
    if score == "sigmoid":
        sel = (torch.sigmoid(logits) + bias).topk(k).indices
        assert torch.equal(rmap, torch.zeros(T, E, dtype=torch.bool).scatter_(1, sel, True))
        assert torch.allclose(probs.sum(-1), torch.full((T,), 2.0), atol=1e-5)  # renormalised, then scaled


def test_router_group_limited_and_bitmap():
    logits = torch.randn(16, 16)
    probs, rmap = fused_topk_with_score_function(logits, 4, True, 4, 2, None, "softmax", None)
    groups_used = rmap.reshape(16, 4, 4).any(-1).sum(-1)
    assert (groups_used <= 2).all()
    _, bm = fused_topk_with_score_function(logits, 4, True, None, None, None, "softmax", None, "bitmap_u8")
    assert bm.dtype == torch.uint8 and bm.shape == (16, 2)


def test_aux_loss_formula():
    T, E, k = 64, 8, 2
    logits = torch.randn(T, E, requires_grad=True)
    rmap, scores = fused_compute_score_for_moe_aux_loss(logits, k, "softmax")
    tpe = rmap.sum(0)
    loss = fused_moe_aux_loss(scores, tpe, T, E, topk=k, coeff=0.01)
    ref = (scores.sum(0) * tpe).sum() * E * 0.01 / (k * T * T)
    assert torch.allclose(loss, ref)
    loss.backward()
    assert logits.grad.abs().sum() > 0


def test_permute_roundtrip_mask_and_index():
    T, E, H, k = 48, 8, 16, 2
    x = torch.randn(T, H, requires_grad=True)
    logits = torch.randn(T, E)
    probs, rmap = fused_topk_with_score_function(logits, k, False, None, None, None, "softmax", None)
    out, rid = moe_permute(x, rmap, T * k)
    # expert-major and stable
    counts = rmap.sum(0)
    off = 0
    for e in range(E):
        toks = rmap[:, e].nonzero().squeeze(1)
        assert torch.equal(out[off:off + counts[e]], x[toks])
        off += int(counts[e])
    y = moe_unpermute(out, rid, merging_probs=probs)
    assert torch.allclose(y, x * probs.sum(-1, keepdim=True), atol=1e-6)
    y.sum().backward()
    assert torch.allclose(x.grad, probs.sum(-1, keepdim=True).expand_as(x), atol=1e-6)
    idx = logits.topk(k).indices.int()
    out2, rid2 = moe_permute(x, idx, 0, map_type="index")
    y2 = moe_unpermute(out2, rid2, map_type="index")
    assert torch.allclose(y2, x * k, atol=1e-5)
    chunks = moe_sort_chunks_by_index(torch.arange(10.)[:, None], torch.tensor([2, 3, 5]), torch.tensor([2, 0, 1]))
    assert chunks.squeeze(1).tolist() == [5., 6., 7., 8., 9., 0., 1., 2., 3., 4.]


def test_mixtral_tiny_trains():
    torch.manual_seed(0)
    cfg = mixtral.MixtralConfig.tiny(params_dtype=torch.float32)
    m = mixtral.MixtralModel(cfg, device="cpu")
    tok = torch.randint(0, cfg.vocab_size, (2, 32))
    loss = m(tok, labels=tok)
    loss.backward()
    assert torch.isfinite(loss)
    assert m.layers[0].moe.router.weight.grad.abs().sum() > 0
    assert m.layers[0].moe.fc1.weight0.grad is not None
    with te.autocast(enabled=True, recipe=R.MXFP8BlockScaling()):
        l2 = m(tok, labels=tok)
    assert abs(l2.item() - loss.item()) < 0.1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ep_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = mixtral.MixtralConfig.tiny(params_dtype=torch.float32, num_layers=1)
        torch.manual_seed(0)
        full = mixtral.MoELayer(cfg, None, "cpu")
        torch.manual_seed(0)
        ep = mixtral.MoELayer(cfg, dist.group.WORLD, "cpu")
        le = cfg.num_experts // world
        with torch.no_grad():
            ep.router.weight.copy_(full.router.weight)
            for i in range(le):
                getattr(ep.fc1, f"weight{i}").copy_(getattr(full.fc1, f"weight{rank * le + i}"))
                getattr(ep.fc2, f"weight{i}").copy_(getattr(full.fc2, f"weight{rank * le + i}"))
        torch.manual_seed(10 + rank)
        x = torch.randn(24, cfg.hidden_size, requires_grad=True)
        y, aux = ep(x)
        (y.sum() + aux).backward()
        xr = x.detach().clone().requires_grad_(True)
        yr, _ = full(xr)
        yr.sum().backward()
        err = ((y - yr).norm() / yr.norm()).item()
        gerr = ((x.grad - xr.grad).norm() / xr.grad.norm()).item()
        q.put((rank, {} if err < 1e-5 and gerr < 2e-2 else {"out": err, "dx": gerr}))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, {"exception": traceback.format_exc()[-1500:]}))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_matches_local():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, bad in res:
        assert not bad, f"rank {rank}: {bad}"


def test_router_quantile_balancing_histogram_and_map_formats():
    """The QB histogram counts, per expert, the bias that expert would have needed to enter each token's top-k
    (cutoff - raw sigmoid score) in uniform bins; routing itself is the usual biased-sigmoid top-k."""
    from transformerengine_b200.router import (QBHistogramMode, RoutingMapFormat, fused_compute_score_for_moe_aux_loss,
                                               fused_topk_with_score_function)
    torch.manual_seed(0)
    T, E, k, bins = 37, 10, 3, 8
    logits = torch.randn(T, E, requires_grad=True)
    bias = torch.randn(E) * 0.2
    hist = torch.zeros(E, bins, dtype=torch.int32)
    bounds = torch.tensor([-0.5, 0.5])
    probs, rmap = fused_topk_with_score_function(logits, k, False, None, None, 1.5, "sigmoid", bias,
                                                 qb_histogram=hist, qb_bin_bounds=bounds,
                                                 qb_histogram_mode="fused_atomic")
    ref_probs, ref_map = fused_topk_with_score_function(logits, k, False, None, None, 1.5, "sigmoid", bias)
    assert torch.equal(rmap, ref_map)
    torch.testing.assert_close(probs, ref_probs)
    want = torch.zeros(E, bins, dtype=torch.int32)
    raw = torch.sigmoid(logits.detach())
    for t in range(T):
        cutoff = (raw[t] + bias).sort(descending=True).values[k]
        for e in range(E):
            b = int(torch.floor((cutoff - raw[t, e] + 0.5) * bins / 1.0))
            want[e, min(max(b, 0), bins - 1)] += 1
    assert torch.equal(hist, want) and int(hist.sum()) == T * E
    # accumulates in place; both mode names give the same counts
    fused_topk_with_score_function(logits, k, False, None, None, 1.5, "sigmoid", bias, qb_histogram=hist,
                                   qb_bin_bounds=bounds, qb_histogram_mode="two_kernel")
    assert torch.equal(hist, 2 * want)
    probs.sum().backward()
    assert logits.grad is not None and torch.isfinite(logits.grad).all()
    for bad in (dict(score_function="softmax"), dict(expert_bias=None), dict(num_groups=2, group_topk=1),
                dict(qb_histogram_mode="other"), dict(qb_bin_bounds=torch.tensor([1.0, 0.0]))):
        kw = dict(logits=logits, topk=k, use_pre_softmax=False, num_groups=None, group_topk=None, scaling_factor=None,
                  score_function="sigmoid", expert_bias=bias, qb_histogram=hist, qb_bin_bounds=bounds,
                  qb_histogram_mode="two_kernel")
        kw.update(bad)
        with pytest.raises(ValueError):
            fused_topk_with_score_function(**kw)
    with pytest.raises(ValueError):
        fused_topk_with_score_function(logits, k, qb_histogram=hist)
    # routing map formats: enum, int and string spellings; bit e % 8 of byte e // 8
    _, packed = fused_topk_with_score_function(logits, k, routing_map_format=RoutingMapFormat.BITMAP_U8)
    _, plain = fused_topk_with_score_function(logits, k, routing_map_format=0)
    assert packed.dtype == torch.uint8 and packed.shape == (T, 2)
    unpacked = torch.stack([(packed[:, e // 8] >> (e % 8)) & 1 for e in range(E)], dim=1).bool()
    assert torch.equal(unpacked, plain)
    m2, _ = fused_compute_score_for_moe_aux_loss(logits, k, "sigmoid", routing_map_format="bitmap_u8")
    assert m2.shape == (T, 2) and m2.dtype == torch.uint8
    assert int(QBHistogramMode.FUSED_ATOMIC) == 1
    with pytest.raises(ValueError):
        fused_topk_with_score_function(logits, k, routing_map_format="BITMAP")


def _ep_buffer_worker(rank, world, port, q):
    import os
    import torch.distributed as dist
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import transformerengine_b200 as te
        E, K, T, H, align = 4, 2, 10, 16, 4
        L = E // world
        te.ep_bootstrap(dist.group.WORLD, num_experts=E, max_tokens_per_rank=T, hidden_dim=H, num_topk=K)
        assert te.is_ep_bootstrapped()
        buf = te.EpBuffer(K, T, H, L, alignment=align, payload_dtype=torch.float32)
        torch.manual_seed(10 + rank)
        x = torch.randn(T, H, requires_grad=True)
        logits = torch.randn(T, E)
        w, idx = torch.softmax(logits, -1).topk(K, dim=-1)
        w = w.clone().requires_grad_()
        counts = te.ep_prepare(buf, idx)
        recv, recv_w, tpe = te.ep_dispatch(buf, x, idx, w)
        assert torch.equal(tpe, counts) and int(buf.total_recv_tokens) == recv.shape[0] == int(tpe.sum())
        assert (tpe % align == 0).all() and recv_w.shape == (recv.shape[0],)
        # "experts": expert e of this rank multiplies by (global expert id + 1); weights applied by the caller
        scale = torch.cat([torch.full((int(n),), float(rank * L + e + 1)) for e, n in enumerate(tpe.tolist())])
        out = te.ep_combine(buf, recv * (scale * recv_w)[:, None])
        x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
        want = x2 * sum(w2[:, k:k + 1] * (idx[:, k:k + 1] + 1).float() for k in range(K))
        err = float((out - want).abs().max())
        out.square().sum().backward()
        want.square().sum().backward()
        gerr = max(float((x.grad - x2.grad).abs().max()), float((w.grad - w2.grad).abs().max()))
        q.put((rank, err, gerr, None))
        te.ep_finalize()
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, None, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_expert_parallel_buffer_api_over_gloo():
    """The reference-style buffer API (bootstrap, EpBuffer, prepare / dispatch / combine) on two gloo ranks: every
    token's expert outputs come back summed, rows arrive grouped by local expert and padded to the alignment."""
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ep_buffer_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, err, gerr, tb in res:
        assert tb is None, tb
        assert err < 1e-5 and gerr < 1e-4, (rank, err, gerr)
