"""Context-parallel attention over gloo ranks versus full-sequence attention on one rank
(test model: reference ``tests/pytorch/attention/test_attention_with_cp.py``)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, comm, causal, result_q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from transformerengine_b200.ops.attention import attention_ref
        from transformerengine_b200.parallel.context_parallel import (attn_forward_func_with_cp,
                                                                      get_batch_on_this_cp_rank)

        torch.manual_seed(0)
        b, hq, hk, s, d = 2, 4, 2, 32, 16
        q = torch.randn(b, hq, s, d, dtype=torch.float64)
        k = torch.randn(b, hk, s, d, dtype=torch.float64)
        v = torch.randn(b, hk, s, d, dtype=torch.float64)
        do = torch.randn(b, hq, s, d, dtype=torch.float64)
        qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
        ref = attention_ref(qf, kf, vf, causal=causal)
        ref.backward(do)

        def shard(t):
            if causal:
                return get_batch_on_this_cp_rank(t, world, rank, seq_dim=2).contiguous()
            return t.chunk(world, dim=2)[rank].contiguous()

        ql, kl, vl = (shard(t).clone().requires_grad_() for t in (q, k, v))
        out = attn_forward_func_with_cp(ql, kl, vl, cp_group=dist.group.WORLD, cp_comm_type=comm, causal=causal)
        out.backward(shard(do))
        errs = [
            (out - shard(ref.detach())).abs().max().item(),
            (ql.grad - shard(qf.grad)).abs().max().item(),
            (kl.grad - shard(kf.grad)).abs().max().item(),
            (vl.grad - shard(vf.grad)).abs().max().item(),
        ]
        result_q.put((rank, max(errs), None))
    except Exception as e:  # noqa: BLE001
        import traceback

        result_q.put((rank, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("comm", ["p2p", "all_gather", "a2a"])
@pytest.mark.parametrize("causal", [True, False])
def test_cp_matches_single_rank(comm, causal):
    world = 2
    ctx = mp.get_context("spawn")
    result_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, comm, causal, result_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [result_q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    for rank, err, tb in results:
        assert tb is None, tb
        assert err < 2e-5, (rank, err)


def test_dual_chunk_layout():
    from transformerengine_b200.parallel.context_parallel import (dual_chunk_positions, get_batch_on_this_cp_rank,
                                                                  pad_thd_sequences_for_cp)

    x = torch.arange(16)[None, :]
    got = get_batch_on_this_cp_rank(x, 4, 1, seq_dim=1)
    assert got.tolist() == [[2, 3, 12, 13]]
    assert dual_chunk_positions(4, 4, 1).tolist() == [2, 3, 12, 13]
    cu = torch.tensor([0, 5, 13])
    assert pad_thd_sequences_for_cp(cu, 2).tolist() == [0, 8, 16]


def _hier_worker(rank, world, port, result_q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from transformerengine_b200.ops.attention import attention_ref
        from transformerengine_b200.parallel.context_parallel import (attn_forward_func_with_cp,
                                                                      get_batch_on_this_cp_rank)

        a2a_groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
        p2p_groups = [dist.new_group([0, 2]), dist.new_group([1, 3])]
        groups = [a2a_groups[rank // 2], p2p_groups[rank % 2]]
        torch.manual_seed(0)
        b, hq, hk, s, d = 1, 4, 2, 64, 16
        q = torch.randn(b, hq, s, d, dtype=torch.float64)
        k = torch.randn(b, hk, s, d, dtype=torch.float64)
        v = torch.randn(b, hk, s, d, dtype=torch.float64)
        do = torch.randn(b, hq, s, d, dtype=torch.float64)
        errs = []
        for causal, window in ((True, None), (False, None), (True, (12, 0))):
            qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
            ref = attention_ref(qf, kf, vf, causal=causal, window=window)
            ref.backward(do)
            if causal:      # dual-chunk shards
                shard = lambda t: get_batch_on_this_cp_rank(t, world, rank, seq_dim=2).contiguous()  # noqa: E731
            else:           # contiguous shards
                shard = lambda t: t.chunk(world, dim=2)[rank].contiguous()  # noqa: E731
            ql, kl, vl = (shard(t).clone().requires_grad_() for t in (q, k, v))
            out = attn_forward_func_with_cp(ql, kl, vl, cp_group=groups, cp_comm_type="a2a+p2p", causal=causal,
                                            window=window)
            out.backward(shard(do))
            errs += [(out - shard(ref.detach())).abs().max().item(), (ql.grad - shard(qf.grad)).abs().max().item(),
                     (kl.grad - shard(kf.grad)).abs().max().item(), (vl.grad - shard(vf.grad)).abs().max().item()]
        result_q.put((rank, max(errs), None))
    except Exception:  # noqa: BLE001
        import traceback

        result_q.put((rank, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_hierarchical_cp_matches_single_rank():
    world = 4
    ctx = mp.get_context("spawn")
    result_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_hier_worker, args=(r, world, port, result_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [result_q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    for rank, err, tb in results:
        assert tb is None, tb
        assert err < 2e-5, (rank, err)


def _thd_worker(rank, world, port, causal, result_q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from transformerengine_b200.attention import thd
        from transformerengine_b200.ops.attention import attention_ref
        from transformerengine_b200.parallel.context_parallel import attn_forward_func_with_cp

        torch.manual_seed(0)
        lens = [8, 24, 16]
        cu = torch.tensor([0, 8, 32, 48], dtype=torch.int32)
        t, hq, hk, d = 48, 4, 2, 16
        q = torch.randn(t, hq, d, dtype=torch.float64)
        k = torch.randn(t, hk, d, dtype=torch.float64)
        v = torch.randn(t, hk, d, dtype=torch.float64)
        do = torch.randn(t, hq, d, dtype=torch.float64)
        qf, kf, vf = (x.clone().requires_grad_() for x in (q, k, v))
        bh = lambda x: x.permute(1, 0, 2).unsqueeze(0)  # noqa: E731
        ref = torch.cat([attention_ref(bh(qf[a:b]), bh(kf[a:b]), bh(vf[a:b]), causal=causal).squeeze(0).permute(1, 0, 2)
                         for a, b in zip(cu[:-1].tolist(), cu[1:].tolist())])
        ref.backward(do)
        idx = thd.thd_get_partitioned_indices(cu, t, world, rank).long()
        ql, kl, vl = (x[idx].clone().requires_grad_() for x in (q, k, v))
        out = attn_forward_func_with_cp(ql, kl, vl, cp_group=dist.group.WORLD, cp_comm_type="p2p", causal=causal,
                                        qkv_format="thd", cu_seqlens=cu // world)
        out.backward(do[idx])
        errs = [
            (out - ref.detach()[idx]).abs().max().item(),
            (ql.grad - qf.grad[idx]).abs().max().item(),
            (kl.grad - kf.grad[idx]).abs().max().item(),
            (vl.grad - vf.grad[idx]).abs().max().item(),
        ]
        result_q.put((rank, max(errs), None))
    except Exception:  # noqa: BLE001
        import traceback

        result_q.put((rank, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("world", [2, 4])
def test_thd_ring_attention_matches_per_sequence_attention(world, causal):
    ctx = mp.get_context("spawn")
    result_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_thd_worker, args=(r, world, port, causal, result_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [result_q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, err, tb in results:
        assert tb is None, f"rank {rank} failed:\n{tb}"
        assert err < 1e-4, f"rank {rank}: max error {err}"


def _cp_utils_worker(rank, world, port, q):
    import os
    import torch.distributed as dist
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import transformerengine_b200 as te
        cu = torch.tensor([0, 5, 12, 14])
        ids = torch.arange(100, 114)
        labels = torch.arange(14)
        f = 2 * world
        ids_p, lab_p, cu_p = te.pad_thd_sequences_for_cp(ids[None], labels[None], cu, f)
        pos = te.generate_positional_ids_for_cp(cu, f)
        mine = te.get_batch_on_this_cp_rank(cu_p, ids_p, lab_p, pos, dist.group.WORLD)
        gathered = [None] * world
        dist.all_gather_object(gathered, tuple(t.tolist() for t in mine))
        q.put((rank, ids_p.tolist(), lab_p.tolist(), cu_p.tolist(), pos.tolist(), gathered, None))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, None, None, None, None, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_packed_batch_helpers_reference_call_forms():
    """Pad a packed batch for context parallelism, number its positions, cut it into the ranks' dual chunks."""
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_cp_utils_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    for r in res:
        assert r[-1] is None, r[-1]
    _, ids_p, lab_p, cu_p, pos, gathered, _ = res[0]
    assert cu_p == [0, 8, 16, 20]                                  # 5 -> 8, 7 -> 8, 2 -> 4
    assert ids_p[:8] == [100, 101, 102, 103, 104, 0, 0, 0] and lab_p[5:8] == [-100] * 3
    assert pos == list(range(8)) + list(range(8)) + list(range(4))
    # rank r owns chunk r and chunk 2 * cp - 1 - r of every padded sequence; together they are the whole batch
    r0, r1 = gathered
    assert r0[2] == [0, 1, 6, 7, 0, 1, 6, 7, 0, 3] and r1[2] == [2, 3, 4, 5, 2, 3, 4, 5, 1, 2]
    assert sorted(r0[0] + r1[0]) == sorted(ids_p)
    # this library's own call forms still work
    import transformerengine_b200 as te
    assert te.pad_thd_sequences_for_cp(torch.tensor([0, 5, 12, 14]), 2).tolist() == [0, 8, 16, 20]
    assert te.get_batch_on_this_cp_rank(torch.arange(8)[None], 2, 0).tolist() == [[0, 1, 6, 7]]
