"""Overlapped data-parallel gradient averaging over gloo ranks."""
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


def _worker(rank, world, port, result_q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from transformerengine_b200.parallel.data_parallel import DataParallelGradSync

        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
        sync = DataParallelGradSync(model.parameters(), None, min_bytes=256)
        torch.manual_seed(100 + rank)
        x = torch.randn(5, 8)
        model(x).square().sum().backward()
        sync.finish()
        got = [p.grad.clone() for p in model.parameters()]
        # reference: average of the per-rank gradients
        ref_model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
        ref_model.load_state_dict(model.state_dict())
        acc = [torch.zeros_like(p) for p in ref_model.parameters()]
        for r in range(world):
            torch.manual_seed(100 + r)
            xr = torch.randn(5, 8)
            ref_model.zero_grad()
            ref_model(xr).square().sum().backward()
            for a, p in zip(acc, ref_model.parameters()):
                a += p.grad / world
        err = max((g - a).abs().max().item() for g, a in zip(got, acc))
        result_q.put((rank, err, None))
    except Exception:  # noqa: BLE001
        import traceback

        result_q.put((rank, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_grad_sync_averages_over_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    for rank, err, tb in res:
        assert tb is None, tb
        assert err < 1e-6, (rank, err)


def _zero_worker(rank, world, port, result_q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import transformerengine_b200 as te
        from transformerengine_b200.parallel.data_parallel import DataParallelGradSync, ShardedOptimizerDataParallel

        def build():
            torch.manual_seed(0)
            return torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))

        def batch(step):
            torch.manual_seed(1000 * step + rank)
            return torch.randn(5, 8)

        # plain data parallel: every rank updates everything
        m1 = build()
        s1 = DataParallelGradSync(m1.parameters(), None, min_bytes=64)
        o1 = te.FusedAdam(m1.parameters(), lr=1e-2, master_weights=True)
        # sharded optimizer
        m2 = build()
        z = ShardedOptimizerDataParallel(m2.parameters(), None)
        owned = z.owned_parameters()
        o2 = te.FusedAdam(owned, lr=1e-2, master_weights=True)
        for step in range(3):
            o1.zero_grad(set_to_none=True)
            m1(batch(step)).square().sum().backward()
            s1.finish()
            o1.step()
            o2.zero_grad(set_to_none=True)
            for p in m2.parameters():
                p.grad = None
            m2(batch(step)).square().sum().backward()
            z.finish_grads()
            o2.step()
            z.sync_parameters()
        err = max((a - b).abs().max().item() for a, b in zip(m1.parameters(), m2.parameters()))
        n_owned = sum(p.numel() for p in owned)
        states = len(o2.state)
        result_q.put((rank, err, (n_owned, states, len(list(m2.parameters()))), None))
    except Exception:  # noqa: BLE001
        import traceback

        result_q.put((rank, None, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_optimizer_matches_plain_data_parallel(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_zero_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    total = 0
    for rank, err, info, tb in res:
        assert tb is None, tb
        assert err < 1e-6, (rank, err)
        n_owned, states, n_params = info
        assert states < n_params           # optimizer state only for the owned parameters (4 tensors: a rank may own none)
        total += n_owned
    assert total == 8 * 16 + 16 + 16 * 4 + 4   # every parameter has exactly one owner
