"""Overlapped data-parallel gradient averaging over gloo ranks."""
import os
import socket

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
