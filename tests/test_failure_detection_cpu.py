"""Failure detection on the host: a rank that leaves between steps, a rank that never joins a barrier and
a rank that raises are all noticed by the survivors as an exception, not a hang (gloo ranks on CPU)."""
import os
import socket
import time

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, scenario, result_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from transformerengine_b200.parallel.health import PeerLostError, RankMonitor, bounded_barrier

    try:
        mon = RankMonitor(max_silence_s=1.0)
        bounded_barrier("start", timeout_s=10.0)
        out = None
        if scenario == "leave":
            # three healthy steps, then the last rank announces its exit between steps
            for step in range(3):
                mon.beat()
                mon.check_peers()
                bounded_barrier(f"step{step}", timeout_s=10.0)
            if rank == world - 1:
                mon.leave()
                out = "left"
            else:
                deadline = time.time() + 10.0
                while out is None and time.time() < deadline:
                    mon.beat()
                    try:
                        mon.check_peers()
                        time.sleep(0.05)
                    except PeerLostError as e:
                        out = ("lost", e.ranks)
        elif scenario == "silent":
            # the last rank stops beating (a hung host thread): its heartbeat ages out
            if rank == world - 1:
                time.sleep(3.0)
                out = "slept"
            else:
                deadline = time.time() + 10.0
                while out is None and time.time() < deadline:
                    mon.beat()
                    try:
                        mon.check_peers()
                        time.sleep(0.05)
                    except PeerLostError as e:
                        out = ("lost", e.ranks)
        elif scenario == "barrier":
            # the last rank raises before the barrier: the others get the error from the barrier, in time
            if rank == world - 1:
                try:
                    raise ValueError("injected failure before the barrier")
                except ValueError:
                    out = "raised"
            else:
                t0 = time.time()
                try:
                    bounded_barrier("never-complete", timeout_s=1.0)
                    out = "passed"
                except PeerLostError as e:
                    out = ("lost", e.ranks, time.time() - t0)
        result_q.put((rank, out))
        # keep the store (hosted by rank 0) alive until everyone has reported
        time.sleep(1.0 if rank else 4.5)
    except Exception:  # noqa: BLE001
        import traceback

        result_q.put((rank, ("exception", traceback.format_exc()[-1500:])))


@pytest.mark.parametrize("scenario", ["leave", "silent", "barrier"])
def test_survivors_get_an_error_not_a_hang(scenario):
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, scenario, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = dict(q.get(timeout=60) for _ in procs)
    finally:
        for p in procs:
            p.join(timeout=15)
            if p.is_alive():
                p.kill()  # exact child processes started above
    for r in range(world - 1):
        assert res[r][0] == "lost" and res[r][1] == [world - 1], res
        if scenario == "barrier":
            assert res[r][2] < 5.0
    assert res[world - 1] in ("left", "slept", "raised")


def test_recover_drops_contexts():
    from transformerengine_b200.parallel import comm_gemm, health

    comm_gemm._CONTEXTS[("x",)] = object()
    comm_gemm._ENABLED["group"] = object()
    health.recover()
    assert not comm_gemm._CONTEXTS and comm_gemm._ENABLED["group"] is None
