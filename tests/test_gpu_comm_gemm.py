"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels on 2+ GPUs against NCCL + dense GEMM."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, result_q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    bad = {}
    logdir = os.environ.get("TEB200_TEST_LOG_DIR")

    def log(msg):
        if logdir:
            with open(os.path.join(logdir, f"comm_gemm_rank{rank}.log"), "a") as f:
                f.write(msg + "\n")

    try:
        import transformerengine_b200 as te
        from transformerengine_b200 import ops
        from transformerengine_b200.parallel.comm_gemm import AllGatherGemm, GemmReduceScatter
        from transformerengine_b200.tensor import MXFP8Quantizer

        g = dist.group.WORLD
        log("imports done")
        T, K, N = 256 * world * 2, 512, 768

        def rel(a, b):
            return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()

        for mx in (False, True):
            torch.manual_seed(100 + rank)
            xl = torch.randn(T // world, K, device="cuda", dtype=torch.bfloat16)
            torch.manual_seed(7)
            w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
            ag = AllGatherGemm(g, T, K, mxfp8=mx, copy_ctas=4)
            log(f"ag context mx={mx}")
            for it in range(3):  # several calls: epochs and the double buffer
                xi = xl * (it + 1)
                xg = torch.empty(T, K, device="cuda", dtype=torch.bfloat16)
                dist.all_gather_into_tensor(xg, xi)
                if mx:
                    q = MXFP8Quantizer(columnwise=False)
                    got = ag(q(xi), q(w))
                    # quantizing the local rows then gathering equals quantizing the gathered rows
                    ref = ops.gemm_nt(ops.as_operand(q(xg)), ops.as_operand(q(w)), out_dtype=torch.bfloat16)
                else:
                    got = ag(xi, w)
                    ref = ops.gemm_nt(xg, w, out_dtype=torch.bfloat16)
                torch.cuda.synchronize()
                log(f"ag call mx={mx} it={it} done")
                te.check_status()
                if not torch.equal(got, ref):
                    bad[f"ag mx={mx} it={it}"] = rel(got, ref)
            # reduce-scatter: K is the sharded dim
            torch.manual_seed(200 + rank)
            xr = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
            wr = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
            rs = GemmReduceScatter(g, T, N)
            for it in range(3):
                xi = xr * (it + 1)
                if mx:
                    q = MXFP8Quantizer(columnwise=False)
                    a_op, b_op = q(xi), q(wr)
                    part = ops.gemm_nt(ops.as_operand(a_op), ops.as_operand(b_op), out_dtype=torch.float32)
                else:
                    a_op, b_op = xi, wr
                    part = ops.gemm_nt(xi, wr, out_dtype=torch.float32)
                ref = torch.empty(T // world, N, device="cuda", dtype=torch.float32)
                dist.reduce_scatter_tensor(ref, part)
                got = rs(a_op, b_op)
                torch.cuda.synchronize()
                log(f"rs call mx={mx} it={it} done")
                te.check_status()
                e = rel(got, ref)
                if not e < 1e-2:
                    bad[f"rs mx={mx} it={it}"] = e
        result_q.put((rank, bad))
    except Exception:  # noqa: BLE001
        import traceback
        log(traceback.format_exc())
        result_q.put((rank, {"exception": traceback.format_exc()[-2000:]}))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def test_fused_collective_gemms():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=150) for _ in procs]
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()  # exact child processes started above
    for rank, bad in res:
        assert not bad, f"rank {rank}: {bad}"
