"""Fused expert-parallel dispatch/combine over NVLink peer memory on 2+ GPUs against the
all-to-all baseline (NCCL)."""
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
            with open(os.path.join(logdir, f"moe_ep_rank{rank}.log"), "a") as f:
                f.write(msg + "\n")

    try:
        import transformerengine_b200 as te
        from transformerengine_b200.parallel.expert_parallel import (FusedExpertParallel, ep_combine, ep_dispatch,
                                                                     fused_ep_combine, fused_ep_dispatch)

        g = dist.group.WORLD
        T, H, L, topk = 192, 256, 2, 2
        E = L * world
        ctx = FusedExpertParallel(g, L, H, T, torch.bfloat16, align=32, topk=topk)
        log("context built")
        for it in range(3):
            torch.manual_seed(1000 * it + rank)
            x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
            logits = torch.randn(T, E, device="cuda")
            probs, rmap = te.fused_topk_with_score_function(logits, topk)
            res = {}
            for name in ("fused", "base"):
                xx = x.clone().requires_grad_()
                pp = probs.clone().requires_grad_()
                if name == "fused":
                    xs, ps, m_splits, st = fused_ep_dispatch(xx, pp, rmap, ctx)
                else:
                    xs, ps, m_splits, st = ep_dispatch(xx, pp, rmap, g, L, 32)
                torch.manual_seed(5)
                wmix = torch.randn(H, H, device="cuda", dtype=torch.bfloat16) * 0.05
                o = (xs.float() @ wmix.float() * ps.float()[:, None]).to(torch.bfloat16)  # stand-in expert
                y = fused_ep_combine(o, st) if name == "fused" else ep_combine(o, st)
                (y.float() * torch.linspace(0.5, 1.5, H, device="cuda")).sum().backward()
                torch.cuda.synchronize()
                te.check_status()
                res[name] = (m_splits, xs.detach(), ps.detach(), y.detach(), xx.grad, pp.grad)
                log(f"it {it} {name} done")
            f, b = res["fused"], res["base"]
            if f[0] != b[0]:
                bad[f"splits it={it}"] = (f[0], b[0])
                continue
            # rows inside an expert slab are ordered by source rank in both paths
            for i, nm in enumerate(["xs", "ps", "y", "gx", "gp"], start=1):
                d = (f[i].float() - b[i].float()).abs().max().item()
                ref = b[i].float().abs().max().item()
                if not d <= 2e-2 * max(ref, 1e-3):
                    bad[f"{nm} it={it}"] = (d, ref)
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


def test_fused_ep_matches_all_to_all():
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
