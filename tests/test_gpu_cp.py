"""Context-parallel attention whose K/V exchange is fused into the attention kernel (peer TMA
reads) on 2+ GPUs, against full-sequence attention in fp32."""
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
            with open(os.path.join(logdir, f"cp_rank{rank}.log"), "a") as f:
                f.write(msg + "\n")

    try:
        import transformerengine_b200 as te
        from transformerengine_b200.ops.attention import attention_ref
        from transformerengine_b200.parallel.context_parallel import (attn_forward_func_with_cp,
                                                                      get_batch_on_this_cp_rank)

        g = dist.group.WORLD
        b, hq, hk, d = 1, 4, 2, 128
        s = 256 * world
        for causal in (True, False):
            for it in range(2):
                torch.manual_seed(10 + it)
                q = torch.randn(b, hq, s, d, device="cuda", dtype=torch.bfloat16)
                k = torch.randn(b, hk, s, d, device="cuda", dtype=torch.bfloat16)
                v = torch.randn(b, hk, s, d, device="cuda", dtype=torch.bfloat16)
                do = torch.randn(b, hq, s, d, device="cuda", dtype=torch.bfloat16)
                qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
                ref = attention_ref(qf, kf, vf, causal=causal)
                ref.backward(do.float())

                def shard(t):
                    if causal:
                        return get_batch_on_this_cp_rank(t, world, rank, seq_dim=2).contiguous()
                    return t.chunk(world, dim=2)[rank].contiguous()

                ql, kl, vl = (shard(t).clone().requires_grad_() for t in (q, k, v))
                out = attn_forward_func_with_cp(ql, kl, vl, cp_group=g, cp_comm_type="p2p", causal=causal)
                out.backward(shard(do))
                torch.cuda.synchronize()
                te.check_status()
                log(f"causal={causal} it={it} done")
                pairs = {"out": (out, shard(ref.detach())), "dq": (ql.grad, shard(qf.grad)),
                         "dk": (kl.grad, shard(kf.grad)), "dv": (vl.grad, shard(vf.grad))}
                for nm, (a, r) in pairs.items():
                    e = (a.float() - r.float()).abs().max().item()
                    m = r.float().abs().max().item()
                    if not e <= 3e-2 * max(m, 1e-3):
                        bad[f"{nm} causal={causal} it={it}"] = (e, m)
        # packed sequences: ring over NCCL, every product one launch of the variable-length kernels
        from transformerengine_b200.attention import thd

        lens = [256 * world, 512 * world, 128 * world]
        cu = torch.tensor([0] + [sum(lens[:i + 1]) for i in range(len(lens))], dtype=torch.int32, device="cuda")
        t = int(cu[-1])
        for causal in (True, False):
            torch.manual_seed(20)
            q = torch.randn(t, hq, d, device="cuda", dtype=torch.bfloat16)
            k = torch.randn(t, hk, d, device="cuda", dtype=torch.bfloat16)
            v = torch.randn(t, hk, d, device="cuda", dtype=torch.bfloat16)
            do = torch.randn(t, hq, d, device="cuda", dtype=torch.bfloat16)
            qf, kf, vf = (x.float().requires_grad_() for x in (q, k, v))
            bh = lambda x: x.permute(1, 0, 2).unsqueeze(0)  # noqa: E731
            ref = torch.cat([attention_ref(bh(qf[a:e]), bh(kf[a:e]), bh(vf[a:e]), causal=causal).squeeze(0).permute(1, 0, 2)
                             for a, e in zip(cu[:-1].tolist(), cu[1:].tolist())])
            ref.backward(do.float())
            idx = thd.thd_get_partitioned_indices(cu, t, world, rank).long()
            ql, kl, vl = (x[idx].clone().requires_grad_() for x in (q, k, v))
            out = attn_forward_func_with_cp(ql, kl, vl, cp_group=g, cp_comm_type="p2p", causal=causal,
                                            qkv_format="thd", cu_seqlens=cu // world)
            out.backward(do[idx])
            torch.cuda.synchronize()
            te.check_status()
            log(f"thd causal={causal} done")
            pairs = {"out": (out, ref.detach()[idx]), "dq": (ql.grad, qf.grad[idx]), "dk": (kl.grad, kf.grad[idx]),
                     "dv": (vl.grad, vf.grad[idx])}
            for nm, (a, r) in pairs.items():
                e = (a.float() - r.float()).abs().max().item()
                m = r.float().abs().max().item()
                if not e <= 3e-2 * max(m, 1e-3):
                    bad[f"thd {nm} causal={causal}"] = (e, m)
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


def test_fused_ring_attention_matches_full_attention():
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
