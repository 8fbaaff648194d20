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
            # all-reduce: the same product, every rank ends with all rows (two contexts' worth of calls: the
            # result buffer is double buffered, an earlier result must survive one further call)
            from transformerengine_b200.parallel.comm_gemm import GemmAllReduce

            ar = GemmAllReduce(g, T, N)
            prev = None
            for it in range(4):
                xi = xr * (it + 1)
                if mx:
                    q = MXFP8Quantizer(columnwise=False)
                    a_op, b_op = q(xi), q(wr)
                    part = ops.gemm_nt(ops.as_operand(a_op), ops.as_operand(b_op), out_dtype=torch.float32)
                else:
                    a_op, b_op = xi, wr
                    part = ops.gemm_nt(xi, wr, out_dtype=torch.float32)
                dist.all_reduce(part)
                got = ar(a_op, b_op)
                torch.cuda.synchronize()
                log(f"ar call mx={mx} it={it} done")
                te.check_status()
                e = rel(got, part)
                if not e < 1e-2:
                    bad[f"ar mx={mx} it={it}"] = e
                if prev is not None and not torch.equal(prev[0], prev[1]):
                    bad[f"ar mx={mx} it={it} previous result overwritten"] = 1.0
                prev = (got, got.clone())
            del ar
        # ---- side gather (the wgrad operand travels next to the GEMM), shapes with more tiles than SMs
        from transformerengine_b200.parallel.comm_gemm import SideSpec
        from transformerengine_b200.parallel.distributed import gather_mxfp8_along_first_dim

        T2, K2, N2 = 1024 * world, 1024, 4096          # (T2/128) * (N2/256) = 128 * world tiles
        R = T2 // world
        torch.manual_seed(300 + rank)
        xl = torch.randn(R, K2, device="cuda", dtype=torch.bfloat16)
        torch.manual_seed(9)
        w2 = torch.randn(N2, K2, device="cuda", dtype=torch.bfloat16)
        q2 = MXFP8Quantizer(rowwise=True, columnwise=True)
        ag_mx = AllGatherGemm(g, T2, K2, mxfp8=True, side=SideSpec.for_mxfp8_columnwise(K2, R))
        ag_hp = AllGatherGemm(g, T2, K2, mxfp8=False, side=SideSpec.for_rows(R, K2 * 2))
        wq = MXFP8Quantizer(columnwise=False)(w2)
        for it in range(3):
            xi = xl * (it + 1)
            xq = q2(xi)
            full = gather_mxfp8_along_first_dim(xq, g)  # NCCL oracle for both copies
            out, gd, gsf = ag_mx(xq, wq, side=(xq._columnwise_data, xq._columnwise_scale_inv))
            ref = ops.gemm_nt(ops.as_operand(full, "rowwise"), ops.as_operand(wq), out_dtype=torch.bfloat16)
            torch.cuda.synchronize()
            te.check_status()
            if not torch.equal(out, ref):
                bad[f"ag+side mx it={it} out"] = rel(out, ref)
            if not torch.equal(gd.view(K2, T2), full._columnwise_data.view(K2, T2)):
                bad[f"ag+side mx it={it} data"] = 1.0
            if not torch.equal(gsf.view(-1), full._columnwise_scale_inv.view(-1)[:gsf.numel()]):
                bad[f"ag+side mx it={it} scales"] = 1.0
            xg = torch.empty(T2, K2, device="cuda", dtype=torch.bfloat16)
            dist.all_gather_into_tensor(xg, xi)
            out, gd, _ = ag_hp(xi, w2, side=(xi, None))
            torch.cuda.synchronize()
            te.check_status()
            if not torch.equal(gd.view(torch.bfloat16).reshape(T2, K2), xg):
                bad[f"ag+side hp it={it} data"] = 1.0
            if not torch.equal(out, ops.gemm_nt(xg, w2, out_dtype=torch.bfloat16)):
                bad[f"ag+side hp it={it} out"] = 1.0
        log("ag side done")
        # reduce-scatter with a side gather of an unrelated operand (the layer input of a column-parallel layer)
        torch.manual_seed(400 + rank)
        xr = torch.randn(T2, K2, device="cuda", dtype=torch.bfloat16)
        wr = torch.randn(N2, K2, device="cuda", dtype=torch.bfloat16)
        C3 = 768
        sl = torch.randn(R, C3, device="cuda", dtype=torch.bfloat16)
        rs_mx = GemmReduceScatter(g, T2, N2, side=SideSpec.for_mxfp8_columnwise(C3, R))
        for it in range(3):
            xi = xr * (it + 1)
            qa, qb = MXFP8Quantizer(columnwise=False)(xi), MXFP8Quantizer(columnwise=False)(wr)
            sq = q2(sl * (it + 1))
            full = gather_mxfp8_along_first_dim(sq, g)
            part = ops.gemm_nt(ops.as_operand(qa), ops.as_operand(qb), out_dtype=torch.float32)
            ref = torch.empty(R, N2, device="cuda", dtype=torch.float32)
            dist.reduce_scatter_tensor(ref, part)
            got, gd, gsf = rs_mx(qa, qb, side=(sq._columnwise_data, sq._columnwise_scale_inv))
            torch.cuda.synchronize()
            te.check_status()
            e = rel(got, ref)
            if not e < 1e-2:
                bad[f"rs+side it={it} out"] = e
            if not torch.equal(gd.view(C3, T2), full._columnwise_data.view(C3, T2)):
                bad[f"rs+side it={it} data"] = 1.0
            if not torch.equal(gsf.view(-1), full._columnwise_scale_inv.view(-1)[:gsf.numel()]):
                bad[f"rs+side it={it} scales"] = 1.0
        log("rs side done")
        # ---- the same launches recorded in a CUDA graph and replayed (odd number of calls per context)
        sync = torch.zeros(1, device="cuda")
        x_static = xl.clone()
        side_stream = torch.cuda.Stream()
        side_stream.wait_stream(torch.cuda.current_stream())

        def body():
            dist.all_reduce(sync)          # replay boundary: no rank runs ahead into the next replay
            outs = []
            for k in range(3):
                xq_ = q2(x_static * (k + 1))
                o, d_, s_ = ag_mx(xq_, wq, side=(xq_._columnwise_data, xq_._columnwise_scale_inv))
                r_, _, _ = rs_mx(MXFP8Quantizer(columnwise=False)(o[:, :K2].contiguous()),
                                 MXFP8Quantizer(columnwise=False)(wr), side=(xq_._columnwise_data[:C3].contiguous(),
                                                                            xq_._columnwise_scale_inv[:C3 // 128 * (R // 128) * 512]))
                outs.append((o, d_, r_))
            return outs

        with torch.cuda.stream(side_stream):
            body()
        torch.cuda.current_stream().wait_stream(side_stream)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            g_outs = body()
        for rep in range(3):
            x_static.copy_(xl * (rep + 2))
            graph.replay()
            torch.cuda.synchronize()
            te.check_status()
            snap = [(o.clone(), d_.clone(), r_.clone()) for o, d_, r_ in g_outs]
            e_outs = body()   # eager launches interleaved with replays: the device-side call counters carry on
            torch.cuda.synchronize()
            te.check_status()
            for k, ((o, d_, r_), (eo, ed, er)) in enumerate(zip(snap, e_outs)):
                if not (torch.equal(o, eo) and torch.equal(d_, ed)):
                    bad[f"graph rep={rep} call={k} ag"] = rel(o, eo)
                if not rel(r_, er) < 1e-2:
                    bad[f"graph rep={rep} call={k} rs"] = rel(r_, er)
        log("graph done")
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
    world = torch.cuda.device_count() if torch.cuda.device_count() in (2, 4, 8) else min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=240) for _ in procs]
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()  # exact child processes started above
    for rank, bad in res:
        assert not bad, f"rank {rank}: {bad}"
