"""Fused collective GEMMs vs NCCL collective + dense GEMM, per shape.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_comm_gemm.py

Device time (CUDA events), max over ranks.  Roofline of a fused op = the slower of
(FLOPs / the measured peak of the dtype) and (bytes over NVLink / 770 GB/s, the measured peer copy rate).
The dtype peaks are the best rates measured on this pool with large GEMMs: bf16 = the cuBLAS burst figure
of MEASURED_PEAKS.json (1640 TFLOP/s fallback), MXFP8 = 3100 TFLOP/s (cuBLASLt block-scaled GEMM through
``torch._scaled_mm``, ``benchmarks/bench_gemm.py``); override with --peak-bf16 / --peak-mxfp8.
Also reports the fused kernel against the NCCL collective followed by this library's dense GEMM, and
(``--side 1``) the fused kernel carrying the side gather of the weight-gradient operand (bulk overlap).
``--timeline 1`` adds the kernels' own time stamps (``%globaltimer`` written by every CTA of one extra launch on
rank 0, microseconds after the first CTA started, as min / mean / max over the CTAs of a role): when the copy
CTAs finished the gated gather and the side gather, when the GEMM CTAs finished their tiles, when their last
store had completed, and when the reduce tail ended.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200 import ops  # noqa: E402
from transformerengine_b200.parallel.comm_gemm import AllGatherGemm, GemmReduceScatter  # noqa: E402
from transformerengine_b200.tensor import MXFP8Quantizer  # noqa: E402

LINK_GBS = 770.0


def timed(fn, iters=10):
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def stamps(fn, n_copy):
    """One launch of ``fn(timeline=...)``; returns {phase: [min, mean, max] us} per role (rank-local)."""
    tl = torch.zeros(148, 4, dtype=torch.int64, device="cuda")
    dist.barrier()
    torch.cuda.synchronize()
    fn(tl)
    torch.cuda.synchronize()
    t = tl.cpu().double()
    t0 = t[:, 0][t[:, 0] > 0].min()

    def mmm(rows, col):
        if rows.numel() == 0 or (rows[:, col] <= 0).all():
            return None
        x = (rows[:, col][rows[:, col] > 0] - t0) / 1e3
        return [round(float(x.min()), 1), round(float(x.mean()), 1), round(float(x.max()), 1)]

    cp, gm = t[:n_copy], t[n_copy:]
    return {"copy_ctas": n_copy, "copy_gated_done": mmm(cp, 1), "copy_side_done": mmm(cp, 2),
            "gemm_tiles_done": mmm(gm, 1), "gemm_stores_done": mmm(gm, 2), "reduce_tail_done": mmm(gm, 3)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kinds", default="mxfp8,bf16", help="operand kinds to time")
    ap.add_argument("--timeline", type=int, default=0, help="add in-kernel time stamps of one launch per kernel")
    ap.add_argument("--shapes", default="llama")
    ap.add_argument("--copy-ctas", type=int, default=0, help="0 = chosen by the library per shape")
    ap.add_argument("--peak-bf16", type=float, default=0.0, help="TFLOP/s; 0 = MEASURED_PEAKS.json or 1640")
    ap.add_argument("--peak-mxfp8", type=float, default=3100.0, help="TFLOP/s")
    ap.add_argument("--side", type=int, default=1, help="also time the kernels with the wgrad side gather")
    a = ap.parse_args()
    peak_bf16 = a.peak_bf16
    if peak_bf16 <= 0:
        pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
        peak_bf16 = json.load(open(pk)).get("bf16_tflops", 1640.4) if os.path.exists(pk) else 1640.4
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    g = dist.group.WORLD
    # (tokens, hidden, full width of the sharded dim)
    shapes = {"llama": [(8192, 4096, 6144), (8192, 4096, 28672)],
              "layer12288": [(4096, 12288, 36864), (4096, 12288, 49152)]}[a.shapes]
    q = MXFP8Quantizer(columnwise=False)
    for T, H, F in shapes:
        Fl = F // world
        for mx in [k == "mxfp8" for k in a.kinds.split(",")]:
            xl = torch.randn(T // world, H, device="cuda", dtype=torch.bfloat16)
            w1 = torch.randn(Fl, H, device="cuda", dtype=torch.bfloat16)
            x2 = torch.randn(T, Fl, device="cuda", dtype=torch.bfloat16)
            w2 = torch.randn(H, Fl, device="cuda", dtype=torch.bfloat16)
            if mx:
                xl_o, w1_o, x2_o, w2_o = q(xl), q(w1), q(x2), q(w2)
            else:
                xl_o, w1_o, x2_o, w2_o = xl, w1, x2, w2
            ag = AllGatherGemm(g, T, H, mxfp8=mx, copy_ctas=a.copy_ctas or None)
            rs = GemmReduceScatter(g, T, H)
            xg = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
            dist.all_gather_into_tensor(xg, xl)
            xg_o = q(xg) if mx else xg
            xg8 = torch.empty(T, H, device="cuda", dtype=torch.uint8 if mx else torch.bfloat16)
            xl8 = xl_o._rowwise_data if mx else xl
            part = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
            outrs = torch.empty(T // world, H, device="cuda", dtype=torch.bfloat16)

            t_ag_fused = timed(lambda: ag(xl_o, w1_o))
            t_ag_gemm = timed(lambda: ops.gemm_nt(ops.as_operand(xg_o), ops.as_operand(w1_o), out_dtype=torch.bfloat16))
            t_ag_nccl = timed(lambda: dist.all_gather_into_tensor(xg8, xl8))
            t_rs_fused = timed(lambda: rs(x2_o, w2_o))
            t_rs_gemm = timed(lambda: ops.gemm_nt(ops.as_operand(x2_o), ops.as_operand(w2_o), out=part))
            t_rs_nccl = timed(lambda: dist.reduce_scatter_tensor(outrs, part))
            te.check_status()
            elem = 1 if mx else 2
            peak = (a.peak_mxfp8 if mx else peak_bf16) * 1e12
            flops = 2.0 * T * H * Fl
            ag_bytes = T * H * elem * (world - 1) / world + (T * H / 32 * (world - 1) / world if mx else 0)
            rs_bytes = T * H * 2 * (world - 1) / world
            roof_ag = max(flops / peak * 1e3, ag_bytes / LINK_GBS / 1e6)
            roof_rs = max(flops / peak * 1e3, rs_bytes / LINK_GBS / 1e6)
            extra = {}
            if a.side and mx:
                # the same kernels carrying the column-wise copy of the local rows for the wgrad that follows
                from transformerengine_b200.parallel.comm_gemm import SideSpec

                R = T // world
                q2 = MXFP8Quantizer(rowwise=True, columnwise=True)
                xs = q2(xl)
                ag_s = AllGatherGemm(g, T, H, mxfp8=True, copy_ctas=a.copy_ctas or None, side=SideSpec.for_mxfp8_columnwise(H, R))
                rs_s = GemmReduceScatter(g, T, H, side=SideSpec.for_mxfp8_columnwise(H, R), copy_ctas=a.copy_ctas or None)
                side = (xs._columnwise_data, xs._columnwise_scale_inv)
                t_ag_side = timed(lambda: ag_s(xs, w1_o, side=side))
                t_rs_side = timed(lambda: rs_s(x2_o, w2_o, side=side))
                te.check_status()
                side_bytes = (T * H + T * H / 32) * (world - 1) / world
                extra = dict(ag_fused_with_side_ms=t_ag_side, rs_fused_with_side_ms=t_rs_side,
                             ag_side_roofline_ms=max(flops / peak * 1e3, (ag_bytes + side_bytes) / LINK_GBS / 1e6),
                             rs_side_roofline_ms=max(flops / peak * 1e3, max(rs_bytes, side_bytes) / LINK_GBS / 1e6))
                extra["ag_side_frac_of_roofline"] = extra["ag_side_roofline_ms"] / t_ag_side
                extra["rs_side_frac_of_roofline"] = extra["rs_side_roofline_ms"] / t_rs_side
                if a.timeline:
                    extra["ag_side_stamps_us"] = stamps(lambda tl: ag_s(xs, w1_o, side=side, timeline=tl),
                                                        a.copy_ctas or ag_s._auto[Fl])
                    extra["rs_side_stamps_us"] = stamps(lambda tl: rs_s(x2_o, w2_o, side=side, timeline=tl),
                                                        a.copy_ctas or rs_s._auto[Fl])
                del ag_s, rs_s
            if a.timeline:
                extra["ag_stamps_us"] = stamps(lambda tl: ag(xl_o, w1_o, timeline=tl), a.copy_ctas or ag._auto[Fl])
                extra["rs_stamps_us"] = stamps(lambda tl: rs(x2_o, w2_o, timeline=tl), 0)
            if rank == 0:
                print(json.dumps(dict(T=T, H=H, F_local=Fl, mxfp8=mx, world=world, peak_tflops=peak / 1e12,
                                      ag_fused_ms=t_ag_fused, ag_gemm_ms=t_ag_gemm, ag_nccl_ms=t_ag_nccl,
                                      ag_roofline_ms=roof_ag, ag_frac_of_roofline=roof_ag / t_ag_fused,
                                      ag_fused_over_nccl_plus_gemm=(t_ag_nccl + t_ag_gemm) / t_ag_fused,
                                      rs_fused_ms=t_rs_fused, rs_gemm_ms=t_rs_gemm, rs_nccl_ms=t_rs_nccl,
                                      rs_roofline_ms=roof_rs, rs_frac_of_roofline=roof_rs / t_rs_fused,
                                      rs_fused_over_nccl_plus_gemm=(t_rs_nccl + t_rs_gemm) / t_rs_fused, **extra)),
                      flush=True)
            del ag, rs
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
