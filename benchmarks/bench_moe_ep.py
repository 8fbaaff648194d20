"""Expert-parallel dispatch + combine: the fused peer-memory kernels against the all-to-all
baseline (NCCL) on the same routing.  Launch with torch.distributed.run, one rank per GPU:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_moe_ep.py

Times forward dispatch + combine and the full forward + backward of both, device time, max over
ranks.  Roofline: bytes that must cross NVLink per rank and direction =
tokens * topk * (ep-1)/ep * hidden * 2 (dispatch) and the same for combine.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200.parallel.expert_parallel import (FusedExpertParallel, ep_combine, ep_dispatch,  # noqa: E402
                                                             fused_ep_combine, fused_ep_dispatch)


def timed(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--profile", action="store_true", help="print rank 0's kernel table of the fused forward + backward")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ep = dist.get_world_size()
    g = dist.group.WORLD
    L = a.experts // ep
    torch.manual_seed(rank)
    x = torch.randn(a.tokens, a.hidden, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    logits = torch.randn(a.tokens, a.experts, device="cuda")
    probs, rmap = te.fused_topk_with_score_function(logits, a.topk)
    probs = probs.detach().requires_grad_()
    ctx = FusedExpertParallel(g, L, a.hidden, a.tokens, torch.bfloat16, align=128, topk=a.topk)

    def fused(bwd):
        xs, ps, _, st = fused_ep_dispatch(x, probs, rmap, ctx)
        y = fused_ep_combine(xs * 1.0, st)
        if bwd:
            y.backward(torch.ones_like(y))

    def base(bwd):
        xs, ps, _, st = ep_dispatch(x, probs, rmap, g, L, 128)
        y = ep_combine(xs * 1.0, st)
        if bwd:
            y.backward(torch.ones_like(y))

    res = {"ep": ep, "tokens": a.tokens, "hidden": a.hidden, "experts": a.experts, "topk": a.topk}
    res["fused_fwd_ms"] = timed(lambda: fused(False), a.iters)
    res["nccl_fwd_ms"] = timed(lambda: base(False), a.iters)
    res["fused_fwd_bwd_ms"] = timed(lambda: fused(True), a.iters)
    res["nccl_fwd_bwd_ms"] = timed(lambda: base(True), a.iters)
    te.check_status()
    if a.profile:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            for _ in range(3):
                fused(True)
            torch.cuda.synchronize()
        if rank == 0:
            print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=22, max_name_column_width=60))
    wire = a.tokens * a.topk * (ep - 1) / ep * a.hidden * 2
    res["nvlink_bytes_per_direction_fwd"] = 2 * wire
    res["nvlink_roofline_fwd_ms"] = 2 * wire / 770e9 * 1e3  # measured 770 GB/s per direction
    res["fused_fwd_fraction_of_roofline"] = res["nvlink_roofline_fwd_ms"] / res["fused_fwd_ms"]
    if rank == 0:
        print(json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
