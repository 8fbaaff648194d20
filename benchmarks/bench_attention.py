"""Fused attention microbenchmark: this library's tcgen05 kernels against torch's SDPA (cuDNN /
flash library kernels) on the same tensors.  Causal GQA, head dim 128, bf16.

    python benchmarks/bench_attention.py --seq 8192 --heads 32 --kv-heads 8 --iters 10
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-library", action="store_true")
    args = ap.parse_args()
    import transformerengine_b200 as te
    from transformerengine_b200.ops import flash

    torch.manual_seed(0)
    b, hq, hk, s = args.batch, args.heads, args.kv_heads, args.seq
    mk = lambda h: torch.randn(b, h, s, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)  # noqa: E731
    q, k, v = mk(hq), mk(hk), mk(hk)
    do = torch.randn(b, hq, s, 128, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2
    fwd_flops = 4.0 * b * hq * s * s * 128 / 2
    res = {"b": b, "hq": hq, "hk": hk, "seq": s, "causal": True, "l2": "256 MB flush between iterations"}

    def own_fwd():
        return flash.flash_attention(q, k, v, None, True)

    def own_fb():
        o = own_fwd()
        o.backward(do)

    res["own_fwd_ms"] = timed(lambda: own_fwd(), args.iters, flush)
    res["own_fwd_bwd_ms"] = timed(own_fb, args.iters, flush)
    te.ops.check_status()
    res["own_fwd_tflops"] = fwd_flops / res["own_fwd_ms"] / 1e9
    res["own_bwd_tflops"] = 2.5 * fwd_flops / (res["own_fwd_bwd_ms"] - res["own_fwd_ms"]) / 1e9
    if not args.no_library:
        sd = torch.nn.functional.scaled_dot_product_attention

        def lib_fwd():
            return sd(q, k, v, is_causal=True, enable_gqa=hq != hk)

        def lib_fb():
            lib_fwd().backward(do)

        res["library_fwd_ms"] = timed(lambda: lib_fwd(), args.iters, flush)
        res["library_fwd_bwd_ms"] = timed(lib_fb, args.iters, flush)
        res["library_fwd_tflops"] = fwd_flops / res["library_fwd_ms"] / 1e9
    print(json.dumps(res))


if __name__ == "__main__":
    main()
