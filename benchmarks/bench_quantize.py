"""Memory-bound kernel microbenchmark: MXFP8 tile quantizer (plain, norm, SwiGLU, dSwiGLU),
norm backward and fused Adam.  Reports achieved GB/s against the algorithmic bytes and
the fraction of the measured copy bandwidth (MEASURED_PEAKS.json when present).

    python benchmarks/bench_quantize.py [--tokens 8192] [--iters 20]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformerengine_b200 import ops  # noqa: E402
from transformerengine_b200.ops import quantize as qz  # noqa: E402
from transformerengine_b200.tensor import MXFP8Quantizer  # noqa: E402


def time_fn(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    peak = 6548.8
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("hbm_gbs", peak)
    T, H, F = a.tokens, 4096, 14336
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    bf = torch.bfloat16
    q = MXFP8Quantizer()
    rows = []

    def report(name, fn, nbytes):
        ms = time_fn(fn, a.iters, flush)
        gbs = nbytes / ms / 1e6
        rows.append(dict(kernel=name, ms=ms, gbs=gbs, frac_of_measured=gbs / peak))
        print(json.dumps(rows[-1]))

    x = torch.randn(T, H, device="cuda", dtype=bf)
    report("quantize_mxfp8 [T,4096] row+col", lambda: qz.quantize_mxfp8(x, torch.float8_e4m3fn), T * H * 4)
    w = torch.randn(2 * F, H, device="cuda", dtype=bf)
    report("quantize_mxfp8 [28672,4096] row+col", lambda: qz.quantize_mxfp8(w, torch.float8_e4m3fn), 2 * F * H * 4)
    g = torch.ones(H, device="cuda", dtype=bf)
    report("rmsnorm stats + norm-quantize [T,4096]",
           lambda: ops.norm_fwd(x, g, None, 1e-5, False, False, quantizer=q, want_hp=False), T * H * (2 + 2 + 2))
    h = torch.randn(T, 2 * F, device="cuda", dtype=bf)
    report("swiglu + quantize [T,28672]->[T,14336]", lambda: ops.activation_fwd(h, "swiglu", quantizer=q, want_hp=False),
           T * 2 * F * 2 + T * F * 2)
    dy = torch.randn(T, F, device="cuda", dtype=bf)
    report("dswiglu + quantize [T,28672]", lambda: ops.activation_bwd(dy, h, "swiglu", quantizer=q, want_hp=False),
           T * F * 2 + T * 2 * F * 2 + T * 2 * F * 2)
    _, _, mu, rs = ops.norm_fwd(x, g, None, 1e-5, False, False)
    report("rmsnorm bwd [T,4096]", lambda: ops.norm_bwd(x, x, mu, rs, g, False, False), T * H * 2 * 3)
    n = 256 << 20
    p, gr = torch.randn(n, device="cuda", dtype=bf), torch.randn(n, device="cuda", dtype=bf)
    m, v, mp = (torch.zeros(n, device="cuda") for _ in range(3))
    report("fused adam 256M params (bf16 g/p, fp32 m/v/master)",
           lambda: ops.multi_tensor_adam([[gr], [p], [m], [v], [mp]], 1e-4, 0.9, 0.95, 1e-8, 1, True, True, 0.1),
           n * (2 + 4 + 4 + 4 + 4 + 4 + 4 + 2))


if __name__ == "__main__":
    main()
