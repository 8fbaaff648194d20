"""GEMM microbenchmark: tcgen05 kernels of this library vs the libraries on the same box:
torch.matmul (cuBLAS bf16) and ``torch._scaled_mm`` with block-wise E8M0 scales (the cuBLASLt MXFP8
path that the reference calls, ``common/gemm/cublaslt_gemm.cu:500-535``).  The library GEMMs are
timed for comparison only; nothing in the package calls them.

    python benchmarks/bench_gemm.py [--shapes llama|layer12288] [--iters 20]

Times with CUDA events after warm-up; an L2-sized buffer is rewritten between
iterations.  Prints TFLOP/s and the fraction of the measured bf16 cuBLAS peak
(MEASURED_PEAKS.json beside the repository root when present).
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200 import ops  # noqa: E402
from transformerengine_b200.tensor import MXFP8Quantizer  # noqa: E402

SHAPES = {
    # (M tokens, N, K)
    "llama": [(8192, 6144, 4096), (8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336),
              (4096, 8192, 8192), (6144, 4096, 8192), (28672, 4096, 8192)],
    "layer12288": [(4096, 6144, 12288), (4096, 12288, 6144), (4096, 49152, 12288), (4096, 12288, 49152)],
    "small": [(1024, 1024, 1024), (2048, 2048, 2048)],
}


def time_fn(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        evs.append((s, e))
    torch.cuda.synchronize()
    ts = sorted(s.elapsed_time(e) for s, e in evs)
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="llama")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    peak = 1640.4
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("bf16_tflops", peak)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    for M, N, K in SHAPES[args.shapes]:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * M * N * K
        t_lib = time_fn(lambda: torch.matmul(a, b.t(), out=out), args.iters, flush)
        t_bf = time_fn(lambda: ops.gemm_nt(a, b, out=out), args.iters, flush)
        qa = MXFP8Quantizer(columnwise=False)(a)
        qb = MXFP8Quantizer(columnwise=False)(b)
        oa, ob = ops.as_operand(qa), ops.as_operand(qb)
        t_mx = time_fn(lambda: ops.gemm_nt(oa, ob, out=out), args.iters, flush)
        te.check_status()
        # library MXFP8: same FP8 payload and the same 128x4-tile scale layout, viewed with torch's dtypes
        t_lib_mx, lib_err = None, None
        try:
            a8, b8 = oa.data.view(torch.float8_e4m3fn), ob.data.view(torch.float8_e4m3fn)
            sa, sb = oa.scale.view(torch.float8_e8m0fnu), ob.scale.view(torch.float8_e8m0fnu)
            ref = torch._scaled_mm(a8, b8.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
            ours = ops.gemm_nt(oa, ob, out_dtype=torch.bfloat16)
            lib_err = ((ours.float() - ref.float()).norm() / ref.float().norm()).item()
            t_lib_mx = time_fn(lambda: torch._scaled_mm(a8, b8.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16),
                               args.iters, flush)
        except Exception as e:  # noqa: BLE001  (library path unavailable in this torch build)
            lib_err = f"{type(e).__name__}: {str(e)[:120]}"
        row = dict(M=M, N=N, K=K, cublas_bf16_ms=t_lib, ours_bf16_ms=t_bf, ours_mxfp8_ms=t_mx,
                   cublaslt_mxfp8_ms=t_lib_mx, cublaslt_mxfp8_tflops=(fl / t_lib_mx / 1e9) if t_lib_mx else None,
                   ours_over_cublaslt_mxfp8=(t_lib_mx / t_mx) if t_lib_mx else None, mxfp8_rel_diff_vs_library=lib_err,
                   cublas_tflops=fl / t_lib / 1e9, ours_bf16_tflops=fl / t_bf / 1e9, ours_mxfp8_tflops=fl / t_mx / 1e9,
                   ours_bf16_frac_of_measured=fl / t_bf / 1e9 / peak)
        rows.append(row)
        print(json.dumps(row))
    if args.json:
        json.dump(rows, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
