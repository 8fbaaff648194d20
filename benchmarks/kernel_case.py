"""Run one kernel of the library a few times on a fixed case (target for ncu captures).

    python benchmarks/kernel_case.py --kernel gemm_mxfp8|gemm_bf16|quantize|swiglu_quantize|adam|rmsnorm_bwd|cross_entropy|attention|rope|nvfp4_quantize|router|permute
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200 import ops  # noqa: E402
from transformerengine_b200.ops import quantize as qz  # noqa: E402
from transformerengine_b200.tensor import MXFP8Quantizer  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True)
    ap.add_argument("--reps", type=int, default=3)
    a = ap.parse_args()
    bf = torch.bfloat16
    T, H, F = 8192, 4096, 14336
    if a.kernel in ("gemm_mxfp8", "gemm_bf16"):
        x = torch.randn(T, H, device="cuda", dtype=bf)
        w = torch.randn(6144, H, device="cuda", dtype=bf)
        out = torch.empty(T, 6144, device="cuda", dtype=bf)
        if a.kernel == "gemm_mxfp8":
            q = MXFP8Quantizer(columnwise=False)
            xo, wo = ops.as_operand(q(x)), ops.as_operand(q(w))
            fn = lambda: ops.gemm_nt(xo, wo, out=out)  # noqa: E731
        else:
            fn = lambda: ops.gemm_nt(x, w, out=out)  # noqa: E731
    elif a.kernel == "quantize":
        x = torch.randn(T, H, device="cuda", dtype=bf)
        fn = lambda: qz.quantize_mxfp8(x, torch.float8_e4m3fn)  # noqa: E731
    elif a.kernel == "swiglu_quantize":
        h = torch.randn(T, 2 * F, device="cuda", dtype=bf)
        q = MXFP8Quantizer()
        fn = lambda: ops.activation_fwd(h, "swiglu", quantizer=q, want_hp=False)  # noqa: E731
    elif a.kernel == "adam":
        n = 64 << 20
        p, g = torch.randn(n, device="cuda", dtype=bf), torch.randn(n, device="cuda", dtype=bf)
        m, v, mp = (torch.zeros(n, device="cuda") for _ in range(3))
        fn = lambda: ops.multi_tensor_adam([[g], [p], [m], [v], [mp]], 1e-4, 0.9, 0.95, 1e-8, 1, True, True, 0.1)  # noqa: E731
    elif a.kernel == "rmsnorm_bwd":
        x = torch.randn(T, H, device="cuda", dtype=bf)
        g = torch.ones(H, device="cuda", dtype=bf)
        _, _, mu, rs = ops.norm_fwd(x, g, None, 1e-5, False, False)
        fn = lambda: ops.norm_bwd(x, x, mu, rs, g, False, False)  # noqa: E731
    elif a.kernel == "cross_entropy":
        lg = torch.randn(2048, 128256, device="cuda", dtype=bf)
        t = torch.randint(0, 128256, (2048,), device="cuda")
        fn = lambda: ops.cross_entropy_fwd_bwd(lg, t, 1.0, inplace_grad=False)  # noqa: E731
    elif a.kernel == "attention":
        # causal GQA, 16 query / 4 key-value heads, seq 4096: forward + both backward kernels
        from transformerengine_b200.ops import flash

        q = torch.randn(1, 16, 4096, 128, device="cuda", dtype=bf, requires_grad=True)
        k = torch.randn(1, 4, 4096, 128, device="cuda", dtype=bf, requires_grad=True)
        v = torch.randn(1, 4, 4096, 128, device="cuda", dtype=bf, requires_grad=True)
        do = torch.randn(1, 16, 4096, 128, device="cuda", dtype=bf)
        fn = lambda: flash.flash_attention(q, k, v, None, True).backward(do)  # noqa: E731
    elif a.kernel == "rope":
        x = torch.randn(8192, 1, 32, 128, device="cuda", dtype=bf)
        f = ops.rope_freqs(torch.arange(8192, device="cuda"), 128, 500000.0, False)
        fn = lambda: ops.rope_apply(x, f)  # noqa: E731
    elif a.kernel == "nvfp4_quantize":
        x = torch.randn(T, H, device="cuda", dtype=bf)
        fn = lambda: qz.quantize_nvfp4(x, with_rht=True)  # noqa: E731
    elif a.kernel == "router":
        lg = torch.randn(65536, 64, device="cuda")
        fn = lambda: te.fused_topk_with_score_function(lg, 6, False, None, None, 1.0, "sigmoid", None)  # noqa: E731
    elif a.kernel == "permute":
        x = torch.randn(T, H, device="cuda", dtype=bf)
        probs, rmap = te.fused_topk_with_score_function(torch.randn(T, 8, device="cuda"), 2)
        fn = lambda: te.moe_unpermute(te.moe_permute_with_probs(x, probs, rmap)[0], te.moe_permute(x, rmap)[1], probs)  # noqa: E731
    else:
        raise SystemExit(f"unknown kernel {a.kernel}")
    for _ in range(a.reps):
        fn()
    torch.cuda.synchronize()
    te.check_status()
    print("ok")


if __name__ == "__main__":
    main()
