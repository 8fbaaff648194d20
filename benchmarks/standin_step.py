"""Library stand-in for the benchmark step -- NOT the reference and not this library.

The unmodified reference cannot be installed on this image (it needs a newer cudnn-frontend), so this
script gives the step-level numbers a same-box yardstick built only from stock PyTorch pieces: the same
Llama-3-8B-architecture step (seq 8192, micro-batch 1) from ``torch.nn`` modules, ``F.rms_norm``,
``F.scaled_dot_product_attention``, MXFP8 GEMMs through ``torch._scaled_mm`` with block-wise E8M0 scales
(the cuBLASLt path the reference calls), a torch-op MXFP8 quantizer (optionally ``torch.compile``-d, as
torchao does), ``F.cross_entropy`` and ``torch.optim.AdamW(fused=True)`` on the bf16 parameters (no fp32 master copy:
that would not fit beside torch's fp32 gradients; it makes the stand-in's optimizer cheaper than the
benchmark's, which is noted in its output).
Same shapes, seeds, synthetic data and timing rules as ``bench.py``.  Data parallel over NCCL for N > 1.

    python benchmarks/standin_step.py --steps 5 --warmup 3 [--layers 32] [--recipe mxfp8|bf16] [--compile 1]

Prints one JSON line with ``"impl": "standin"``.
"""
import argparse
import json
import math
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

E4M3_MAX = 448.0


def to_blocked(s: torch.Tensor) -> torch.Tensor:
    """[rows, cols] uint8 scales -> the 128x4-tile layout cuBLASLt expects, flattened."""
    rows, cols = s.shape
    rb, cb = (rows + 127) // 128, (cols + 3) // 4
    if (rows, cols) != (rb * 128, cb * 4):
        s = F.pad(s, (0, cb * 4 - cols, 0, rb * 128 - rows))
    blocks = s.view(rb, 128, cb, 4).permute(0, 2, 1, 3)
    return blocks.reshape(-1, 4, 32, 4).transpose(1, 2).reshape(-1, 32, 16).flatten()


def mx_quant(x: torch.Tensor):
    """[R, C] 16-bit -> (E4M3 [R, C], E8M0 scales in GEMM layout); blocks of 32 along C."""
    R, C = x.shape
    xb = x.view(R, C // 32, 32).float()
    amax = xb.abs().amax(-1).clamp_min(2.0 ** -127)
    e = torch.ceil(torch.log2(amax / E4M3_MAX)).clamp(-127, 127)
    q = (xb * torch.exp2(-e).unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(R, C)
    return q, to_blocked((e + 127).to(torch.uint8)).view(torch.float8_e8m0fnu)


_QUANT = mx_quant


def mx_mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a [M, K] @ b[N, K]^T with both operands quantized along K."""
    qa, sa = _QUANT(a)
    qb, sb = _QUANT(b)
    return torch._scaled_mm(qa, qb.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)


class MXLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return mx_mm(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = mx_mm(dy, w.t().contiguous())
        dw = mx_mm(dy.t().contiguous(), x.t().contiguous())
        return dx, dw


def linear(x, w, mx):
    x2 = x.reshape(-1, x.shape[-1])
    y = MXLinearFn.apply(x2, w) if mx else x2 @ w.t()
    return y.reshape(*x.shape[:-1], w.shape[0])


def rope(x, cos, sin):  # x [b, h, s, d]
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return x * cos + torch.cat((-x2, x1), -1) * sin


class Layer(torch.nn.Module):
    def __init__(self, H, FFN, NH, NKV):
        super().__init__()
        d = H // NH
        mk = lambda *s: torch.nn.Parameter(torch.empty(*s, device="cuda", dtype=torch.bfloat16).normal_(0, 0.02))  # noqa: E731
        self.qkv, self.proj = mk(H + 2 * NKV * d, H), mk(H, H)
        self.fc1, self.fc2 = mk(2 * FFN, H), mk(H, FFN)
        self.n1 = torch.nn.Parameter(torch.ones(H, device="cuda", dtype=torch.bfloat16))
        self.n2 = torch.nn.Parameter(torch.ones(H, device="cuda", dtype=torch.bfloat16))
        self.NH, self.NKV, self.d, self.FFN = NH, NKV, d, FFN


def layer_fwd(L, x, cos, sin, mx):
    b, s, H = x.shape
    h = F.rms_norm(x, (H,), L.n1, 1e-5)
    qkv = linear(h, L.qkv, mx)
    q, k, v = torch.split(qkv, (L.NH * L.d, L.NKV * L.d, L.NKV * L.d), -1)
    q = rope(q.view(b, s, L.NH, L.d).transpose(1, 2), cos, sin)
    k = rope(k.view(b, s, L.NKV, L.d).transpose(1, 2), cos, sin)
    v = v.view(b, s, L.NKV, L.d).transpose(1, 2)
    o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    x = x + linear(o.transpose(1, 2).reshape(b, s, H), L.proj, mx)
    h = F.rms_norm(x, (H,), L.n2, 1e-5)
    g, u = linear(h, L.fc1, mx).split(L.FFN, -1)
    return x + linear(F.silu(g) * u, L.fc2, mx)


def main():
    global _QUANT
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--recipe", default="mxfp8", choices=["mxfp8", "bf16"])
    ap.add_argument("--compile", type=int, default=1, help="torch.compile the torch-op quantizer")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl")
    torch.manual_seed(0)
    V, H, FFN, NH, NKV = 128256, 4096, 14336, 32, 8
    mx = a.recipe == "mxfp8"
    if mx and a.compile:
        try:
            _QUANT = torch.compile(mx_quant, dynamic=False)
            _QUANT(torch.randn(256, 256, device="cuda", dtype=torch.bfloat16))
        except Exception as e:  # noqa: BLE001
            print(f"quantizer compile failed ({type(e).__name__}); running it eagerly", file=sys.stderr)
            _QUANT = mx_quant
    bf = dict(device="cuda", dtype=torch.bfloat16)
    emb = torch.nn.Parameter(torch.empty(V, H, **bf).normal_(0, 0.02))
    head = torch.nn.Parameter(torch.empty(V, H, **bf).normal_(0, 0.02))
    fnorm = torch.nn.Parameter(torch.ones(H, **bf))
    layers = [Layer(H, FFN, NH, NKV) for _ in range(a.layers)]
    params = [emb, head, fnorm] + [p for L in layers for p in L.parameters()]
    opt = torch.optim.AdamW(params, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
    d = H // NH
    inv = 1.0 / (500000.0 ** (torch.arange(0, d, 2, device="cuda").float() / d))
    ang = torch.outer(torch.arange(a.seq, device="cuda").float(), inv)
    cos = torch.cat((ang, ang), -1).cos().to(torch.bfloat16)[None, None]
    sin = torch.cat((ang, ang), -1).sin().to(torch.bfloat16)[None, None]
    gen = torch.Generator().manual_seed(1234 + rank)
    host = [torch.randint(0, V, (1, a.seq), generator=gen).pin_memory() for _ in range(4)]
    dev = [h.cuda() for h in host]

    def step(tok):
        opt.zero_grad(set_to_none=True)
        x = F.embedding(tok, emb)
        for L in layers:
            x = layer_fwd(L, x, cos, sin, mx)
        x = F.rms_norm(x, (H,), fnorm, 1e-5)
        logits = linear(x, head, mx)
        loss = F.cross_entropy(logits[0, :-1].float(), tok[0, 1:])
        loss.backward()
        if world > 1:
            for p in params:
                dist.all_reduce(p.grad, op=dist.ReduceOp.AVG)
        opt.step()
        return loss

    def timed(fn):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(a.steps):
            fn(i)
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for i in range(a.warmup):
        step(dev[i % 4])
    ms = timed(lambda i: step(dev[i % 4]))
    losses = []
    ms2 = timed(lambda i: losses.append(float(step(host[i % 4].cuda(non_blocking=True)).item())))
    if rank == 0:
        tok_s = a.seq * world * a.steps / (ms / 1e3)
        print(json.dumps({"impl": "standin", "what": "torch.nn + SDPA + torch._scaled_mm MXFP8 + AdamW(fused); not the reference",
                          "metric": "tokens_per_second", "value": tok_s, "unit": "tokens/s", "n_gpus": world,
                          "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
                          "e2e": {"value": a.seq * world * a.steps / (ms2 / 1e3), "ms_per_step": ms2 / a.steps,
                                  "last_loss": losses[-1]},
                          "config": {"model": f"llama3-8b-arch-{a.layers}L", "seq_len": a.seq, "recipe": a.recipe,
                                     "quantizer_compiled": bool(mx and _QUANT is not mx_quant),
                                     "optimizer": "torch AdamW fused on bf16 parameters (no fp32 master)",
                                     "parallelism": f"dp{world}" if world > 1 else "single"},
                          "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
