"""Quick start: a small GPT-style stack trained for a few steps under a low-precision recipe, saved and restored.

    python examples/quickstart.py                       # one GPU (or CPU: the reference path runs the same code)
    python examples/quickstart.py --recipe nvfp4 --steps 20
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/quickstart.py --tp 2

What it shows: ``te.TransformerLayer`` with RMSNorm / SwiGLU / grouped-query attention and rotary embeddings,
``te.autocast`` with a recipe object, ``te.FusedAdam`` with fp32 master weights, tensor + sequence parallelism with
the fused collective GEMMs (``te.initialize_ub``), and a state dict round trip that keeps the FP8 metadata.
(Counterpart of the reference's ``examples/pytorch`` scripts and ``docs/examples/quickstart.ipynb``.)
"""
import argparse
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200.common import recipe as R  # noqa: E402

RECIPES = {"bf16": None, "delayed": R.DelayedScaling, "current": R.Float8CurrentScaling, "mxfp8": R.MXFP8BlockScaling,
           "block": R.Float8BlockScaling, "nvfp4": R.NVFP4BlockScaling}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--recipe", default="mxfp8", choices=sorted(RECIPES))
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--hidden", type=int, default=512)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (launch with torch.distributed.run)")
    a = ap.parse_args(argv)

    cuda = torch.cuda.is_available()
    tp_group = None
    if a.tp > 1:
        local = int(os.environ.get("LOCAL_RANK", 0))
        if cuda:
            torch.cuda.set_device(local)
        dist.init_process_group("nccl" if cuda else "gloo")
        tp_group = dist.group.WORLD
        if cuda:
            te.initialize_ub(tp_group=tp_group)       # fused all-gather -> GEMM / GEMM -> reduce-scatter kernels
    dev = "cuda" if cuda else "cpu"
    dtype = torch.bfloat16 if cuda else torch.float32
    heads = max(a.hidden // 128, 2)
    torch.manual_seed(1234 + (dist.get_rank() if a.tp > 1 else 0))

    layers = torch.nn.ModuleList([
        te.TransformerLayer(a.hidden, 4 * a.hidden, heads, num_gqa_groups=max(heads // 2, 1), normalization="RMSNorm",
                            activation="swiglu", bias=False, hidden_dropout=0.0, attention_dropout=0.0,
                            self_attn_mask_type="causal", fuse_qkv_params=True, params_dtype=dtype, device=dev,
                            tp_group=tp_group, tp_size=a.tp, set_parallel_mode=a.tp > 1, sequence_parallel=a.tp > 1,
                            layer_number=i + 1)
        for i in range(a.layers)])
    rope = te.RotaryPositionEmbedding(a.hidden // heads)(a.seq).to(dev)
    opt = te.FusedAdam(layers.parameters(), lr=3e-4, master_weights=(dtype != torch.float32))
    recipe = RECIPES[a.recipe]() if RECIPES[a.recipe] is not None else None

    seq_local = a.seq // a.tp                          # sequence parallelism: every rank holds a slice of the tokens
    target = torch.randn(seq_local, a.batch, a.hidden, device=dev, dtype=dtype)
    x = torch.randn(seq_local, a.batch, a.hidden, device=dev, dtype=dtype)
    losses = []
    for step in range(a.steps):
        opt.zero_grad(set_to_none=True)
        h = x
        with te.autocast(enabled=recipe is not None, recipe=recipe):
            for layer in layers:
                h = layer(h, rotary_pos_emb=rope)
        loss = (h.float() - target.float()).square().mean()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    if cuda:
        te.check_status()                              # raises if a bounded device wait ran out

    # state dict round trip: quantization metadata travels in the _extra_state entries
    buf = io.BytesIO()
    torch.save(layers.state_dict(), buf)
    buf.seek(0)
    layers.load_state_dict(torch.load(buf, weights_only=False))
    if a.tp == 1 or dist.get_rank() == 0:
        print(f"recipe={a.recipe} device={dev} tp={a.tp} loss {losses[0]:.4f} -> {losses[-1]:.4f} over {a.steps} steps")
    if a.tp > 1:
        te.destroy_ub()
        dist.destroy_process_group()
    return losses


if __name__ == "__main__":
    main()
