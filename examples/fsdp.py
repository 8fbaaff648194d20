"""Fully sharded data parallelism (PyTorch FSDP2, ``fully_shard``) over a stack of this library's layers, with the
parameters optionally created quantized so that the all-gathers move FP8 bytes and scales.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/fsdp.py
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/fsdp.py \
        --layers 8 --hidden 4096 --quantized-init mxfp8

Every ``TransformerLayer`` is one FSDP unit; its parameters are sharded along their first dimension and gathered
right before the layer runs.  With ``--quantized-init`` the parameters are ``Float8Tensor`` / ``MXFP8Tensor``
objects: their ``fsdp_pre_all_gather`` / ``fsdp_post_all_gather`` hooks hand FSDP the raw payload and rebuild the
quantized tensor on the other side, so no high-precision copy of the weights crosses the wire.
(Counterpart of the reference's ``examples/pytorch/fsdp`` and ``examples/pytorch/quantized_model_init/fully_shard.py``.)
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200.common import recipe as R  # noqa: E402

RECIPES = {"none": None, "current": R.Float8CurrentScaling, "mxfp8": R.MXFP8BlockScaling}


class Stack(torch.nn.Module):
    def __init__(self, layers):
        super().__init__()
        self.layers = torch.nn.ModuleList(layers)

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x


def main(argv=None):
    from torch.distributed.fsdp import fully_shard
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--quantized-init", default="none", choices=sorted(RECIPES),
                    help="create the parameters quantized under this recipe (and train under it)")
    a = ap.parse_args(argv)

    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl" if cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev, dtype = ("cuda", torch.bfloat16) if cuda else ("cpu", torch.float32)
    recipe = RECIPES[a.quantized_init]() if RECIPES[a.quantized_init] else None

    torch.manual_seed(0)                                        # the same initial weights on every rank
    heads = max(a.hidden // 128, 2)
    with te.quantized_model_init(enabled=recipe is not None, recipe=recipe):
        model = Stack([
            te.TransformerLayer(a.hidden, 4 * a.hidden, heads, normalization="RMSNorm", activation="swiglu", bias=False,
                                hidden_dropout=0.0, attention_dropout=0.0, self_attn_mask_type="causal",
                                fuse_qkv_params=True, params_dtype=dtype, device=dev, layer_number=i + 1)
            for i in range(a.layers)])
    for layer in model.layers:
        fully_shard(layer)
    fully_shard(model)
    layers = model.layers
    opt = te.FusedAdam([p for p in model.parameters() if p.requires_grad], lr=1e-3, master_weights=True)

    torch.manual_seed(100 + rank)                               # data parallel: every rank has its own batch
    x = torch.randn(a.seq, a.batch, a.hidden, device=dev, dtype=dtype)
    target = torch.randn_like(x)
    losses = []
    for _ in range(a.steps):
        opt.zero_grad(set_to_none=True)
        with te.autocast(enabled=recipe is not None, recipe=recipe):
            h = model(x)
        loss = (h.float() - target.float()).square().mean()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    shard = layers[0].layernorm_mlp.fc1_weight
    local = shard._local_tensor if hasattr(shard, "_local_tensor") else shard
    if rank == 0:
        print(f"world {world}, parameters {type(local).__name__} shards of shape {tuple(local.shape)}; "
              f"loss {losses[0]:.4f} -> {losses[-1]:.4f}")
    dist.destroy_process_group()
    return losses


if __name__ == "__main__":
    main()
