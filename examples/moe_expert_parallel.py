"""Mixture-of-experts training with expert parallelism: the experts of every layer are spread over the ranks, tokens
travel to their experts and back by all-to-all.

    python examples/moe_expert_parallel.py                                              # one process, all experts
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/moe_expert_parallel.py

Each MoE layer runs: router (``fused_topk_with_score_function``) -> dispatch (permute by expert, pad every expert's
slab, all-to-all; on GPUs one fused kernel writes straight into the peers' buffers) -> ``GroupedLinear`` experts with
the routing probability folded into the SwiGLU -> combine.  Attention and the router are replicated, so their
gradients are averaged over the expert-parallel group, which here is also the data-parallel group.
(Counterpart of the reference's ``examples/pytorch/ep`` and ``docs/examples/te_mixtral``.)
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200.common import recipe as R  # noqa: E402
from transformerengine_b200.models import MixtralConfig, MixtralModel  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--experts", type=int, default=4)
    ap.add_argument("--fp8", type=int, default=0)
    a = ap.parse_args(argv)

    cuda = torch.cuda.is_available()
    distributed = "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", 1)) > 1
    if distributed:
        if cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl" if cuda else "gloo")
    rank = dist.get_rank() if distributed else 0
    world = dist.get_world_size() if distributed else 1
    dev, dtype = ("cuda", torch.bfloat16) if cuda else ("cpu", torch.float32)

    torch.manual_seed(0)
    cfg = MixtralConfig.tiny(num_experts=a.experts, params_dtype=dtype, pad_align=32)
    model = MixtralModel(cfg, ep_group=dist.group.WORLD if distributed else None, device=dev)
    replicated = [p for n, p in model.named_parameters() if ".moe.fc" not in n]
    if distributed:
        for p in replicated:                                    # same start for the replicated parameters
            dist.broadcast(p.data, 0)
    opt = te.FusedAdam(model.parameters(), lr=1e-3, master_weights=(dtype != torch.float32))
    recipe = R.MXFP8BlockScaling() if a.fp8 else None

    torch.manual_seed(10 + rank)
    tokens = torch.randint(0, cfg.vocab_size, (a.batch, a.seq), device=dev)
    losses = []
    for _ in range(a.steps):
        opt.zero_grad(set_to_none=True)
        with te.autocast(enabled=recipe is not None, recipe=recipe):
            loss = model(tokens, labels=tokens)
        loss.backward()
        if distributed:
            for p in replicated:
                if p.grad is not None:
                    dist.all_reduce(p.grad)
                    p.grad.div_(world)
        opt.step()
        losses.append(float(loss.detach()))
    if rank == 0:
        per = cfg.num_experts // world
        print(f"{world} rank(s), {per} of {cfg.num_experts} experts each: loss {losses[0]:.3f} -> {losses[-1]:.3f}")
    if distributed:
        dist.destroy_process_group()
    return losses


if __name__ == "__main__":
    main()
