"""Per-kernel time table of one training step (torch.profiler, CUDA activity only).

    python benchmarks/profile_step.py --layers 2 [--seq 8192] [--recipe mxfp8] [--model llama|mixtral]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200.models import llama, mixtral  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--recipe", default="mxfp8")
    ap.add_argument("--rows", type=int, default=40)
    ap.add_argument("--model", default="llama", choices=["llama", "mixtral"])
    a = ap.parse_args()
    if a.model == "mixtral":
        cfg = mixtral.MixtralConfig.mixtral_8x7b(num_layers=a.layers)
        model = mixtral.MixtralModel(cfg)
    else:
        cfg = llama.LlamaConfig.llama3_8b(num_layers=a.layers)
        model = llama.LlamaModel(cfg)
    opt = te.FusedAdam(model.parameters(), lr=1e-4, master_weights=True)
    rec = te.recipe.MXFP8BlockScaling() if a.recipe == "mxfp8" else None
    tok = torch.randint(0, cfg.vocab_size, (1, a.seq), device="cuda")

    def step():
        opt.zero_grad(set_to_none=True)
        with te.autocast(enabled=rec is not None, recipe=rec):
            loss = model(tok, labels=tok)
        loss.backward()
        opt.step()

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=a.rows, max_name_column_width=70))


if __name__ == "__main__":
    main()
