"""Host-side (Python) cost of one training step: cProfile over a few steps of a small-depth
model, sorted by own time.  The GPU work is asynchronous, so this shows where the launching
thread spends its time.

    python benchmarks/profile_host.py --layers 4
"""
import argparse
import cProfile
import io
import os
import pstats
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200.models import llama  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--rows", type=int, default=35)
    a = ap.parse_args()
    cfg = llama.LlamaConfig.llama3_8b(num_layers=a.layers)
    model = llama.LlamaModel(cfg)
    opt = te.FusedAdam(model.parameters(), lr=1e-4, master_weights=True)
    rec = te.recipe.MXFP8BlockScaling()
    tok = torch.randint(0, cfg.vocab_size, (1, a.seq), device="cuda")

    def step():
        opt.zero_grad(set_to_none=True)
        with te.autocast(enabled=True, recipe=rec):
            loss = model(tok, labels=tok)
        loss.backward()
        opt.step()

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    # host time of a step with the GPU queue empty at the start (launch-side cost only)
    t0 = time.perf_counter()
    step()
    t_launch = time.perf_counter() - t0
    torch.cuda.synchronize()
    t_total = time.perf_counter() - t0
    print(f"layers={a.layers}: host launch time {t_launch * 1e3:.1f} ms, step wall {t_total * 1e3:.1f} ms")
    pr = cProfile.Profile()
    pr.enable()
    for _ in range(3):
        step()
    pr.disable()
    torch.cuda.synchronize()
    s = io.StringIO()
    pstats.Stats(pr, stream=s).sort_stats("tottime").print_stats(a.rows)
    print(s.getvalue())


if __name__ == "__main__":
    main()
