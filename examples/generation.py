"""Batched text generation on the key/value cache: ragged prompts, paged or contiguous cache, sampling options.

    python examples/generation.py                          # Gemma architecture, random weights
    python examples/generation.py --family qwen3 --paged 1 --temperature 0.7 --top-p 0.9

Shows ``model.generate`` (prefill once, then one token per sequence and step), ``InferenceParams`` created by
``model.make_inference_params`` and reused across calls, and sequences leaving the batch at their stop token.
(Counterpart of the generation part of the reference's ``docs/examples/te_gemma`` tutorial.)
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformerengine_b200 import models as M  # noqa: E402

FAMILIES = {"llama": ("LlamaConfig", "LlamaModel"), "mistral": ("MistralConfig", "MistralModel"),
            "gemma": ("GemmaConfig", "GemmaModel"), "qwen3": ("Qwen3Config", "Qwen3Model"),
            "gpt": ("GPTConfig", "GPTModel"), "mixtral": ("MixtralConfig", "MixtralModel")}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", default="gemma", choices=sorted(FAMILIES))
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=12, help="longest prompt; the others are shorter")
    ap.add_argument("--new-tokens", type=int, default=16)
    ap.add_argument("--paged", type=int, default=0)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    a = ap.parse_args(argv)

    cuda = torch.cuda.is_available()
    dev, dtype = ("cuda", torch.bfloat16) if cuda else ("cpu", torch.float32)
    cfg_name, model_name = FAMILIES[a.family]
    cfg = getattr(M, cfg_name).tiny(params_dtype=dtype)
    model = getattr(M, model_name)(cfg, device=dev).eval()

    torch.manual_seed(0)
    prompts = torch.randint(1, cfg.vocab_size, (a.batch, a.prompt), device=dev)
    lengths = torch.tensor([max(a.prompt - 2 * i, 1) for i in range(a.batch)])
    total = a.prompt + a.new_tokens
    cache = dict(is_paged=True, page_size=16, total_num_pages=a.batch * -(-total // 16)) if a.paged else {}
    params = model.make_inference_params(a.batch, total, **cache)

    t0 = time.perf_counter()
    out = model.generate(prompts, a.new_tokens, prompt_lengths=lengths, temperature=a.temperature, top_k=a.top_k,
                         top_p=a.top_p, eos_token_id=None, inference_params=params)
    if cuda:
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for i in range(a.batch):
        n = int(lengths[i])
        print(f"seq {i}: prompt {n:3d} tokens -> {out[i, n:n + a.new_tokens].tolist()}")
    print(f"{a.family}: {a.batch * a.new_tokens} tokens in {dt * 1e3:.1f} ms "
          f"({'paged' if a.paged else 'contiguous'} cache, {dev})")
    return out


if __name__ == "__main__":
    main()
