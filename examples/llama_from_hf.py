"""Take a Hugging Face Llama checkpoint, train it with this library's kernels, decode from it, and hand it back.

    python examples/llama_from_hf.py                          # random tiny Llama made from a transformers config
    python examples/llama_from_hf.py --hf-path /ckpt/llama-3-8b --recipe mxfp8 --steps 50 --seq 2048

Steps: (1) build or load a ``transformers.LlamaForCausalLM``; (2) ``models.hf.llama_from_hf`` fuses its q/k/v and
gate/up matrices into this library's ``LlamaModel`` (the logits agree to fp32 rounding, which the script checks);
(3) a few optimizer steps under ``te.autocast`` with the chosen recipe; (4) ``model.generate`` on the key/value
cache; (5) ``export_hf_llama_state_dict`` loads back into the Hugging Face model.
(Counterpart of the reference's ``docs/examples/te_llama`` tutorial.)
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200.common import recipe as R  # noqa: E402
from transformerengine_b200.models import hf  # noqa: E402

RECIPES = {"none": None, "delayed": R.DelayedScaling, "current": R.Float8CurrentScaling, "mxfp8": R.MXFP8BlockScaling,
           "nvfp4": R.NVFP4BlockScaling}


def main(argv=None):
    import transformers
    ap = argparse.ArgumentParser()
    ap.add_argument("--hf-path", default=None, help="local directory of a Llama checkpoint (default: random tiny model)")
    ap.add_argument("--recipe", default="none", choices=sorted(RECIPES))
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--new-tokens", type=int, default=8)
    a = ap.parse_args(argv)

    cuda = torch.cuda.is_available()
    dev, dtype = ("cuda", torch.bfloat16) if cuda else ("cpu", torch.float32)
    if a.hf_path:
        ref = transformers.LlamaForCausalLM.from_pretrained(a.hf_path, torch_dtype=dtype)
    else:
        ref = transformers.LlamaForCausalLM(transformers.LlamaConfig(
            vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=4096, tie_word_embeddings=False,
            attn_implementation="eager")).to(dtype)
    ref = ref.to(dev).eval()
    model = hf.llama_from_hf(ref, device=dev, params_dtype=dtype)

    vocab = model.cfg.vocab_size
    tokens = torch.randint(0, vocab, (a.batch, a.seq), device=dev)
    with torch.no_grad():
        want = ref(tokens).logits.float()
        got = model.eval()(tokens).transpose(0, 1).float()
    err = float((got - want).abs().max())
    print(f"converted: max |logit difference| to the Hugging Face model = {err:.2e}")

    model.train()
    opt = te.FusedAdam(model.parameters(), lr=1e-4, master_weights=(dtype != torch.float32))
    recipe = RECIPES[a.recipe]() if RECIPES[a.recipe] else None
    losses = []
    for _ in range(a.steps):
        opt.zero_grad(set_to_none=True)
        with te.autocast(enabled=recipe is not None, recipe=recipe):
            loss = model(tokens, labels=tokens)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    print(f"trained {a.steps} steps ({a.recipe}): loss {losses[0]:.3f} -> {losses[-1]:.3f}")

    out = model.generate(tokens[:, :8], a.new_tokens, temperature=0.8, top_p=0.95)
    print("generated:", out[0, 8:].tolist())

    ref.load_state_dict(hf.export_hf_llama_state_dict(model))
    with torch.no_grad():
        back = float((ref(tokens).logits.float() - model.eval()(tokens).transpose(0, 1).float()).abs().max())
    print(f"exported back: max |logit difference| = {back:.2e}")
    return err, losses, back


if __name__ == "__main__":
    main()
