"""Encoder-decoder training: a small T5 learns to reverse token sequences, then decodes greedily.

    python examples/seq2seq_t5.py --steps 300

Shows ``TransformerLayer(layer_type="decoder")`` with cross-attention over an encoder output, relative position
biases passed as ``core_attention_bias``, padding masks on the encoder keys, teacher forcing with shifted labels.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import transformerengine_b200 as te  # noqa: E402
from transformerengine_b200.common import recipe as R  # noqa: E402
from transformerengine_b200.models import T5Config, T5Model  # noqa: E402


def batch_of(n, length, vocab, dev):
    """Source sequences of random lengths (right-padded with 0) and their reversals, closed by the stop token 1."""
    src = torch.zeros(n, length, dtype=torch.long, device=dev)
    tgt = torch.full((n, length + 1), -100, dtype=torch.long, device=dev)
    mask = torch.zeros(n, length, dtype=torch.long, device=dev)
    for i in range(n):
        k = int(torch.randint(length // 2, length + 1, (1,)))
        seq = torch.randint(2, vocab, (k,), device=dev)
        src[i, :k], mask[i, :k] = seq, 1
        tgt[i, :k], tgt[i, k] = seq.flip(0), 1
    return src, mask, tgt


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--length", type=int, default=8)
    ap.add_argument("--vocab", type=int, default=32)
    ap.add_argument("--fp8", type=int, default=0, help="1: run the GEMMs under the MXFP8 recipe")
    a = ap.parse_args(argv)
    cuda = torch.cuda.is_available()
    dev, dtype = ("cuda", torch.bfloat16) if cuda else ("cpu", torch.float32)
    torch.manual_seed(0)
    model = T5Model(T5Config.tiny(vocab_size=a.vocab, params_dtype=dtype, tie_embeddings=True), device=dev)
    opt = te.FusedAdam(model.parameters(), lr=3e-3, master_weights=(dtype != torch.float32))
    recipe = R.MXFP8BlockScaling() if a.fp8 else None
    losses = []
    for _ in range(a.steps):
        src, mask, tgt = batch_of(a.batch, a.length, a.vocab, dev)
        opt.zero_grad(set_to_none=True)
        with te.autocast(enabled=recipe is not None, recipe=recipe):
            loss = model(src, mask, labels=tgt)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    src, mask, tgt = batch_of(4, a.length, a.vocab, dev)
    out = model.generate(src, a.length + 1, mask, eos_token_id=1)
    for i in range(4):
        k = int(mask[i].sum())
        print("source  ", src[i, :k].tolist(), "\ndecoded ", out[i, 1:k + 2].tolist())
    print(f"loss {losses[0]:.3f} -> {sum(losses[-10:]) / len(losses[-10:]):.3f} over {a.steps} steps")
    return losses


if __name__ == "__main__":
    main()
