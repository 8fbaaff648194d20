"""Autoregressive decoding on the key/value cache for the decoder-only model families of this package.

``generate(model, prompt, max_new_tokens)`` prefills the cache with the whole prompt in one pass (prompts of
different lengths are right-padded and passed with ``prompt_lengths``), then feeds one token per sequence and
step.  The model only has to provide::

    model.make_inference_params(max_batch_size, max_sequence_length, **kw) -> InferenceParams
    model(tokens [b, s], inference_params=params) -> logits [b, s, vocab]   (or [s, b, vocab] with
                                                                            model.logits_seq_first = True)

Sampling: greedy (``temperature == 0``), temperature, top-k and nucleus (top-p) filtering; sequences that have
produced ``eos_token_id`` keep emitting ``pad_token_id`` and leave the cache (their pages go back to the pool of
a paged cache).  (Reference: the generation loop of ``docs/examples/te_gemma/te_gemma.py`` built on
``InferenceParams``; the loop here is this library's own.)
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import torch


def sample_logits(logits: torch.Tensor, temperature: float = 0.0, top_k: Optional[int] = None,
                  top_p: Optional[float] = None, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """``logits [b, vocab]`` -> token ids ``[b]``."""
    logits = logits.float()
    if temperature is None or temperature <= 0.0:
        return logits.argmax(dim=-1)
    logits = logits / temperature
    if top_k is not None and 0 < top_k < logits.shape[-1]:
        kth = torch.topk(logits, top_k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and 0.0 < top_p < 1.0:
        srt, idx = torch.sort(logits, dim=-1, descending=True)
        probs = torch.softmax(srt, dim=-1)
        before = probs.cumsum(dim=-1) - probs       # mass of the tokens ranked above this one
        srt = srt.masked_fill(before >= top_p, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, srt)
    probs = torch.softmax(logits, dim=-1)
    return torch.multinomial(probs, 1, generator=generator).squeeze(-1)


@torch.no_grad()
def generate(model, prompt: torch.Tensor, max_new_tokens: int, *, prompt_lengths: Optional[torch.Tensor] = None,
             temperature: float = 0.0, top_k: Optional[int] = None, top_p: Optional[float] = None,
             eos_token_id: Optional[int] = None, pad_token_id: int = 0, generator: Optional[torch.Generator] = None,
             inference_params=None, **cache_kwargs) -> torch.Tensor:
    """Returns ``[b, max(prompt_lengths) + max_new_tokens]`` token ids: each row holds its prompt, then the
    generated tokens, then ``pad_token_id``."""
    was_training = model.training
    model.eval()
    b, s0 = prompt.shape
    dev = prompt.device
    lens = [s0] * b if prompt_lengths is None else [int(x) for x in prompt_lengths]
    assert len(lens) == b and all(0 < n <= s0 for n in lens)
    total = max(lens) + max_new_tokens
    params = inference_params or model.make_inference_params(b, total, **cache_kwargs)
    seq_first = getattr(model, "logits_seq_first", False)

    out = torch.full((b, total), pad_token_id, dtype=prompt.dtype, device=dev)
    for i, n in enumerate(lens):
        out[i, :n] = prompt[i, :n]

    def last_logits(tokens, step_lens):
        logits = model(tokens, inference_params=params)
        if seq_first:
            logits = logits.transpose(0, 1)
        idx = torch.tensor([n - 1 for n in step_lens], device=logits.device)
        return logits[torch.arange(len(step_lens), device=logits.device), idx]

    alive = list(range(b))                        # sequence ids still decoding, in batch order of each step
    params.pre_step(OrderedDict((i, lens[i]) for i in alive))
    logits = last_logits(prompt, [lens[i] for i in alive])
    pos = list(lens)
    for step in range(max_new_tokens):
        nxt = sample_logits(logits, temperature, top_k, top_p, generator)
        keep = []
        for row, (sid, tok) in enumerate(zip(alive, nxt.tolist())):
            out[sid, pos[sid]] = tok
            pos[sid] += 1
            if eos_token_id is None or tok != eos_token_id:
                keep.append((row, sid))
        if not keep or step == max_new_tokens - 1:
            break
        rows = [r for r, _ in keep]
        alive = [sid for _, sid in keep]
        step_tokens = nxt[rows].reshape(-1, 1).to(prompt.dtype)
        params.pre_step(OrderedDict((sid, 1) for sid in alive))
        logits = last_logits(step_tokens, [1] * len(alive))
    if was_training:
        model.train()
    return out
