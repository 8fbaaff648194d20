"""Which attention path a configuration takes, and why (counterpart of the reference's backend selection,
``attention/dot_product_attention/utils.py`` ``get_attention_backend``: there the choice is between FlashAttention,
cuDNN fused attention and the unfused PyTorch path; here between this library's fused kernels, the library SDPA and
the reference math).

    from transformerengine_b200.attention.utils import AttentionParams, get_attention_backend
    backend, reasons = get_attention_backend(AttentionParams(head_dim=64, attention_dropout=0.1))

The answer is a pure function of the parameters (no tensors needed), so it can be logged once at model build time;
``DotProductAttention`` itself decides per call with the same rules (``ops/attention.py``, ``ops/flash.py``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

FUSED, LIBRARY, REFERENCE = "fused_kernels", "library_sdpa", "reference_math"


@dataclass
class AttentionParams:
    qkv_dtype: torch.dtype = torch.bfloat16
    qkv_format: str = "sbhd"                  # "sbhd", "bshd" or "thd"
    num_heads: int = 16
    num_gqa_groups: int = 16
    head_dim: int = 128
    head_dim_v: Optional[int] = None
    max_seqlen_q: int = 128
    max_seqlen_kv: int = 128
    attn_mask_type: str = "causal"
    window_size: Optional[Tuple[int, int]] = None
    core_attention_bias_type: str = "no_bias"
    attention_dropout: float = 0.0
    softmax_type: str = "vanilla"
    has_attention_mask: bool = False          # an explicit (arbitrary or padding) mask tensor is passed
    score_mod: bool = False
    context_parallel: bool = False
    cp_comm_type: str = "p2p"
    fp8: bool = False
    is_training: bool = True
    device: str = "cuda"


def get_attention_backend(p: AttentionParams) -> Tuple[str, List[str]]:
    """Returns ``(backend, reasons)``: the path ``DotProductAttention`` takes for these parameters and, when it is
    not the fused kernels, every condition that rules them out."""
    from ..ops import _ext
    from ..utils.config import get_config

    why: List[str] = []
    if p.fp8:
        why.append("FP8 attention: Q, K, V, the output and the gradients are rounded to FP8 at the kernels' boundary; "
                   "the kernels themselves run in 16 bits")
    if p.device != "cuda" or not torch.cuda.is_available() or not _ext.available():
        why.append("no CUDA device / extension: the reference math runs (this is the CPU oracle path)")
        return REFERENCE, why
    if p.qkv_dtype not in (torch.bfloat16, torch.float16):
        why.append(f"dtype {p.qkv_dtype}: the kernels take fp16 / bf16")
    if p.head_dim != 128 or (p.head_dim_v or p.head_dim) != 128:
        why.append(f"head dim {p.head_dim} / {p.head_dim_v or p.head_dim}: the kernels are built for 128")
    if p.num_heads % max(p.num_gqa_groups, 1):
        why.append("query heads must be a multiple of the key / value heads")
    if p.core_attention_bias_type != "no_bias":
        why.append(f"bias ({p.core_attention_bias_type}) runs the reference math")
    if p.attention_dropout > 0.0 and p.is_training:
        why.append("attention dropout runs the reference math")
    if p.softmax_type != "vanilla":
        why.append(f"softmax_type={p.softmax_type!r} runs the reference math")
    if p.has_attention_mask or p.attn_mask_type == "arbitrary":
        why.append("an explicit mask tensor runs the reference math (padding given as cu_seqlens stays on the kernels)")
    if p.score_mod:
        why.append("score_mod runs the reference math")
    blockers = [w for w in why if "FP8" not in w]
    if not blockers:
        if get_config().attention_backend == "library":
            return LIBRARY, ["attention_backend='library' was requested (A/B timing)"]
        if get_config().attention_backend == "reference":
            return REFERENCE, ["attention_backend='reference' was requested (numerics debugging)"]
        return FUSED, [w for w in why if "FP8" in w]
    windowed = p.window_size is not None and (p.window_size[0] >= 0 or p.window_size[1] > 0)
    plain = not any(k in w for w in blockers for k in ("bias", "dropout", "softmax_type", "mask", "score_mod"))
    if plain and not windowed and p.qkv_format != "thd" and not p.context_parallel \
            and p.qkv_dtype in (torch.bfloat16, torch.float16) and get_config().attention_backend != "reference":
        return LIBRARY, why
    return REFERENCE, why
