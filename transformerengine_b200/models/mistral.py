"""Mistral-architecture decoder: the Llama block with sliding-window causal attention (each token attends to the
last ``sliding_window`` tokens; the attention kernels skip the key blocks left of the window)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .llama import LlamaConfig, LlamaModel


@dataclass
class MistralConfig(LlamaConfig):
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    ffn_hidden_size: int = 14336
    rope_theta: float = 10000.0
    sliding_window: Optional[int] = 4096

    @staticmethod
    def mistral_7b(**kw) -> "MistralConfig":
        return MistralConfig(**kw)

    @staticmethod
    def tiny(**kw) -> "MistralConfig":
        d = dict(vocab_size=512, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, ffn_hidden_size=256,
                 sliding_window=8)
        d.update(kw)
        return MistralConfig(**d)


class MistralModel(LlamaModel):
    def __init__(self, cfg: MistralConfig, tp_group=None, sequence_parallel: bool = True, device=None):
        super().__init__(cfg, tp_group=tp_group, sequence_parallel=sequence_parallel, device=device)
