"""Qwen3-architecture decoder: the Llama block with an RMSNorm over every head of the queries and keys (one weight
vector of ``head_dim`` shared by all heads) applied before the rotary embedding, and a head dimension set
independently of ``hidden_size / num_heads``."""
from __future__ import annotations

from dataclasses import dataclass

from .llama import LlamaConfig, LlamaModel


@dataclass
class Qwen3Config(LlamaConfig):
    vocab_size: int = 151936
    hidden_size: int = 4096
    num_layers: int = 36
    num_heads: int = 32
    num_kv_heads: int = 8
    ffn_hidden_size: int = 12288
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    head_dim: int = 128
    qk_norm: bool = True

    @staticmethod
    def qwen3_8b(**kw) -> "Qwen3Config":
        return Qwen3Config(**kw)

    @staticmethod
    def tiny(**kw) -> "Qwen3Config":
        d = dict(vocab_size=512, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, ffn_hidden_size=256,
                 head_dim=48)
        d.update(kw)
        return Qwen3Config(**d)


class Qwen3Model(LlamaModel):
    def __init__(self, cfg: Qwen3Config, tp_group=None, sequence_parallel: bool = True, device=None):
        super().__init__(cfg, tp_group=tp_group, sequence_parallel=sequence_parallel, device=device)
