"""Gemma-architecture decoder: the Llama block with GeGLU (tanh GELU), RMSNorm weights stored as ``gamma - 1``,
a head dimension that is set independently of ``hidden_size / num_heads`` (256), token embeddings scaled by
``sqrt(hidden_size)`` and an output head tied to the embedding table.  Decoding on the key/value cache comes from
``LlamaModel.generate``.  (Reference: ``docs/examples/te_gemma``; this model is assembled from this library's own
modules.)"""
from __future__ import annotations

from dataclasses import dataclass

from .llama import LlamaConfig, LlamaModel


@dataclass
class GemmaConfig(LlamaConfig):
    vocab_size: int = 256000
    hidden_size: int = 3072
    num_layers: int = 28
    num_heads: int = 16
    num_kv_heads: int = 16
    ffn_hidden_size: int = 24576
    rms_eps: float = 1e-6
    rope_theta: float = 10000.0
    head_dim: int = 256
    activation: str = "geglu"
    zero_centered_gamma: bool = True
    tie_embeddings: bool = True

    def __post_init__(self):
        if self.embedding_scale is None:
            self.embedding_scale = float(self.hidden_size) ** 0.5

    @staticmethod
    def gemma_7b(**kw) -> "GemmaConfig":
        return GemmaConfig(**kw)

    @staticmethod
    def gemma_2b(**kw) -> "GemmaConfig":
        d = dict(hidden_size=2048, num_layers=18, num_heads=8, num_kv_heads=1, ffn_hidden_size=16384)
        d.update(kw)
        return GemmaConfig(**d)

    @staticmethod
    def tiny(**kw) -> "GemmaConfig":
        d = dict(vocab_size=512, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=1, ffn_hidden_size=256,
                 head_dim=64)
        d.update(kw)
        return GemmaConfig(**d)


class GemmaModel(LlamaModel):
    def __init__(self, cfg: GemmaConfig, tp_group=None, sequence_parallel: bool = True, device=None):
        super().__init__(cfg, tp_group=tp_group, sequence_parallel=sequence_parallel, device=device)
