"""BERT-architecture encoder: token + position + segment embeddings, post-LayerNorm blocks (the residual stream is
normalised AFTER each sub-layer), bidirectional attention with a padding mask, masked-language-model head tied to
the token embeddings and an optional pooler.  A block is one ``TransformerLayer`` in its post-norm form
(``output_layernorm=True, apply_residual_connection_post_layernorm=True``): the attention projection reads the
block input directly, the MLP's fused LayerNorm is the post-attention norm, and the layer's output norm closes the
block.  (Reference: the BERT-style layers of ``tests/pytorch/test_numerics.py``; this model is assembled from this
library's own modules.)"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import torch

from ..fusible.ops import GELU
from ..modules.layernorm_linear import LayerNorm
from ..modules.linear import Linear
from ..transformer import TransformerLayer


@dataclass
class BertConfig:
    vocab_size: int = 30522
    max_positions: int = 512
    type_vocab_size: int = 2
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    ffn_hidden_size: int = 3072
    layernorm_eps: float = 1e-12
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    init_std: float = 0.02
    add_pooler: bool = False
    params_dtype: torch.dtype = torch.bfloat16

    @staticmethod
    def bert_base(**kw) -> "BertConfig":
        return BertConfig(**kw)

    @staticmethod
    def bert_large(**kw) -> "BertConfig":
        return BertConfig(hidden_size=1024, num_layers=24, num_heads=16, ffn_hidden_size=4096, **kw)

    @staticmethod
    def tiny(**kw) -> "BertConfig":
        d = dict(vocab_size=512, max_positions=64, hidden_size=128, num_layers=2, num_heads=4, ffn_hidden_size=256)
        d.update(kw)
        return BertConfig(**d)


class BertModel(torch.nn.Module):
    def __init__(self, cfg: BertConfig, device=None):
        super().__init__()
        self.cfg = cfg
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        init = lambda t: torch.nn.init.normal_(t, 0.0, cfg.init_std)  # noqa: E731
        kw = dict(dtype=cfg.params_dtype, device=device)
        self.word_embeddings = torch.nn.Embedding(cfg.vocab_size, cfg.hidden_size, **kw)
        self.position_embeddings = torch.nn.Embedding(cfg.max_positions, cfg.hidden_size, **kw)
        self.token_type_embeddings = torch.nn.Embedding(cfg.type_vocab_size, cfg.hidden_size, **kw)
        for e in (self.word_embeddings, self.position_embeddings, self.token_type_embeddings):
            init(e.weight)
        self.embedding_norm = LayerNorm(cfg.hidden_size, eps=cfg.layernorm_eps, params_dtype=cfg.params_dtype,
                                        device=device)
        self.layers = torch.nn.ModuleList([
            TransformerLayer(cfg.hidden_size, cfg.ffn_hidden_size, cfg.num_heads, layernorm_epsilon=cfg.layernorm_eps,
                             hidden_dropout=cfg.hidden_dropout, attention_dropout=cfg.attention_dropout,
                             init_method=init, output_layer_init_method=init, layer_number=i + 1,
                             self_attn_mask_type="no_mask", params_dtype=cfg.params_dtype, fuse_qkv_params=True,
                             qkv_weight_interleaved=False, bias=True, activation="gelu", normalization="LayerNorm",
                             output_layernorm=True, apply_residual_connection_post_layernorm=True, device=device,
                             attn_input_format="sbhd")
            for i in range(cfg.num_layers)])
        # masked-language-model head: dense + GELU + LayerNorm, then the tied decoder with its own bias
        self.head_transform = Linear(cfg.hidden_size, cfg.hidden_size, bias=True, init_method=init,
                                     params_dtype=cfg.params_dtype, device=device)
        self.head_act = GELU()
        self.head_norm = LayerNorm(cfg.hidden_size, eps=cfg.layernorm_eps, params_dtype=cfg.params_dtype, device=device)
        self.decoder = Linear(cfg.hidden_size, cfg.vocab_size, bias=True, init_method=init,
                              params_dtype=cfg.params_dtype, device=device)
        self.decoder.weight = self.word_embeddings.weight
        self.pooler = Linear(cfg.hidden_size, cfg.hidden_size, bias=True, init_method=init,
                             params_dtype=cfg.params_dtype, device=device) if cfg.add_pooler else None

    def encode(self, tokens: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
               token_type_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tokens ``[b, s]``; ``attention_mask [b, s]`` with 1 / True for REAL tokens (the Hugging Face convention).
        Returns hidden states ``[s, b, hidden]`` (rows of padded positions are meaningless)."""
        b, s = tokens.shape
        pos = torch.arange(s, device=tokens.device)[None, :].expand(b, s)
        tt = torch.zeros_like(tokens) if token_type_ids is None else token_type_ids
        x = self.word_embeddings(tokens) + self.position_embeddings(pos) + self.token_type_embeddings(tt)
        x = self.embedding_norm(x).transpose(0, 1).contiguous()            # [s, b, h]
        if self.cfg.hidden_dropout > 0 and self.training:
            x = torch.nn.functional.dropout(x, self.cfg.hidden_dropout)
        if attention_mask is None:
            mask, mask_type = None, "no_mask"
        else:
            # library convention: True = masked out; a [b, 1, 1, s] mask hides padded KEYS from every query
            mask, mask_type = (~attention_mask.bool()).reshape(b, 1, 1, s), "arbitrary"
        for layer in self.layers:
            x = layer(x, attention_mask=mask, self_attn_mask_type=mask_type)
        return x

    def forward(self, tokens: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                token_type_ids: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None):
        """Masked-language-model logits ``[s, b, vocab]``, or the mean loss over positions whose ``labels [b, s]``
        are not -100."""
        x = self.encode(tokens, attention_mask, token_type_ids)
        logits = self.decoder(self.head_norm(self.head_act(self.head_transform(x))))
        if labels is None:
            return logits
        return torch.nn.functional.cross_entropy(logits.float().reshape(-1, logits.shape[-1]),
                                                 labels.t().reshape(-1), ignore_index=-100)

    def pooled(self, hidden_sbh: torch.Tensor) -> torch.Tensor:
        """tanh(dense(first token)) as in the original model; needs ``add_pooler=True``."""
        assert self.pooler is not None, "construct the model with add_pooler=True"
        return torch.tanh(self.pooler(hidden_sbh[0]))


# ------------------------------------------------------------------------------- Hugging Face BERT checkpoints
def bert_config_from_hf(hf_config, **overrides) -> BertConfig:
    d = dict(vocab_size=hf_config.vocab_size, max_positions=hf_config.max_position_embeddings,
             type_vocab_size=hf_config.type_vocab_size, hidden_size=hf_config.hidden_size,
             num_layers=hf_config.num_hidden_layers, num_heads=hf_config.num_attention_heads,
             ffn_hidden_size=hf_config.intermediate_size, layernorm_eps=hf_config.layer_norm_eps)
    d.update(overrides)
    return BertConfig(**d)


def convert_hf_bert_state_dict(hf_sd: Mapping[str, torch.Tensor], num_layers: int) -> Dict[str, torch.Tensor]:
    """``transformers.BertForMaskedLM`` state dict -> ``BertModel``."""
    e = "bert.embeddings."
    out = {"word_embeddings.weight": hf_sd[e + "word_embeddings.weight"],
           "position_embeddings.weight": hf_sd[e + "position_embeddings.weight"],
           "token_type_embeddings.weight": hf_sd[e + "token_type_embeddings.weight"],
           "embedding_norm.weight": hf_sd[e + "LayerNorm.weight"], "embedding_norm.bias": hf_sd[e + "LayerNorm.bias"],
           "head_transform.weight": hf_sd["cls.predictions.transform.dense.weight"],
           "head_transform.bias": hf_sd["cls.predictions.transform.dense.bias"],
           "head_norm.weight": hf_sd["cls.predictions.transform.LayerNorm.weight"],
           "head_norm.bias": hf_sd["cls.predictions.transform.LayerNorm.bias"],
           "decoder.weight": hf_sd[e + "word_embeddings.weight"], "decoder.bias": hf_sd["cls.predictions.bias"]}
    if "bert.pooler.dense.weight" in hf_sd:
        out["pooler.weight"], out["pooler.bias"] = hf_sd["bert.pooler.dense.weight"], hf_sd["bert.pooler.dense.bias"]
    for i in range(num_layers):
        h, t = f"bert.encoder.layer.{i}.", f"layers.{i}."
        a = h + "attention.self."
        out.update({
            t + "self_attention.qkv.weight": torch.cat([hf_sd[a + f"{x}.weight"] for x in ("query", "key", "value")]),
            t + "self_attention.qkv.bias": torch.cat([hf_sd[a + f"{x}.bias"] for x in ("query", "key", "value")]),
            t + "self_attention.proj.weight": hf_sd[h + "attention.output.dense.weight"],
            t + "self_attention.proj.bias": hf_sd[h + "attention.output.dense.bias"],
            t + "layernorm_mlp.layer_norm_weight": hf_sd[h + "attention.output.LayerNorm.weight"],
            t + "layernorm_mlp.layer_norm_bias": hf_sd[h + "attention.output.LayerNorm.bias"],
            t + "layernorm_mlp.fc1_weight": hf_sd[h + "intermediate.dense.weight"],
            t + "layernorm_mlp.fc1_bias": hf_sd[h + "intermediate.dense.bias"],
            t + "layernorm_mlp.fc2_weight": hf_sd[h + "output.dense.weight"],
            t + "layernorm_mlp.fc2_bias": hf_sd[h + "output.dense.bias"],
            t + "layernorm.weight": hf_sd[h + "output.LayerNorm.weight"],
            t + "layernorm.bias": hf_sd[h + "output.LayerNorm.bias"],
        })
    return out


def bert_from_hf(hf_model, device=None, **config_overrides) -> BertModel:
    """A ``BertModel`` with the weights of a ``transformers.BertForMaskedLM`` whose ``hidden_act`` is the tanh GELU
    (``gelu_new`` / ``gelu_pytorch_tanh``: this library's GELU; the erf form differs in the fourth decimal)."""
    from .hf import _load
    sd = hf_model.state_dict()
    cfg = bert_config_from_hf(hf_model.config, add_pooler="bert.pooler.dense.weight" in sd, **config_overrides)
    model = BertModel(cfg, device=device)
    _load(model, convert_hf_bert_state_dict(sd, cfg.num_layers))
    return model
