"""T5-architecture encoder-decoder (v1.1 form): pre-RMSNorm blocks without biases, gated tanh-GELU MLPs, learned
relative-position biases added to the attention scores (one table per stack, shared by its layers), decoder blocks
with causal self-attention followed by cross-attention over the encoder output.

An encoder block is a ``TransformerLayer(layer_type="encoder")``, a decoder block a
``TransformerLayer(layer_type="decoder")`` (self-attention, cross-attention with the norm fused into the query
projection, MLP); the position bias goes in as ``core_attention_bias`` of type ``post_scale_bias``.  The original
model does not scale the scores by ``1/sqrt(d)``: the library's attention does, so a converted checkpoint's query
projections are multiplied by ``sqrt(d)`` once at load time, which is the same function.
(Reference: the encoder / decoder ``layer_type`` of ``pytorch/transformer.py`` and the T5-style layers of
``tests/pytorch/test_numerics.py``; this model is assembled from this library's own modules.)"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import torch

from ..modules.layernorm_linear import RMSNorm
from ..modules.linear import Linear
from ..transformer import TransformerLayer


@dataclass
class T5Config:
    vocab_size: int = 32128
    hidden_size: int = 768
    head_dim: int = 64
    num_heads: int = 12
    ffn_hidden_size: int = 2048
    num_layers: int = 12                     # encoder blocks
    num_decoder_layers: Optional[int] = None  # None: same as the encoder
    relative_buckets: int = 32
    relative_max_distance: int = 128
    rms_eps: float = 1e-6
    activation: str = "geglu"                # v1.1; "relu" is the original model's MLP
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    init_std: float = 0.02
    decoder_start_token_id: int = 0
    tie_embeddings: bool = False             # the head shares the embedding table
    scale_decoder_outputs: bool = False      # original T5 (not v1.1): the head reads hidden_size ** -0.5 * output
    params_dtype: torch.dtype = torch.bfloat16

    @property
    def decoder_layers(self) -> int:
        return self.num_layers if self.num_decoder_layers is None else self.num_decoder_layers

    @staticmethod
    def t5_v1_1_base(**kw) -> "T5Config":
        return T5Config(**kw)

    @staticmethod
    def t5_v1_1_xxl(**kw) -> "T5Config":
        return T5Config(hidden_size=4096, num_heads=64, ffn_hidden_size=10240, num_layers=24, **kw)

    @staticmethod
    def tiny(**kw) -> "T5Config":
        d = dict(vocab_size=512, hidden_size=128, head_dim=32, num_heads=4, ffn_hidden_size=256, num_layers=2,
                 relative_buckets=8, relative_max_distance=16)
        d.update(kw)
        return T5Config(**d)


def relative_position_bucket(rel: torch.Tensor, bidirectional: bool, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bucket index of ``rel = key position - query position``: exact buckets for small offsets, log-spaced ones up
    to ``max_distance``, one shared bucket beyond.  Bidirectional stacks spend half of the buckets on each sign; a
    causal stack only looks back."""
    bucket = torch.zeros_like(rel)
    if bidirectional:
        num_buckets //= 2
        bucket = bucket + (rel > 0).to(rel.dtype) * num_buckets
        rel = rel.abs()
    else:
        rel = -torch.clamp(rel, max=0)
    exact = num_buckets // 2
    large = exact + (torch.log(rel.float().clamp(min=1) / exact) / math.log(max_distance / exact)
                     * (num_buckets - exact)).to(rel.dtype)
    large = torch.clamp(large, max=num_buckets - 1)
    return bucket + torch.where(rel < exact, rel, large)


class RelativePositionBias(torch.nn.Module):
    """``[1, heads, s_q, s_k]`` additive score bias from a ``[buckets, heads]`` table."""

    def __init__(self, cfg: T5Config, bidirectional: bool, device=None):
        super().__init__()
        self.bidirectional, self.buckets, self.max_distance = bidirectional, cfg.relative_buckets, cfg.relative_max_distance
        self.table = torch.nn.Embedding(cfg.relative_buckets, cfg.num_heads, dtype=cfg.params_dtype, device=device)
        torch.nn.init.normal_(self.table.weight, 0.0, cfg.init_std)

    def forward(self, sq: int, sk: int) -> torch.Tensor:
        dev = self.table.weight.device
        # queries are the LAST sq positions of the sk keys (sq == sk in training, sq < sk never occurs here)
        qpos = torch.arange(sk - sq, sk, device=dev)[:, None]
        kpos = torch.arange(sk, device=dev)[None, :]
        idx = relative_position_bucket(kpos - qpos, self.bidirectional, self.buckets, self.max_distance)
        return self.table(idx).permute(2, 0, 1)[None].contiguous()


class T5Model(torch.nn.Module):
    def __init__(self, cfg: T5Config, device=None):
        super().__init__()
        self.cfg = cfg
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        init = lambda t: torch.nn.init.normal_(t, 0.0, cfg.init_std)  # noqa: E731
        self.shared = torch.nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=cfg.params_dtype, device=device)
        init(self.shared.weight)

        def block(i, kind):
            return TransformerLayer(cfg.hidden_size, cfg.ffn_hidden_size, cfg.num_heads, kv_channels=cfg.head_dim,
                                    layernorm_epsilon=cfg.rms_eps, hidden_dropout=cfg.hidden_dropout,
                                    attention_dropout=cfg.attention_dropout, init_method=init,
                                    output_layer_init_method=init, layer_number=i + 1,
                                    self_attn_mask_type="causal" if kind == "decoder" else "no_mask",
                                    enc_dec_attn_mask_type="no_mask", params_dtype=cfg.params_dtype,
                                    fuse_qkv_params=True, qkv_weight_interleaved=False, bias=False,
                                    activation=cfg.activation, normalization="RMSNorm", layer_type=kind,
                                    device=device, attn_input_format="sbhd")

        self.encoder = torch.nn.ModuleList([block(i, "encoder") for i in range(cfg.num_layers)])
        self.decoder = torch.nn.ModuleList([block(i, "decoder") for i in range(cfg.decoder_layers)])
        self.encoder_bias = RelativePositionBias(cfg, True, device)
        self.decoder_bias = RelativePositionBias(cfg, False, device)
        norm = dict(eps=cfg.rms_eps, params_dtype=cfg.params_dtype, device=device)
        self.encoder_norm, self.decoder_norm = RMSNorm(cfg.hidden_size, **norm), RMSNorm(cfg.hidden_size, **norm)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, bias=False, init_method=init,
                              params_dtype=cfg.params_dtype, device=device)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.shared.weight

    @staticmethod
    def _key_mask(attention_mask, b, s):
        """Hugging Face mask (1 = real token) -> the library's ``[b, 1, 1, s]`` mask (True = hidden key)."""
        return None if attention_mask is None else (~attention_mask.bool()).reshape(b, 1, 1, s)

    def encode(self, tokens: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tokens ``[b, s]`` -> encoder output ``[s, b, hidden]``."""
        b, s = tokens.shape
        x = self.shared(tokens).transpose(0, 1).contiguous()
        bias = self.encoder_bias(s, s).to(x.dtype)
        mask = self._key_mask(attention_mask, b, s)
        for layer in self.encoder:
            x = layer(x, attention_mask=mask, self_attn_mask_type="arbitrary" if mask is not None else "no_mask",
                      core_attention_bias_type="post_scale_bias", core_attention_bias=bias)
        return self.encoder_norm(x)

    def decode(self, decoder_tokens: torch.Tensor, encoder_output: torch.Tensor,
               attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """decoder tokens ``[b, t]`` and encoder output ``[s, b, hidden]`` -> logits ``[t, b, vocab]``."""
        b, t = decoder_tokens.shape
        y = self.shared(decoder_tokens).transpose(0, 1).contiguous()
        bias = self.decoder_bias(t, t).to(y.dtype)
        mask = self._key_mask(attention_mask, b, encoder_output.shape[0])
        for layer in self.decoder:
            y = layer(y, encoder_output=encoder_output, enc_dec_attn_mask=mask,
                      enc_dec_attn_mask_type="arbitrary" if mask is not None else "no_mask",
                      core_attention_bias_type="post_scale_bias", core_attention_bias=bias)
        y = self.decoder_norm(y)
        if self.cfg.scale_decoder_outputs:
            y = y * (self.cfg.hidden_size ** -0.5)
        return self.lm_head(y)

    def shift_right(self, labels: torch.Tensor) -> torch.Tensor:
        """Decoder inputs of teacher forcing: the start token, then the labels (ignored positions become pad 0)."""
        start = torch.full_like(labels[:, :1], self.cfg.decoder_start_token_id)
        return torch.cat([start, labels[:, :-1]], dim=1).masked_fill_(
            torch.cat([torch.zeros_like(start, dtype=torch.bool), labels[:, :-1] == -100], dim=1), 0)

    def forward(self, tokens: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                decoder_tokens: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None):
        """Logits ``[t, b, vocab]`` for ``decoder_tokens``; with ``labels [b, t]`` the decoder inputs are the labels
        shifted right and the mean loss over labels != -100 is returned."""
        if decoder_tokens is None:
            assert labels is not None, "pass decoder_tokens or labels"
            decoder_tokens = self.shift_right(labels)
        logits = self.decode(decoder_tokens, self.encode(tokens, attention_mask), attention_mask)
        if labels is None:
            return logits
        return torch.nn.functional.cross_entropy(logits.float().reshape(-1, logits.shape[-1]),
                                                 labels.t().reshape(-1), ignore_index=-100)

    @torch.no_grad()
    def generate(self, tokens: torch.Tensor, max_new_tokens: int, attention_mask: Optional[torch.Tensor] = None,
                 eos_token_id: Optional[int] = None) -> torch.Tensor:
        """Greedy decoding: the encoder runs once, the decoder re-reads its own prefix at every step."""
        was_training = self.training
        self.eval()
        enc = self.encode(tokens, attention_mask)
        out = torch.full((tokens.shape[0], 1), self.cfg.decoder_start_token_id, dtype=tokens.dtype, device=tokens.device)
        done = torch.zeros(tokens.shape[0], dtype=torch.bool, device=tokens.device)
        for _ in range(max_new_tokens):
            nxt = self.decode(out, enc, attention_mask)[-1].float().argmax(-1)
            nxt = nxt.masked_fill(done, 0)
            out = torch.cat([out, nxt[:, None].to(out.dtype)], dim=1)
            if eos_token_id is not None:
                done |= nxt == eos_token_id
                if bool(done.all()):
                    break
        if was_training:
            self.train()
        return out


# --------------------------------------------------------------------------------- Hugging Face T5 checkpoints
def t5_config_from_hf(hf_config, **overrides) -> T5Config:
    act = {"gated-gelu": "geglu", "relu": "relu", "gated-silu": "swiglu"}.get(hf_config.feed_forward_proj)
    if act is None:
        raise ValueError(f"feed_forward_proj={hf_config.feed_forward_proj!r} has no counterpart here")
    d = dict(vocab_size=hf_config.vocab_size, hidden_size=hf_config.d_model, head_dim=hf_config.d_kv,
             num_heads=hf_config.num_heads, ffn_hidden_size=hf_config.d_ff, num_layers=hf_config.num_layers,
             num_decoder_layers=hf_config.num_decoder_layers, relative_buckets=hf_config.relative_attention_num_buckets,
             relative_max_distance=hf_config.relative_attention_max_distance, rms_eps=hf_config.layer_norm_epsilon,
             activation=act, decoder_start_token_id=hf_config.decoder_start_token_id or 0,
             tie_embeddings=bool(getattr(hf_config, "tie_word_embeddings", False)),
             scale_decoder_outputs=bool(getattr(hf_config, "scale_decoder_outputs",
                                                getattr(hf_config, "tie_word_embeddings", False))))
    d.update(overrides)
    return T5Config(**d)


def convert_hf_t5_state_dict(hf_sd: Mapping[str, torch.Tensor], cfg: T5Config) -> Dict[str, torch.Tensor]:
    """``transformers.T5ForConditionalGeneration`` state dict -> ``T5Model``."""
    qs = math.sqrt(cfg.head_dim)       # the library scales scores by 1/sqrt(d); the checkpoint's model does not
    gated = cfg.activation != "relu"
    out = {"shared.weight": hf_sd["shared.weight"],
           "lm_head.weight": hf_sd["shared.weight"] if cfg.tie_embeddings else hf_sd.get("lm_head.weight",
                                                                                         hf_sd["shared.weight"]),
           "encoder_norm.weight": hf_sd["encoder.final_layer_norm.weight"],
           "decoder_norm.weight": hf_sd["decoder.final_layer_norm.weight"],
           "encoder_bias.table.weight": hf_sd["encoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight"],
           "decoder_bias.table.weight": hf_sd["decoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight"]}

    def mlp(h, t):
        ff = h + "DenseReluDense."
        fc1 = torch.cat([hf_sd[ff + "wi_0.weight"], hf_sd[ff + "wi_1.weight"]]) if gated else hf_sd[ff + "wi.weight"]
        return {t + "layernorm_mlp.layer_norm_weight": hf_sd[h + "layer_norm.weight"],
                t + "layernorm_mlp.fc1_weight": fc1, t + "layernorm_mlp.fc2_weight": hf_sd[ff + "wo.weight"]}

    def self_attn(h, t):
        a = h + "SelfAttention."
        return {t + "self_attention.layernorm_qkv.layer_norm_weight": hf_sd[h + "layer_norm.weight"],
                t + "self_attention.layernorm_qkv.weight": torch.cat([hf_sd[a + "q.weight"] * qs, hf_sd[a + "k.weight"],
                                                                      hf_sd[a + "v.weight"]]),
                t + "self_attention.proj.weight": hf_sd[a + "o.weight"]}

    for i in range(cfg.num_layers):
        h, t = f"encoder.block.{i}.layer.", f"encoder.{i}."
        out.update(self_attn(h + "0.", t))
        out.update(mlp(h + "1.", t))
    for i in range(cfg.decoder_layers):
        h, t = f"decoder.block.{i}.layer.", f"decoder.{i}."
        out.update(self_attn(h + "0.", t))
        c = h + "1.EncDecAttention."
        out.update({t + "inter_attention.layernorm_query.layer_norm_weight": hf_sd[h + "1.layer_norm.weight"],
                    t + "inter_attention.layernorm_query.weight": hf_sd[c + "q.weight"] * qs,
                    t + "inter_attention.key_value.weight": torch.cat([hf_sd[c + "k.weight"], hf_sd[c + "v.weight"]]),
                    t + "inter_attention.proj.weight": hf_sd[c + "o.weight"]})
        out.update(mlp(h + "2.", t))
    return out


def t5_from_hf(hf_model, device=None, **config_overrides) -> T5Model:
    """A ``T5Model`` with the weights of a ``transformers.T5ForConditionalGeneration`` (tied or untied head; ReLU
    or gated MLP)."""
    from .hf import _load
    cfg = t5_config_from_hf(hf_model.config, **config_overrides)
    model = T5Model(cfg, device=device)
    _load(model, convert_hf_t5_state_dict(hf_model.state_dict(), cfg))
    return model
