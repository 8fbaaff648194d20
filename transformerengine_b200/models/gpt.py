"""GPT-architecture decoder (GPT-2 / Megatron GPT): learned position embeddings, pre-LayerNorm blocks with biases,
tanh-GELU MLP, multi-head attention, output head tied to the token embeddings.  Every block is one
``TransformerLayer`` (LayerNorm fused into the QKV and MLP projections).  Tensor parallelism shards the blocks the
Megatron way and the embedding table / head along the vocabulary; decoding runs on the key/value cache.
(Reference: the GPT encoder of ``docs/examples/quickstart.ipynb`` and the GPT layers of ``tests/pytorch/test_numerics.py``;
this model is assembled from this library's own modules.)"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import torch

from ..modules.layernorm_linear import LayerNorm
from ..modules.linear import Linear
from ..parallel import distributed as D
from ..transformer import TransformerLayer
from .llama import VocabParallelEmbedding, _FusedCrossEntropy, _GatherFromSP


@dataclass
class GPTConfig:
    vocab_size: int = 50257
    max_positions: int = 1024
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    ffn_hidden_size: Optional[int] = None      # None: 4 * hidden_size
    layernorm_eps: float = 1e-5
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    init_std: float = 0.02
    params_dtype: torch.dtype = torch.bfloat16
    recompute: bool = False

    @property
    def ffn(self) -> int:
        return self.ffn_hidden_size or 4 * self.hidden_size

    @staticmethod
    def gpt2_small(**kw) -> "GPTConfig":
        return GPTConfig(**kw)

    @staticmethod
    def gpt2_xl(**kw) -> "GPTConfig":
        return GPTConfig(hidden_size=1600, num_layers=48, num_heads=25, **kw)

    @staticmethod
    def gpt3_175b(**kw) -> "GPTConfig":
        return GPTConfig(vocab_size=51200, max_positions=2048, hidden_size=12288, num_layers=96, num_heads=96, **kw)

    @staticmethod
    def tiny(**kw) -> "GPTConfig":
        d = dict(vocab_size=512, max_positions=64, hidden_size=128, num_layers=2, num_heads=4)
        d.update(kw)
        return GPTConfig(**d)

    def num_params(self) -> int:
        h, f = self.hidden_size, self.ffn
        per_layer = (3 * h * h + 3 * h) + (h * h + h) + (h * f + f) + (f * h + h) + 4 * h
        return self.num_layers * per_layer + (self.vocab_size + self.max_positions) * h + 2 * h


class GPTModel(torch.nn.Module):
    logits_seq_first = True  # forward returns [s, b, vocab]

    def __init__(self, cfg: GPTConfig, tp_group=None, sequence_parallel: bool = True, device=None):
        super().__init__()
        self.cfg = cfg
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.tp_group = tp_group
        self.tp_size = D.get_world_size(tp_group) if tp_group is not None else 1
        self.sp = sequence_parallel and self.tp_size > 1
        init = lambda t: torch.nn.init.normal_(t, 0.0, cfg.init_std)  # noqa: E731
        out_init = lambda t: torch.nn.init.normal_(t, 0.0, cfg.init_std / (2 * cfg.num_layers) ** 0.5)  # noqa: E731
        self.embedding = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, tp_group, self.sp, cfg.params_dtype,
                                                device, cfg.init_std)
        self.position_embedding = torch.nn.Embedding(cfg.max_positions, cfg.hidden_size, dtype=cfg.params_dtype,
                                                     device=device)
        init(self.position_embedding.weight)
        self.layers = torch.nn.ModuleList([
            TransformerLayer(cfg.hidden_size, cfg.ffn, cfg.num_heads, layernorm_epsilon=cfg.layernorm_eps,
                             hidden_dropout=cfg.hidden_dropout, attention_dropout=cfg.attention_dropout,
                             init_method=init, output_layer_init_method=out_init, layer_number=i + 1,
                             self_attn_mask_type="causal", tp_group=tp_group, tp_size=self.tp_size,
                             params_dtype=cfg.params_dtype, sequence_parallel=self.sp,
                             set_parallel_mode=self.tp_size > 1, fuse_qkv_params=True, qkv_weight_interleaved=False,
                             bias=True, activation="gelu", normalization="LayerNorm", device=device,
                             attn_input_format="sbhd")
            for i in range(cfg.num_layers)])
        self.final_norm = LayerNorm(cfg.hidden_size, eps=cfg.layernorm_eps, sequence_parallel=self.sp,
                                    params_dtype=cfg.params_dtype, device=device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, bias=False, init_method=init,
                              params_dtype=cfg.params_dtype, device=device, tp_group=tp_group, tp_size=self.tp_size,
                              parallel_mode="column" if self.tp_size > 1 else None, sequence_parallel=self.sp)
        self.lm_head.weight = self.embedding.weight     # tied (sharded along the vocabulary alike)

    def make_inference_params(self, max_batch_size: int, max_sequence_length: int, **kw):
        from ..attention.inference import InferenceParams
        cfg = self.cfg
        kw.setdefault("device", self.embedding.weight.device)
        return InferenceParams(max_batch_size, max_sequence_length, num_heads_kv=cfg.num_heads // self.tp_size,
                               head_dim_k=cfg.hidden_size // cfg.num_heads, dtype=cfg.params_dtype,
                               qkv_format="sbhd", **kw)

    def generate(self, prompt: torch.Tensor, max_new_tokens: int, **kw) -> torch.Tensor:
        from .generation import generate
        return generate(self, prompt, max_new_tokens, **kw)

    def forward(self, tokens: torch.Tensor, labels: Optional[torch.Tensor] = None, inference_params=None):
        """tokens [b, s].  Mean next-token loss when ``labels`` is given (shifted inside), else logits
        ``[s, b, vocab(/tp)]``.  With ``inference_params`` the tokens are each sequence's new tokens."""
        b, s = tokens.shape
        ids = tokens.t().contiguous()                                     # [s, b]
        pos = torch.arange(s, device=tokens.device)[:, None].expand(s, b)
        if inference_params is not None:
            assert not self.sp, "incremental decoding runs without sequence parallelism"
            pos = pos + inference_params.sequence_start_positions(b, tokens.device).to(pos.dtype)[None, :]
            pos = pos.clamp(max=self.cfg.max_positions - 1)                # padded slots past a short prompt
        x = self.embedding(ids)
        pe = self.position_embedding(pos)
        if self.sp:
            pe = pe.chunk(self.tp_size, dim=0)[D.get_rank(self.tp_group)]
        x = x + pe
        if self.cfg.hidden_dropout > 0 and self.training:
            x = torch.nn.functional.dropout(x, self.cfg.hidden_dropout)
        for layer in self.layers:
            if inference_params is not None:
                x = layer(x, inference_params=inference_params)
            elif self.cfg.recompute and torch.is_grad_enabled():
                x = D.checkpoint(layer, x)
            else:
                x = layer(x)
        logits = self.lm_head(self.final_norm(x))
        if labels is None:
            return logits
        tgt = torch.full_like(ids, -100)
        tgt[:-1] = labels.t()[1:]
        vocab_start = D.get_rank(self.tp_group) * (self.cfg.vocab_size // self.tp_size) if self.tp_size > 1 else 0
        return _FusedCrossEntropy.apply(logits, tgt, self.tp_group if self.tp_size > 1 else None, vocab_start)


# ------------------------------------------------------------------------------- Hugging Face GPT-2 checkpoints
def gpt_config_from_hf(hf_config, **overrides) -> GPTConfig:
    d = dict(vocab_size=hf_config.vocab_size, max_positions=hf_config.n_positions, hidden_size=hf_config.n_embd,
             num_layers=hf_config.n_layer, num_heads=hf_config.n_head, ffn_hidden_size=hf_config.n_inner,
             layernorm_eps=hf_config.layer_norm_epsilon)
    d.update(overrides)
    return GPTConfig(**d)


def convert_hf_gpt2_state_dict(hf_sd: Mapping[str, torch.Tensor], num_layers: int, tp_rank: int = 0,
                               tp_size: int = 1) -> Dict[str, torch.Tensor]:
    """``transformers.GPT2LMHeadModel`` state dict -> ``GPTModel`` (this rank's tensor-parallel shard).  GPT-2 stores
    its projections as ``[in, out]`` (``Conv1D``); they are transposed to the ``[out, in]`` of this library's GEMMs.
    Column-parallel matrices are cut along their output rows (q, k and v each on their own), row-parallel ones
    along their input columns, the embedding table along the vocabulary; norms, positions and the biases of the
    row-parallel layers are replicated."""
    r, n = tp_rank, tp_size
    rows = lambda w: w[r * (w.shape[0] // n):(r + 1) * (w.shape[0] // n)]           # noqa: E731
    cols = lambda w: w[:, r * (w.shape[1] // n):(r + 1) * (w.shape[1] // n)]        # noqa: E731
    wte = rows(hf_sd["transformer.wte.weight"])
    out = {"embedding.weight": wte, "lm_head.weight": wte,
           "position_embedding.weight": hf_sd["transformer.wpe.weight"],
           "final_norm.weight": hf_sd["transformer.ln_f.weight"], "final_norm.bias": hf_sd["transformer.ln_f.bias"]}
    for i in range(num_layers):
        h, t = f"transformer.h.{i}.", f"layers.{i}."
        qkv_w = hf_sd[h + "attn.c_attn.weight"].t()                     # [3h, h]: q rows, k rows, v rows
        qkv_b = hf_sd[h + "attn.c_attn.bias"]
        out.update({
            t + "self_attention.layernorm_qkv.layer_norm_weight": hf_sd[h + "ln_1.weight"],
            t + "self_attention.layernorm_qkv.layer_norm_bias": hf_sd[h + "ln_1.bias"],
            t + "self_attention.layernorm_qkv.weight": torch.cat([rows(p) for p in qkv_w.chunk(3, dim=0)]).contiguous(),
            t + "self_attention.layernorm_qkv.bias": torch.cat([rows(p) for p in qkv_b.chunk(3, dim=0)]),
            t + "self_attention.proj.weight": cols(hf_sd[h + "attn.c_proj.weight"].t()).contiguous(),
            t + "self_attention.proj.bias": hf_sd[h + "attn.c_proj.bias"],
            t + "layernorm_mlp.layer_norm_weight": hf_sd[h + "ln_2.weight"],
            t + "layernorm_mlp.layer_norm_bias": hf_sd[h + "ln_2.bias"],
            t + "layernorm_mlp.fc1_weight": rows(hf_sd[h + "mlp.c_fc.weight"].t()).contiguous(),
            t + "layernorm_mlp.fc1_bias": rows(hf_sd[h + "mlp.c_fc.bias"]),
            t + "layernorm_mlp.fc2_weight": cols(hf_sd[h + "mlp.c_proj.weight"].t()).contiguous(),
            t + "layernorm_mlp.fc2_bias": hf_sd[h + "mlp.c_proj.bias"],
        })
    return out


def load_hf_gpt2(model: GPTModel, hf_sd: Mapping[str, torch.Tensor]) -> None:
    """Fill a ``GPTModel`` (tensor-parallel or not) from a ``transformers.GPT2LMHeadModel`` state dict."""
    from .hf import _load
    rank = D.get_rank(model.tp_group) if model.tp_size > 1 else 0
    _load(model, convert_hf_gpt2_state_dict(hf_sd, model.cfg.num_layers, rank, model.tp_size))


def gpt_from_hf(hf_model, tp_group=None, device=None, **config_overrides) -> GPTModel:
    """A ``GPTModel`` with the weights of a ``transformers.GPT2LMHeadModel`` (``activation_function`` must be the
    tanh GELU, ``gelu_new``, which is GPT-2's)."""
    model = GPTModel(gpt_config_from_hf(hf_model.config, **config_overrides), tp_group=tp_group, device=device)
    load_hf_gpt2(model, hf_model.state_dict())
    return model
