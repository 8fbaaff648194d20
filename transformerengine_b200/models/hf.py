"""Hugging Face checkpoints <-> this package's models (Llama, Mistral, Gemma, Qwen3, Mixtral).

The Hugging Face layouts keep one matrix per projection; the models here fuse them the way the kernels want
them (one QKV GEMM, one gate+up GEMM, one grouped GEMM per expert set):

====================================================  =====================================================
Hugging Face                                           here
====================================================  =====================================================
``model.embed_tokens.weight``                          ``embedding.weight``
``…layers.i.input_layernorm.weight``                   ``layers.i.self_attention.layernorm_qkv.layer_norm_weight``
``…self_attn.{q,k,v}_proj.weight`` (three)             ``…self_attention.layernorm_qkv.weight`` = cat(q, k, v)
``…self_attn.o_proj.weight``                           ``…self_attention.proj.weight``
``…post_attention_layernorm.weight``                   ``…layernorm_mlp.layer_norm_weight``
``…mlp.{gate,up}_proj.weight`` (two)                   ``…layernorm_mlp.fc1_weight`` = cat(gate, up)
``…mlp.down_proj.weight``                              ``…layernorm_mlp.fc2_weight``
``model.norm.weight`` / ``lm_head.weight``             ``final_norm.weight`` / ``lm_head.weight``
====================================================  =====================================================

Both rotate-half conventions agree (the Hugging Face q/k projections are stored for the non-interleaved
rotation, which is this library's default), so no row permutation is needed.  With tensor parallelism every rank
converts the full checkpoint and keeps its shard (``tp_rank`` / ``tp_size``): column-parallel matrices are cut
along the output rows PER PROJECTION (q, k, v, gate and up separately), row-parallel ones along the input
columns, embeddings and the head along the vocabulary.
(Reference: the weight mapping of ``docs/examples/te_llama/te_llama.py`` and ``te_gemma``; the code here is this
library's own and also goes the other way.)
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch


def _rows(w: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    n = w.shape[0] // size
    return w[rank * n:(rank + 1) * n]


def _cols(w: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    n = w.shape[1] // size
    return w[:, rank * n:(rank + 1) * n]


# ------------------------------------------------------------------------------------------------ Llama
def _common_fields(hf_config) -> dict:
    rope_theta = getattr(hf_config, "rope_theta", None)
    if rope_theta is None:
        rp = getattr(hf_config, "rope_parameters", None) or {}
        rope_theta = rp.get("rope_theta", 10000.0)
    return dict(vocab_size=hf_config.vocab_size, hidden_size=hf_config.hidden_size,
                num_layers=hf_config.num_hidden_layers, num_heads=hf_config.num_attention_heads,
                num_kv_heads=getattr(hf_config, "num_key_value_heads", None) or hf_config.num_attention_heads,
                ffn_hidden_size=hf_config.intermediate_size, rms_eps=hf_config.rms_norm_eps,
                rope_theta=float(rope_theta))


def llama_config_from_hf(hf_config, **overrides):
    """``LlamaConfig`` of this package from a ``transformers.LlamaConfig`` (or any object with its fields)."""
    from .llama import LlamaConfig
    d = _common_fields(hf_config)
    if getattr(hf_config, "head_dim", None) and hf_config.head_dim != d["hidden_size"] // d["num_heads"]:
        d["head_dim"] = hf_config.head_dim
    d["tie_embeddings"] = bool(getattr(hf_config, "tie_word_embeddings", False))
    d.update(overrides)
    return LlamaConfig(**d)


def mistral_config_from_hf(hf_config, **overrides):
    from .mistral import MistralConfig
    d = _common_fields(hf_config)
    d["sliding_window"] = getattr(hf_config, "sliding_window", None)
    if getattr(hf_config, "head_dim", None):
        d["head_dim"] = hf_config.head_dim
    d.update(overrides)
    return MistralConfig(**d)


def gemma_config_from_hf(hf_config, **overrides):
    from .gemma import GemmaConfig
    d = _common_fields(hf_config)
    d["head_dim"] = hf_config.head_dim
    d.update(overrides)
    return GemmaConfig(**d)


def qwen3_config_from_hf(hf_config, **overrides):
    from .qwen import Qwen3Config
    d = _common_fields(hf_config)
    d["head_dim"] = getattr(hf_config, "head_dim", None) or d["hidden_size"] // d["num_heads"]
    d["tie_embeddings"] = bool(getattr(hf_config, "tie_word_embeddings", False))
    d.update(overrides)
    return Qwen3Config(**d)


def convert_hf_llama_state_dict(hf_sd: Mapping[str, torch.Tensor], num_layers: int, tp_rank: int = 0,
                                tp_size: int = 1) -> Dict[str, torch.Tensor]:
    """Hugging Face ``LlamaForCausalLM`` state dict -> state dict of ``LlamaModel`` (this rank's shard)."""
    r, n = tp_rank, tp_size
    out: Dict[str, torch.Tensor] = {"embedding.weight": _rows(hf_sd["model.embed_tokens.weight"], r, n)}
    for i in range(num_layers):
        h, t = f"model.layers.{i}.", f"layers.{i}."
        q, k, v = (hf_sd[h + f"self_attn.{x}_proj.weight"] for x in "qkv")
        out[t + "self_attention.layernorm_qkv.layer_norm_weight"] = hf_sd[h + "input_layernorm.weight"]
        out[t + "self_attention.layernorm_qkv.weight"] = torch.cat([_rows(q, r, n), _rows(k, r, n), _rows(v, r, n)])
        out[t + "self_attention.proj.weight"] = _cols(hf_sd[h + "self_attn.o_proj.weight"], r, n)
        if h + "self_attn.q_norm.weight" in hf_sd:      # per-head norms (Qwen3): one vector for all heads
            out[t + "self_attention.q_norm.weight"] = hf_sd[h + "self_attn.q_norm.weight"]
            out[t + "self_attention.k_norm.weight"] = hf_sd[h + "self_attn.k_norm.weight"]
        out[t + "layernorm_mlp.layer_norm_weight"] = hf_sd[h + "post_attention_layernorm.weight"]
        out[t + "layernorm_mlp.fc1_weight"] = torch.cat([_rows(hf_sd[h + "mlp.gate_proj.weight"], r, n),
                                                         _rows(hf_sd[h + "mlp.up_proj.weight"], r, n)])
        out[t + "layernorm_mlp.fc2_weight"] = _cols(hf_sd[h + "mlp.down_proj.weight"], r, n)
    out["final_norm.weight"] = hf_sd["model.norm.weight"]
    head = hf_sd.get("lm_head.weight", hf_sd["model.embed_tokens.weight"])   # tied embeddings have no head entry
    out["lm_head.weight"] = _rows(head, r, n)
    return out


def export_hf_llama_state_dict(model) -> Dict[str, torch.Tensor]:
    """State dict of an unsharded ``LlamaModel`` in the Hugging Face ``LlamaForCausalLM`` naming."""
    assert model.tp_size == 1, "export an unsharded model (gather the shards first)"
    cfg, sd = model.cfg, model.state_dict()
    d = cfg.dim_per_head
    nq, nk, f = cfg.num_heads * d, cfg.num_kv_heads * d, cfg.ffn_hidden_size
    out = {"model.embed_tokens.weight": sd["embedding.weight"], "model.norm.weight": sd["final_norm.weight"],
           "lm_head.weight": sd["lm_head.weight"]}
    for i in range(cfg.num_layers):
        h, t = f"model.layers.{i}.", f"layers.{i}."
        q, k, v = torch.split(sd[t + "self_attention.layernorm_qkv.weight"], (nq, nk, nk))
        gate, up = torch.split(sd[t + "layernorm_mlp.fc1_weight"], (f, f))
        out.update({h + "self_attn.q_proj.weight": q, h + "self_attn.k_proj.weight": k, h + "self_attn.v_proj.weight": v,
                    h + "self_attn.o_proj.weight": sd[t + "self_attention.proj.weight"],
                    h + "input_layernorm.weight": sd[t + "self_attention.layernorm_qkv.layer_norm_weight"],
                    h + "post_attention_layernorm.weight": sd[t + "layernorm_mlp.layer_norm_weight"],
                    h + "mlp.gate_proj.weight": gate, h + "mlp.up_proj.weight": up,
                    h + "mlp.down_proj.weight": sd[t + "layernorm_mlp.fc2_weight"]})
        if cfg.qk_norm:
            out[h + "self_attn.q_norm.weight"] = sd[t + "self_attention.q_norm.weight"]
            out[h + "self_attn.k_norm.weight"] = sd[t + "self_attention.k_norm.weight"]
    return out


def _load(model: torch.nn.Module, converted: Dict[str, torch.Tensor]) -> None:
    """Copy converted tensors into the model's parameters (names must all exist; ``_extra_state`` entries of the
    model, which hold quantization state, are left alone)."""
    own = model.state_dict()
    missing = [k for k in own if not k.endswith("_extra_state") and k not in converted]
    unexpected = [k for k in converted if k not in own]
    if missing or unexpected:
        raise KeyError(f"checkpoint does not match the model: missing {missing[:4]}, unexpected {unexpected[:4]}")
    with torch.no_grad():
        for k, v in converted.items():
            if own[k].shape != v.shape:
                raise ValueError(f"{k}: checkpoint {tuple(v.shape)} vs model {tuple(own[k].shape)}")
            own[k].copy_(v)     # state_dict tensors alias the parameters


def load_hf_llama(model, hf_sd: Mapping[str, torch.Tensor]) -> None:
    """Fill a ``LlamaModel`` or one of its sibling families (Mistral, Gemma, Qwen3; sharded or not) from the
    Hugging Face state dict of the same architecture: the families share the checkpoint naming."""
    from ..parallel import distributed as D
    rank = D.get_rank(model.tp_group) if model.tp_size > 1 else 0
    _load(model, convert_hf_llama_state_dict(hf_sd, model.cfg.num_layers, rank, model.tp_size))


def _from_hf(model_cls, cfg, hf_model, tp_group, device):
    model = model_cls(cfg, tp_group=tp_group, device=device)
    load_hf_llama(model, hf_model.state_dict())
    return model


def llama_from_hf(hf_model, tp_group=None, device=None, **config_overrides):
    """A ``LlamaModel`` with the weights of a ``transformers.LlamaForCausalLM``."""
    from .llama import LlamaModel
    return _from_hf(LlamaModel, llama_config_from_hf(hf_model.config, **config_overrides), hf_model, tp_group, device)


def mistral_from_hf(hf_model, tp_group=None, device=None, **config_overrides):
    """A ``MistralModel`` with the weights of a ``transformers.MistralForCausalLM``."""
    from .mistral import MistralModel
    return _from_hf(MistralModel, mistral_config_from_hf(hf_model.config, **config_overrides), hf_model, tp_group, device)


def gemma_from_hf(hf_model, tp_group=None, device=None, **config_overrides):
    """A ``GemmaModel`` with the weights of a ``transformers.GemmaForCausalLM``."""
    from .gemma import GemmaModel
    return _from_hf(GemmaModel, gemma_config_from_hf(hf_model.config, **config_overrides), hf_model, tp_group, device)


def qwen3_from_hf(hf_model, tp_group=None, device=None, **config_overrides):
    """A ``Qwen3Model`` with the weights of a ``transformers.Qwen3ForCausalLM``."""
    from .qwen import Qwen3Model
    return _from_hf(Qwen3Model, qwen3_config_from_hf(hf_model.config, **config_overrides), hf_model, tp_group, device)


# ---------------------------------------------------------------------------------------------- Mixtral
def mixtral_config_from_hf(hf_config, **overrides):
    from .mixtral import MixtralConfig
    d = _common_fields(hf_config)
    d.update(num_experts=hf_config.num_local_experts, topk=hf_config.num_experts_per_tok,
             aux_loss_coeff=getattr(hf_config, "router_aux_loss_coef", 0.01))
    d.update(overrides)
    return MixtralConfig(**d)


def convert_hf_mixtral_state_dict(hf_sd: Mapping[str, torch.Tensor], num_layers: int, num_experts: int,
                                  ep_rank: int = 0, ep_size: int = 1) -> Dict[str, torch.Tensor]:
    """Hugging Face ``MixtralForCausalLM`` state dict -> state dict of ``MixtralModel``.  Both expert layouts are
    read: stacked ``mlp.experts.gate_up_proj [E, 2f, h]`` / ``down_proj [E, h, f]``, and the older one matrix per
    expert ``block_sparse_moe.experts.e.{w1 (gate), w3 (up), w2 (down)}``.  With expert parallelism a rank keeps
    experts ``[ep_rank * E/ep_size, (ep_rank + 1) * E/ep_size)``; everything else is replicated."""
    per = num_experts // ep_size
    out: Dict[str, torch.Tensor] = {"embedding.weight": hf_sd["model.embed_tokens.weight"],
                                    "final_norm.weight": hf_sd["model.norm.weight"],
                                    "lm_head.weight": hf_sd.get("lm_head.weight", hf_sd["model.embed_tokens.weight"])}
    for i in range(num_layers):
        h, t = f"model.layers.{i}.", f"layers.{i}."
        q, k, v = (hf_sd[h + f"self_attn.{x}_proj.weight"] for x in "qkv")
        out[t + "attn.layernorm_qkv.layer_norm_weight"] = hf_sd[h + "input_layernorm.weight"]
        out[t + "attn.layernorm_qkv.weight"] = torch.cat([q, k, v])
        out[t + "attn.proj.weight"] = hf_sd[h + "self_attn.o_proj.weight"]
        out[t + "pre_moe_norm.weight"] = hf_sd[h + "post_attention_layernorm.weight"]
        stacked = h + "mlp.experts.gate_up_proj" in hf_sd
        out[t + "moe.router.weight"] = hf_sd[h + ("mlp.gate.weight" if stacked else "block_sparse_moe.gate.weight")]
        for j in range(per):
            e = ep_rank * per + j
            if stacked:
                fc1, fc2 = hf_sd[h + "mlp.experts.gate_up_proj"][e], hf_sd[h + "mlp.experts.down_proj"][e]
            else:
                x = h + f"block_sparse_moe.experts.{e}."
                fc1, fc2 = torch.cat([hf_sd[x + "w1.weight"], hf_sd[x + "w3.weight"]]), hf_sd[x + "w2.weight"]
            out[t + f"moe.fc1.weight{j}"] = fc1
            out[t + f"moe.fc2.weight{j}"] = fc2
    return out


def load_hf_mixtral(model, hf_sd: Mapping[str, torch.Tensor]) -> None:
    from ..parallel import distributed as D
    moe = model.layers[0].moe
    rank = D.get_rank(moe.ep_group) if moe.ep_size > 1 else 0
    _load(model, convert_hf_mixtral_state_dict(hf_sd, model.cfg.num_layers, model.cfg.num_experts, rank, moe.ep_size))


def mixtral_from_hf(hf_model, ep_group=None, device=None, **config_overrides):
    """A ``MixtralModel`` with the weights of a ``transformers.MixtralForCausalLM``."""
    from .mixtral import MixtralModel
    model = MixtralModel(mixtral_config_from_hf(hf_model.config, **config_overrides), ep_group=ep_group, device=device)
    load_hf_mixtral(model, hf_model.state_dict())
    return model
