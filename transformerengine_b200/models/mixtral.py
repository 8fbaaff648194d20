"""Mixtral-architecture MoE decoder: GQA attention + top-k routed SwiGLU experts with the
load-balancing auxiliary loss, optional expert parallelism (experts sharded over ``ep_group``,
tokens exchanged by all-to-all).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..attention.multi_head_attention import MultiheadAttention
from ..attention.rope import RotaryPositionEmbedding
from ..modules.grouped_linear import GroupedLinear
from ..modules.layernorm_linear import RMSNorm
from ..modules.linear import Linear
from ..moe import (fused_moe_aux_loss, fused_topk_with_score_function, moe_permute_and_pad_with_probs,
                   moe_unpermute)
from ..parallel import distributed as D
from ..utils.config import get_config
from ..parallel.expert_parallel import (ep_combine, ep_dispatch, fused_ep_combine, fused_ep_dispatch,
                                        get_fused_ep)
from .llama import _FusedCrossEntropy


@dataclass
class MixtralConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    ffn_hidden_size: int = 14336
    num_experts: int = 8
    topk: int = 2
    aux_loss_coeff: float = 0.01
    rms_eps: float = 1e-5
    rope_theta: float = 1e6
    init_std: float = 0.02
    params_dtype: torch.dtype = torch.bfloat16
    pad_align: int = 128  # expert slabs are padded to whole 128-row scale tiles

    @staticmethod
    def mixtral_8x7b(**kw) -> "MixtralConfig":
        return MixtralConfig(**kw)

    @staticmethod
    def tiny(**kw) -> "MixtralConfig":
        d = dict(vocab_size=512, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, ffn_hidden_size=256,
                 num_experts=4, topk=2, pad_align=32)
        d.update(kw)
        return MixtralConfig(**d)


class _ActScaled(torch.autograd.Function):
    """SwiGLU with each output row scaled by its routing probability (fused kernel on CUDA)."""

    @staticmethod
    def forward(ctx, x, probs, act):  # type: ignore[override]
        y, _ = ops.activation_fwd(x, act, row_scale=probs)
        ctx.save_for_backward(x, probs)
        ctx.act = act
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x, probs = ctx.saved_tensors
        dy = dy.contiguous()
        dx, _, _ = ops.activation_bwd(dy, x, ctx.act, row_scale=probs)
        # d(probs)[r] = <dy[r], act(x)[r]>: the unscaled activation from the fused kernel, then a
        # 16-bit product and an fp32 row sum (a batched dot through the library ran as a 3.5 ms gemv,
        # the fp32 reference activation as several strided element-wise passes)
        unscaled, _ = ops.activation_fwd(x, ctx.act)
        dprobs = ops.row_dot(dy.reshape(-1, dy.shape[-1]), unscaled.to(dy.dtype).reshape(-1, dy.shape[-1])).to(probs.dtype).reshape(probs.shape)
        return dx, dprobs, None


class MoELayer(torch.nn.Module):
    """Router -> dispatch (permute, pad, all-to-all) -> expert MLPs -> combine."""

    def __init__(self, cfg: MixtralConfig, ep_group=None, device=None):
        super().__init__()
        self.cfg = cfg
        self.ep_group = ep_group
        self.ep_size = D.get_world_size(ep_group) if ep_group is not None else 1
        assert cfg.num_experts % self.ep_size == 0
        self.local_experts = cfg.num_experts // self.ep_size
        init = lambda t: torch.nn.init.normal_(t, 0.0, cfg.init_std)  # noqa: E731
        self.router = torch.nn.Linear(cfg.hidden_size, cfg.num_experts, bias=False, dtype=torch.float32, device=device)
        init(self.router.weight)
        self.fc1 = GroupedLinear(self.local_experts, cfg.hidden_size, 2 * cfg.ffn_hidden_size, bias=False,
                                 init_method=init, params_dtype=cfg.params_dtype, device=device)
        self.fc2 = GroupedLinear(self.local_experts, cfg.ffn_hidden_size, cfg.hidden_size, bias=False,
                                 init_method=init, params_dtype=cfg.params_dtype, device=device)

    def forward(self, x: torch.Tensor):
        """x [tokens, hidden] -> (y [tokens, hidden], aux loss)."""
        cfg = self.cfg
        T = x.shape[0]
        logits = self.router(x.float())
        probs, rmap = fused_topk_with_score_function(logits, cfg.topk, False, None, None, None, "softmax", None)
        scores = torch.softmax(logits, dim=-1)
        tokens_per_expert = rmap.sum(0)
        if self.ep_size > 1:
            tpe = tokens_per_expert.clone()
            dist.all_reduce(tpe, group=self.ep_group)
            total = T * self.ep_size
        else:
            tpe, total = tokens_per_expert, T
        aux = fused_moe_aux_loss(scores, tpe, total, cfg.num_experts, topk=cfg.topk, coeff=cfg.aux_loss_coeff)
        fused = self.ep_size > 1 and x.is_cuda and get_config().fused_ep \
            and x.dtype in (torch.bfloat16, torch.float16)
        if fused:
            ep = get_fused_ep(self.ep_group, self.local_experts, cfg.hidden_size, T, x.dtype, cfg.pad_align, cfg.topk)
            xs, ps, m_splits, state = fused_ep_dispatch(x, probs, rmap, ep)
        elif self.ep_size > 1:
            xs, ps, m_splits, state = ep_dispatch(x, probs, rmap, self.ep_group, self.local_experts, cfg.pad_align)
        else:
            xs, ps, row_id_map, _, padded = moe_permute_and_pad_with_probs(x, probs, rmap, tokens_per_expert,
                                                                           cfg.pad_align)
            m_splits = [int(v) for v in padded.tolist()]
        h = self.fc1(xs, m_splits)
        a = _ActScaled.apply(h, ps.float(), "swiglu")
        o = self.fc2(a, m_splits)
        if fused:
            y = fused_ep_combine(o, state)
        elif self.ep_size > 1:
            y = ep_combine(o, state)
        else:
            y = moe_unpermute(o, row_id_map)
        return y.to(x.dtype), aux


class MixtralBlock(torch.nn.Module):
    def __init__(self, cfg: MixtralConfig, layer_number: int, ep_group=None, device=None):
        super().__init__()
        init = lambda t: torch.nn.init.normal_(t, 0.0, cfg.init_std)  # noqa: E731
        self.attn = MultiheadAttention(cfg.hidden_size, cfg.num_heads, attention_dropout=0.0,
                                       layernorm_epsilon=cfg.rms_eps, init_method=init, output_layer_init_method=init,
                                       layer_number=layer_number, attn_mask_type="causal",
                                       num_gqa_groups=cfg.num_kv_heads, params_dtype=cfg.params_dtype,
                                       input_layernorm=True, fuse_qkv_params=True, qkv_weight_interleaved=False,
                                       bias=False, normalization="RMSNorm", device=device, qkv_format="sbhd")
        self.pre_moe_norm = RMSNorm(cfg.hidden_size, eps=cfg.rms_eps, params_dtype=cfg.params_dtype, device=device)
        self.moe = MoELayer(cfg, ep_group, device)

    def forward(self, x, freqs, inference_params=None):
        x = x + self.attn(x, rotary_pos_emb=freqs, inference_params=inference_params)
        s, b, h = x.shape
        y, aux = self.moe(self.pre_moe_norm(x).reshape(s * b, h))
        return x + y.reshape(s, b, h), aux


class MixtralModel(torch.nn.Module):
    def __init__(self, cfg: MixtralConfig, ep_group=None, device=None):
        super().__init__()
        self.cfg = cfg
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        init = lambda t: torch.nn.init.normal_(t, 0.0, cfg.init_std)  # noqa: E731
        self.embedding = torch.nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=cfg.params_dtype, device=device)
        init(self.embedding.weight)
        self.layers = torch.nn.ModuleList([MixtralBlock(cfg, i + 1, ep_group, device) for i in range(cfg.num_layers)])
        self.final_norm = RMSNorm(cfg.hidden_size, eps=cfg.rms_eps, params_dtype=cfg.params_dtype, device=device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, bias=False, init_method=init,
                              params_dtype=cfg.params_dtype, device=device)
        self.rope = RotaryPositionEmbedding(cfg.hidden_size // cfg.num_heads, rotary_base=cfg.rope_theta)

    logits_seq_first = True  # forward returns [s, b, vocab]

    def make_inference_params(self, max_batch_size: int, max_sequence_length: int, **kw):
        """Key/value cache for incremental decoding with this model."""
        from ..attention.inference import InferenceParams
        cfg = self.cfg
        kw.setdefault("device", self.embedding.weight.device)
        return InferenceParams(max_batch_size, max_sequence_length, num_heads_kv=cfg.num_kv_heads,
                               head_dim_k=cfg.hidden_size // cfg.num_heads, dtype=cfg.params_dtype,
                               qkv_format="sbhd", **kw)

    def generate(self, prompt: torch.Tensor, max_new_tokens: int, **kw) -> torch.Tensor:
        """Decoding on the key/value cache; see ``models.generation.generate`` for the options."""
        from .generation import generate
        return generate(self, prompt, max_new_tokens, **kw)

    def forward(self, tokens: torch.Tensor, labels: Optional[torch.Tensor] = None, inference_params=None):
        ids = tokens.t().contiguous()
        x = self.embedding(ids)
        n_pos = tokens.shape[1] if inference_params is None else inference_params.max_sequence_length
        freqs = self.rope(n_pos).to(x.device)
        aux_total = 0.0
        for layer in self.layers:
            x, aux = layer(x, freqs, inference_params)
            aux_total = aux_total + aux
        logits = self.lm_head(self.final_norm(x))
        if labels is None:
            return logits
        tgt = torch.full_like(ids, -100)
        tgt[:-1] = labels.t()[1:]
        return _FusedCrossEntropy.apply(logits, tgt, None, 0) + aux_total
