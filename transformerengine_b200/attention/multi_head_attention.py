"""``MultiheadAttention``: (norm +) QKV projection, RoPE, core attention, output projection.

Sub-module and parameter names follow the reference so that checkpoints load
unchanged: ``layernorm_qkv`` / ``qkv`` (self attention), ``layernorm_query`` /
``query_layer`` + ``key_value`` (cross attention), ``core_attention``, ``proj``,
``q_norm`` / ``k_norm`` (reference: ``pytorch/attention/multi_head_attention.py:47-958``).
"""
from __future__ import annotations

import collections
from typing import Callable, List, Optional, Tuple, Union

import torch

from ..modules.base import get_default_init_method
from ..modules.layernorm_linear import LayerNorm, LayerNormLinear, RMSNorm
from ..modules.linear import Linear
from ..parallel import distributed as D
from .dot_product_attention import DotProductAttention
from ..utils.config import get_config
from .rope import apply_rotary_pos_emb, rotate_packed_qkv_


class MultiheadAttention(torch.nn.Module):
    def __init__(self, hidden_size: int, num_attention_heads: int, kv_channels: Optional[int] = None,
                 attention_dropout: float = 0.1, layernorm_epsilon: float = 1e-5,
                 init_method: Optional[Callable] = None, output_layer_init_method: Optional[Callable] = None,
                 layer_number: Optional[int] = None, attn_mask_type: str = "causal",
                 window_size: Optional[Tuple[int, int]] = None, tp_group=None, tp_size: int = 1,
                 num_gqa_groups: Optional[int] = None, fuse_wgrad_accumulation: bool = False,
                 get_rng_state_tracker: Optional[Callable] = None, sequence_parallel: bool = False,
                 params_dtype: Optional[torch.dtype] = None, return_bias: bool = False,
                 return_layernorm_output: bool = False, input_layernorm: bool = False,
                 attention_type: str = "self", set_parallel_mode: bool = False, fuse_qkv_params: bool = False,
                 zero_centered_gamma: bool = False, qkv_weight_interleaved: bool = True,
                 ub_overlap_ag: bool = False, ub_overlap_rs: bool = False, ub_overlap_rs_dgrad: bool = False,
                 ub_bulk_dgrad: bool = False, ub_bulk_wgrad: bool = False, bias: bool = True,
                 normalization: str = "LayerNorm", device: Union[torch.device, str] = None,
                 qkv_format: str = "sbhd", name: Optional[str] = None, qk_norm_type: Optional[str] = None,
                 qk_norm_eps: float = 1e-6, qk_norm_before_rope: bool = False, seq_length: Optional[int] = None,
                 micro_batch_size: Optional[int] = None, softmax_type: str = "vanilla",
                 rotary_pos_interleaved: bool = False, bottom_right_diagonal: Optional[bool] = None) -> None:
        super().__init__()
        self.rotary_pos_interleaved = rotary_pos_interleaved
        self.bottom_right_diagonal = bottom_right_diagonal
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.qkv_format = qkv_format
        self.attn_mask_type, self.window_size = attn_mask_type, window_size
        self.layer_number = layer_number
        self.input_layernorm = input_layernorm
        self.attention_type = attention_type
        self.get_rng_state_tracker = get_rng_state_tracker
        self.tp_group = tp_group
        self.return_layernorm_output = return_layernorm_output
        self.params_dtype = torch.get_default_dtype() if params_dtype is None else params_dtype
        self.num_attention_heads = num_attention_heads
        self.return_bias = return_bias
        self.qk_norm_before_rope = qk_norm_before_rope
        self.name = name
        kv_channels = kv_channels if kv_channels else hidden_size // num_attention_heads
        init_method = init_method or get_default_init_method()
        output_layer_init_method = output_layer_init_method or get_default_init_method()
        if not fuse_qkv_params:
            qkv_weight_interleaved = False
        self.qkv_weight_interleaved = qkv_weight_interleaved
        self.tp_size = tp_size if tp_group is None else D.get_world_size(tp_group)
        self.sequence_parallel = (self.tp_size > 1) and sequence_parallel
        self.hidden_size_per_attention_head = kv_channels
        self.num_attention_heads_per_partition = num_attention_heads // self.tp_size
        self.num_gqa_groups = num_attention_heads if num_gqa_groups is None else num_gqa_groups
        assert num_attention_heads % self.num_gqa_groups == 0
        assert self.num_gqa_groups % self.tp_size == 0, "GQA groups must divide by the TP size"
        self.num_gqa_groups_per_partition = self.num_gqa_groups // self.tp_size
        self.hidden_size_q = kv_channels * num_attention_heads
        self.hidden_size_kv = kv_channels * self.num_gqa_groups
        common = dict(fuse_wgrad_accumulation=fuse_wgrad_accumulation, tp_group=tp_group, tp_size=self.tp_size,
                      get_rng_state_tracker=get_rng_state_tracker, sequence_parallel=sequence_parallel,
                      params_dtype=self.params_dtype, device=device)
        mode = "column" if set_parallel_mode else None
        self.q_norm, self.k_norm = None, None
        if qk_norm_type is not None:
            cls = {"L2Normalization": None, "RMSNorm": RMSNorm, "LayerNorm": LayerNorm}[qk_norm_type]
            if cls is not None:
                self.q_norm = cls(kv_channels, eps=qk_norm_eps, params_dtype=self.params_dtype, device=device)
                self.k_norm = cls(kv_channels, eps=qk_norm_eps, params_dtype=self.params_dtype, device=device)
            else:
                self._l2_eps = qk_norm_eps
        self.qk_norm_type = qk_norm_type
        if attention_type == "self":
            split = collections.OrderedDict([("query", self.hidden_size_q), ("key", self.hidden_size_kv),
                                             ("value", self.hidden_size_kv)]) if not fuse_qkv_params else None
            out = self.hidden_size_q + 2 * self.hidden_size_kv
            if input_layernorm:
                self.layernorm_qkv = LayerNormLinear(
                    hidden_size, out, eps=layernorm_epsilon, init_method=init_method, bias=bias,
                    return_bias=False, parallel_mode=mode, return_layernorm_output=return_layernorm_output,
                    parameters_split=split, zero_centered_gamma=zero_centered_gamma, normalization=normalization,
                    name=f"{name}.layernorm_linear_qkv" if name else None, **common)
            else:
                self.qkv = Linear(hidden_size, out, init_method=init_method, bias=bias, return_bias=False,
                                  parallel_mode=mode, parameters_split=split,
                                  name=f"{name}.linear_qkv" if name else None, **common)
        else:
            if input_layernorm:
                self.layernorm_query = LayerNormLinear(
                    hidden_size, self.hidden_size_q, eps=layernorm_epsilon, init_method=init_method, bias=bias,
                    return_bias=False, parallel_mode=mode, return_layernorm_output=return_layernorm_output,
                    parameters_split=("query",) if not fuse_qkv_params else None,
                    zero_centered_gamma=zero_centered_gamma, normalization=normalization, **common)
            else:
                self.query_layer = Linear(hidden_size, self.hidden_size_q, init_method=init_method, bias=bias,
                                          return_bias=False, parallel_mode=mode, **common)
            self.key_value = Linear(hidden_size, 2 * self.hidden_size_kv, init_method=init_method, bias=bias,
                                    return_bias=False, parallel_mode=mode,
                                    parameters_split=("key", "value") if not fuse_qkv_params else None, **common)
        self.core_attention = DotProductAttention(
            num_attention_heads, kv_channels, num_gqa_groups=self.num_gqa_groups,
            attention_dropout=attention_dropout, qkv_format=qkv_format, tp_size=self.tp_size,
            get_rng_state_tracker=get_rng_state_tracker, sequence_parallel=sequence_parallel, tp_group=tp_group,
            layer_number=layer_number, attention_type=attention_type, attn_mask_type=attn_mask_type,
            window_size=window_size, softmax_type=softmax_type)
        self.proj = Linear(self.hidden_size_q, hidden_size, init_method=output_layer_init_method, bias=bias,
                           return_bias=return_bias, parallel_mode="row" if set_parallel_mode else None,
                           name=f"{name}.proj" if name else None, **common)

    def set_tensor_parallel_group(self, tp_group) -> None:
        self.tp_group = tp_group
        for m in self.children():
            if hasattr(m, "set_tensor_parallel_group"):
                m.set_tensor_parallel_group(tp_group)

    def set_context_parallel_group(self, cp_group, cp_global_ranks, cp_stream, cp_comm_type="p2p") -> None:
        self.core_attention.set_context_parallel_group(cp_group, cp_global_ranks, cp_stream, cp_comm_type)

    def _qk_norm(self, t, norm):
        if self.qk_norm_type is None:
            return t
        if norm is None:  # L2 normalisation
            return (t.float() * torch.rsqrt(t.float().pow(2).sum(-1, keepdim=True) + self._l2_eps)).to(t.dtype)
        return norm(t)

    def forward(self, hidden_states: torch.Tensor, attention_mask=None, encoder_output: Optional[torch.Tensor] = None,
                attn_mask_type: Optional[str] = None, window_size: Optional[Tuple[int, int]] = None,
                is_first_microbatch: Optional[bool] = None, checkpoint_core_attention: bool = False,
                inference_params=None, rotary_pos_emb=None, core_attention_bias_type: str = "no_bias",
                core_attention_bias: Optional[torch.Tensor] = None, alibi_slopes: Optional[torch.Tensor] = None,
                cu_seqlens_q=None, cu_seqlens_kv=None, cu_seqlens_q_padded=None, cu_seqlens_kv_padded=None,
                max_seqlen_q=None, max_seqlen_kv=None, fast_zero_fill: bool = True, pad_between_seqs=None,
                bottom_right_diagonal: Optional[bool] = None):
        d = self.hidden_size_per_attention_head
        hq, hk = self.num_attention_heads_per_partition, self.num_gqa_groups_per_partition
        ln_out = None
        if self.attention_type == "self":
            if self.input_layernorm:
                res = self.layernorm_qkv(hidden_states, is_first_microbatch=is_first_microbatch)
                mixed, ln_out = res if self.return_layernorm_output else (res, None)
            else:
                mixed = self.qkv(hidden_states, is_first_microbatch=is_first_microbatch)
            lead = mixed.shape[:-1]
            rope_done = False
            if (rotary_pos_emb is not None and inference_params is None and self.qkv_format in ("sbhd", "bshd")
                    and not (self.qk_norm_type is not None and self.qk_norm_before_rope)
                    and mixed.dim() == 3 and mixed.is_contiguous() and get_config().fused_qkv_rope):
                # split + both rotations in one launch, in place on the projection output
                q_emb, k_emb = rotary_pos_emb if isinstance(rotary_pos_emb, (tuple, list)) else (rotary_pos_emb,) * 2
                cpg = self.core_attention.cp_group
                cp_size = D.get_world_size(cpg) if cpg is not None else 1
                mixed = rotate_packed_qkv_(mixed, q_emb, k_emb, self.qkv_format,
                                           "grouped" if self.qkv_weight_interleaved else "blocked", hq, hk, d,
                                           interleaved=self.rotary_pos_interleaved,
                                           cp_size=cp_size, cp_rank=D.get_rank(cpg) if cp_size > 1 else 0)
                rope_done = True
            if self.qkv_weight_interleaved:
                g = hq // hk
                mixed = mixed.reshape(*lead, hk, g + 2, d)
                q, k, v = torch.split(mixed, (g, 1, 1), dim=-2)
                q = q.reshape(*lead, hq, d)
                k, v = k.reshape(*lead, hk, d), v.reshape(*lead, hk, d)
            else:
                q, k, v = torch.split(mixed, (hq * d, hk * d, hk * d), dim=-1)
                q = q.reshape(*lead, hq, d)
                k, v = k.reshape(*lead, hk, d), v.reshape(*lead, hk, d)
        else:
            kv = self.key_value(encoder_output, is_first_microbatch=is_first_microbatch)
            kl = kv.shape[:-1]
            if self.qkv_weight_interleaved:
                kv = kv.reshape(*kl, hk, 2 * d)
                k, v = torch.split(kv, d, dim=-1)
            else:
                k, v = torch.split(kv, hk * d, dim=-1)
            k, v = k.reshape(*kl, hk, d), v.reshape(*kl, hk, d)
            if self.input_layernorm:
                res = self.layernorm_query(hidden_states, is_first_microbatch=is_first_microbatch)
                ql, ln_out = res if self.return_layernorm_output else (res, None)
            else:
                ql = self.query_layer(hidden_states, is_first_microbatch=is_first_microbatch)
            q = ql.reshape(*ql.shape[:-1], hq, d)
        if self.qk_norm_type is not None and self.qk_norm_before_rope:
            q, k = self._qk_norm(q, self.q_norm), self._qk_norm(k, self.k_norm)
        if rotary_pos_emb is not None and not (self.attention_type == "self" and rope_done):
            q_emb, k_emb = rotary_pos_emb if isinstance(rotary_pos_emb, (tuple, list)) else (rotary_pos_emb,) * 2
            fmt = self.qkv_format
            if fmt in ("sbhd", "bshd") and inference_params is None:
                sdim = 0 if fmt == "sbhd" else 1
                cp_size = D.get_world_size(self.core_attention.cp_group) if self.core_attention.cp_group is not None else 1
                cp_rank = D.get_rank(self.core_attention.cp_group) if cp_size > 1 else 0
                il = self.rotary_pos_interleaved
                q = apply_rotary_pos_emb(q, q_emb, fmt, cp_size=cp_size, cp_rank=cp_rank, interleaved=il)
                k = apply_rotary_pos_emb(k, k_emb, fmt, cp_size=cp_size, cp_rank=cp_rank, interleaved=il)
            elif inference_params is not None:
                start = inference_params.sequence_start_positions(q.shape[1 if fmt == "sbhd" else 0], q.device)
                q = apply_rotary_pos_emb(q, q_emb, fmt, start_positions=start, interleaved=self.rotary_pos_interleaved)
                k = apply_rotary_pos_emb(k, k_emb, fmt, start_positions=start, interleaved=self.rotary_pos_interleaved)
            else:
                q = apply_rotary_pos_emb(q, q_emb, "thd", cu_seqlens=cu_seqlens_q, interleaved=self.rotary_pos_interleaved)
                k = apply_rotary_pos_emb(k, k_emb, "thd", cu_seqlens=cu_seqlens_kv if cu_seqlens_kv is not None else cu_seqlens_q,
                                         interleaved=self.rotary_pos_interleaved)
        if self.qk_norm_type is not None and not self.qk_norm_before_rope:
            q, k = self._qk_norm(q, self.q_norm), self._qk_norm(k, self.k_norm)
        ctx = self.core_attention(q, k, v, attention_mask=attention_mask, qkv_format=self.qkv_format,
                                  cu_seqlens_q=cu_seqlens_q, cu_seqlens_kv=cu_seqlens_kv,
                                  cu_seqlens_q_padded=cu_seqlens_q_padded, cu_seqlens_kv_padded=cu_seqlens_kv_padded,
                                  pad_between_seqs=pad_between_seqs, fast_zero_fill=fast_zero_fill,
                                  max_seqlen_q=max_seqlen_q, max_seqlen_kv=max_seqlen_kv,
                                  attn_mask_type=attn_mask_type, window_size=window_size,
                                  checkpoint_core_attention=checkpoint_core_attention,
                                  core_attention_bias_type=core_attention_bias_type,
                                  core_attention_bias=core_attention_bias, alibi_slopes=alibi_slopes,
                                  inference_params=inference_params,
                                  bottom_right_diagonal=(self.bottom_right_diagonal if bottom_right_diagonal is None
                                                         else bottom_right_diagonal))
        proj = self.proj(ctx, is_first_microbatch=is_first_microbatch)
        if self.return_bias:
            out, b = proj
        else:
            out, b = proj, None
        outs = [out]
        if self.return_bias:
            outs.append(b)
        if self.input_layernorm and self.return_layernorm_output:
            outs.append(ln_out)
        return outs[0] if len(outs) == 1 else tuple(outs)
