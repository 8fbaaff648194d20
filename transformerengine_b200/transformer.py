"""``TransformerLayer``: attention block + MLP block with residuals, pre- or post-norm,
encoder / decoder variants, parallel attention+MLP, drop path
(reference: ``pytorch/transformer.py:69-986``)."""
from __future__ import annotations

from typing import Callable, Optional, Tuple, Union

import torch

from .attention.multi_head_attention import MultiheadAttention
from .modules.layernorm_linear import LayerNorm, RMSNorm
from .modules.layernorm_mlp import LayerNormMLP
from .parallel import distributed as D


class DropPath(torch.nn.Module):
    """Stochastic depth: drop whole samples of the residual branch."""

    def __init__(self, drop_prob: float = 0.0) -> None:
        super().__init__()
        self.drop_prob = drop_prob

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.drop_prob == 0.0 or not self.training:
            return x
        keep = 1 - self.drop_prob
        shape = (x.shape[0],) + (1,) * (x.ndim - 1)
        mask = torch.empty(shape, dtype=x.dtype, device=x.device).bernoulli_(keep)
        return x.div(keep) * mask


def _bias_dropout_add(x, bias, residual, prob, training):
    if bias is not None:
        x = x + bias
    if prob > 0.0 and training:
        x = torch.nn.functional.dropout(x, p=prob, training=True)
    return residual + x


class TransformerLayer(torch.nn.Module):
    def __init__(self, hidden_size: int, ffn_hidden_size: int, num_attention_heads: int,
                 num_gqa_groups: Optional[int] = None, layernorm_epsilon: float = 1e-5, hidden_dropout: float = 0.1,
                 attention_dropout: float = 0.1, init_method: Optional[Callable] = None,
                 output_layer_init_method: Optional[Callable] = None, layer_number: Optional[int] = None,
                 kv_channels: Optional[int] = None, self_attn_mask_type: str = "causal",
                 window_size: Optional[Tuple[int, int]] = None, enc_dec_attn_mask_type: str = "no_mask",
                 enc_dec_window_size: Optional[Tuple[int, int]] = None, tp_group=None, tp_size: int = 1,
                 params_dtype: Optional[torch.dtype] = None, get_rng_state_tracker: Optional[Callable] = None,
                 fuse_wgrad_accumulation: bool = False, seq_length: Optional[int] = None,
                 micro_batch_size: Optional[int] = None, sequence_parallel: bool = False,
                 apply_residual_connection_post_layernorm: bool = False, output_layernorm: bool = False,
                 parallel_attention_mlp: bool = False, layer_type: str = "encoder", drop_path_rate: float = 0.0,
                 set_parallel_mode: bool = False, fuse_qkv_params: bool = False, rotary_pos_interleaved: bool = False,
                 zero_centered_gamma: bool = False, qkv_weight_interleaved: bool = True, ub_tp_comm_overlap: bool = False,
                 ub_overlap_ag: bool = True, ub_overlap_rs: bool = True, ub_overlap_rs_dgrad: bool = False,
                 ub_bulk_dgrad: bool = True, ub_bulk_wgrad: bool = True, bias: bool = True,
                 activation: str = "gelu", activation_params: Optional[dict] = None, normalization: str = "LayerNorm",
                 device: Union[torch.device, str] = None, attn_input_format: str = "sbhd", name: Optional[str] = None,
                 qk_norm_type: Optional[str] = None, qk_norm_eps: float = 1e-6, qk_norm_before_rope: bool = False,
                 softmax_type: str = "vanilla", bottom_right_diagonal: Optional[bool] = None,
                 enc_dec_bottom_right_diagonal: Optional[bool] = None) -> None:
        super().__init__()
        self.bottom_right_diagonal = bottom_right_diagonal
        self.enc_dec_bottom_right_diagonal = enc_dec_bottom_right_diagonal
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        params_dtype = torch.get_default_dtype() if params_dtype is None else params_dtype
        self.self_attn_mask_type, self.window_size = self_attn_mask_type, window_size
        self.enc_dec_attn_mask_type, self.enc_dec_window_size = enc_dec_attn_mask_type, enc_dec_window_size
        self.tp_size = tp_size if tp_group is None else D.get_world_size(tp_group)
        self.sequence_parallel = (self.tp_size > 1) and sequence_parallel
        self.layer_number = layer_number
        self.output_layernorm = output_layernorm
        self.layer_type = layer_type
        self.apply_residual_connection_post_layernorm = apply_residual_connection_post_layernorm
        self.parallel_attention_mlp = parallel_attention_mlp
        self.hidden_dropout = hidden_dropout
        self.get_rng_state_tracker = get_rng_state_tracker
        self.attn_input_format = attn_input_format
        self.name = name
        assert layer_type in ("encoder", "decoder")
        if parallel_attention_mlp:
            assert layer_type == "encoder" and not apply_residual_connection_post_layernorm and not output_layernorm
        attn_kwargs = dict(kv_channels=kv_channels, attention_dropout=attention_dropout,
                           layernorm_epsilon=layernorm_epsilon, init_method=init_method,
                           output_layer_init_method=output_layer_init_method, layer_number=layer_number,
                           tp_group=tp_group, tp_size=self.tp_size, num_gqa_groups=num_gqa_groups,
                           fuse_wgrad_accumulation=fuse_wgrad_accumulation,
                           get_rng_state_tracker=get_rng_state_tracker, sequence_parallel=sequence_parallel,
                           params_dtype=params_dtype, return_layernorm_output=apply_residual_connection_post_layernorm,
                           set_parallel_mode=set_parallel_mode, fuse_qkv_params=fuse_qkv_params,
                           zero_centered_gamma=zero_centered_gamma, qkv_weight_interleaved=qkv_weight_interleaved,
                           bias=bias, normalization=normalization, device=device, qkv_format=attn_input_format,
                           qk_norm_type=qk_norm_type, qk_norm_eps=qk_norm_eps,
                           qk_norm_before_rope=qk_norm_before_rope, softmax_type=softmax_type,
                           rotary_pos_interleaved=rotary_pos_interleaved)
        self.self_attention = MultiheadAttention(hidden_size, num_attention_heads, **attn_kwargs,
                                                 input_layernorm=not output_layernorm, attention_type="self",
                                                 attn_mask_type=self_attn_mask_type, window_size=window_size,
                                                 return_bias=not parallel_attention_mlp,
                                                 name=f"{name}.self_attention" if name else None)
        if layer_type == "decoder":
            self.inter_attention = MultiheadAttention(hidden_size, num_attention_heads, **attn_kwargs,
                                                      input_layernorm=True, attention_type="cross",
                                                      attn_mask_type=enc_dec_attn_mask_type,
                                                      window_size=enc_dec_window_size, return_bias=True,
                                                      name=f"{name}.inter_attention" if name else None)
        self.layernorm_mlp = LayerNormMLP(
            hidden_size, ffn_hidden_size, eps=layernorm_epsilon, fuse_wgrad_accumulation=fuse_wgrad_accumulation,
            tp_group=tp_group, tp_size=self.tp_size, get_rng_state_tracker=get_rng_state_tracker,
            init_method=init_method, output_layer_init_method=output_layer_init_method, bias=bias,
            return_bias=not parallel_attention_mlp, sequence_parallel=sequence_parallel, params_dtype=params_dtype,
            return_layernorm_output=apply_residual_connection_post_layernorm, set_parallel_mode=set_parallel_mode,
            zero_centered_gamma=zero_centered_gamma, activation=activation, activation_params=activation_params,
            normalization=normalization, device=device, name=f"{name}.layernorm_mlp" if name else None)
        self.drop_path = DropPath(drop_path_rate) if drop_path_rate > 0.0 else None
        if output_layernorm:
            cls = LayerNorm if normalization == "LayerNorm" else RMSNorm
            self.layernorm = cls(hidden_size, eps=layernorm_epsilon, sequence_parallel=self.sequence_parallel,
                                 params_dtype=params_dtype, zero_centered_gamma=zero_centered_gamma, device=device)

    def set_tensor_parallel_group(self, tp_group) -> None:
        for m in self.children():
            if hasattr(m, "set_tensor_parallel_group"):
                m.set_tensor_parallel_group(tp_group)

    def set_context_parallel_group(self, cp_group, cp_global_ranks, cp_stream, cp_comm_type="p2p") -> None:
        for m in self.children():
            if hasattr(m, "set_context_parallel_group"):
                m.set_context_parallel_group(cp_group, cp_global_ranks, cp_stream, cp_comm_type)

    def _bda(self, x, bias, residual):
        if self.drop_path is not None:
            out = torch.nn.functional.dropout((x + bias) if bias is not None else x, p=self.hidden_dropout,
                                              training=self.training)
            return residual + self.drop_path(out)
        if self.get_rng_state_tracker is not None and self.hidden_dropout > 0 and self.training and not self.sequence_parallel:
            return _bias_dropout_add(x, bias, residual, self.hidden_dropout, self.training)
        return _bias_dropout_add(x, bias, residual, self.hidden_dropout, self.training)

    def forward(self, hidden_states: torch.Tensor, attention_mask=None, self_attn_mask_type: Optional[str] = None,
                window_size: Optional[Tuple[int, int]] = None, encoder_output: Optional[torch.Tensor] = None,
                enc_dec_attn_mask=None, enc_dec_attn_mask_type: Optional[str] = None,
                enc_dec_window_size: Optional[Tuple[int, int]] = None, is_first_microbatch: Optional[bool] = None,
                checkpoint_core_attention: bool = False, inference_params=None, rotary_pos_emb=None,
                core_attention_bias_type: str = "no_bias", core_attention_bias: Optional[torch.Tensor] = None,
                alibi_slopes: Optional[torch.Tensor] = None, cu_seqlens_q=None, cu_seqlens_kv=None,
                cu_seqlens_q_padded=None, cu_seqlens_kv_padded=None, max_seqlen_q=None, max_seqlen_kv=None,
                fast_zero_fill: bool = True, pad_between_seqs=None, bottom_right_diagonal: Optional[bool] = None,
                enc_dec_bottom_right_diagonal: Optional[bool] = None):
        mask_type = self_attn_mask_type or self.self_attn_mask_type
        brd = self.bottom_right_diagonal if bottom_right_diagonal is None else bottom_right_diagonal
        enc_dec_brd = (self.enc_dec_bottom_right_diagonal if enc_dec_bottom_right_diagonal is None
                       else enc_dec_bottom_right_diagonal)
        window = window_size if window_size is not None else self.window_size
        attn_out = self.self_attention(
            hidden_states, attention_mask=attention_mask, attn_mask_type=mask_type, window_size=window,
            inference_params=inference_params, is_first_microbatch=is_first_microbatch,
            checkpoint_core_attention=checkpoint_core_attention, rotary_pos_emb=rotary_pos_emb,
            core_attention_bias_type=core_attention_bias_type, core_attention_bias=core_attention_bias,
            alibi_slopes=alibi_slopes, cu_seqlens_q=cu_seqlens_q, cu_seqlens_kv=cu_seqlens_kv,
            cu_seqlens_q_padded=cu_seqlens_q_padded, cu_seqlens_kv_padded=cu_seqlens_kv_padded,
            max_seqlen_q=max_seqlen_q, max_seqlen_kv=max_seqlen_kv, fast_zero_fill=fast_zero_fill,
            pad_between_seqs=pad_between_seqs, bottom_right_diagonal=brd)
        if self.parallel_attention_mlp:
            mlp_out = self.layernorm_mlp(hidden_states, is_first_microbatch=is_first_microbatch)
            out = hidden_states + torch.nn.functional.dropout(attn_out + mlp_out, p=self.hidden_dropout,
                                                              training=self.training)
            return out
        if self.apply_residual_connection_post_layernorm and not self.output_layernorm:
            attn_o, attn_b, residual = attn_out
        else:
            attn_o, attn_b = attn_out
            residual = hidden_states
        hidden = self._bda(attn_o, attn_b, residual)
        if self.layer_type == "decoder":
            inter = self.inter_attention(hidden, attention_mask=enc_dec_attn_mask,
                                         attn_mask_type=enc_dec_attn_mask_type or self.enc_dec_attn_mask_type,
                                         window_size=enc_dec_window_size if enc_dec_window_size is not None else self.enc_dec_window_size,
                                         encoder_output=encoder_output, is_first_microbatch=is_first_microbatch,
                                         checkpoint_core_attention=checkpoint_core_attention,
                                         bottom_right_diagonal=enc_dec_brd)
            if self.apply_residual_connection_post_layernorm:
                io, ib, residual = inter
            else:
                io, ib = inter
                residual = hidden
            hidden = self._bda(io, ib, residual)
        mlp = self.layernorm_mlp(hidden, is_first_microbatch=is_first_microbatch)
        if self.apply_residual_connection_post_layernorm:
            mo, mb, residual = mlp
        else:
            mo, mb = mlp
            residual = hidden
        out = self._bda(mo, mb, residual)
        if self.output_layernorm:
            out = self.layernorm(out)
        return out
