"""``DotProductAttention``: softmax(Q K^T / sqrt(d) + mask) V with GQA, the mask
types, sliding windows, bias, softmax variants, packed (thd) sequences, KV cache
and context parallelism (reference: ``pytorch/attention/dot_product_attention/
dot_product_attention.py:415-1380``, backend selection ``utils.py:393``).
"""
from __future__ import annotations

import math
import os
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import torch

import sys

from .. import ops
from ..ops import flash
from ..parallel import distributed as D
from ..utils.config import get_config

_MASK_TYPES = ("no_mask", "padding", "causal", "padding_causal", "causal_bottom_right",
               "padding_causal_bottom_right", "arbitrary")


def _padding_mask_from_cu(cu_q, cu_kv, sq, sk, device):
    """[b,1,sq,sk] bool, True = masked, from cumulative sequence lengths."""
    lq = (cu_q[1:] - cu_q[:-1]).to(device)
    lk = (cu_kv[1:] - cu_kv[:-1]).to(device)
    qi = torch.arange(sq, device=device)[None, :, None]
    ki = torch.arange(sk, device=device)[None, None, :]
    m = (qi >= lq[:, None, None]) | (ki >= lk[:, None, None])
    return m[:, None]


class DotProductAttention(torch.nn.Module):
    def __init__(self, num_attention_heads: int, kv_channels: Union[int, Tuple[int, int]],
                 num_gqa_groups: Optional[int] = None, attention_dropout: float = 0.0, qkv_format: str = "sbhd",
                 attn_mask_type: str = "causal", window_size: Optional[Tuple[int, int]] = None,
                 sequence_parallel: bool = False, tp_size: int = 1, get_rng_state_tracker: Optional[Callable] = None,
                 tp_group=None, layer_number: Optional[int] = None, attention_type: str = "self", cp_group=None,
                 cp_global_ranks: Optional[List[int]] = None, cp_stream=None, cp_comm_type: str = "p2p",
                 softmax_scale: Optional[float] = None, softmax_type: str = "vanilla",
                 return_max_logit: bool = False, bottom_right_diagonal: Optional[bool] = None,
                 name: Optional[str] = None) -> None:
        super().__init__()
        self.bottom_right_diagonal, self.name = bottom_right_diagonal, name
        # return_max_logit: forward returns (output, per-head maximum of the masked scaled scores); the maximum
        # comes from a pass of its own over Q K^T (the attention kernels do not export it)
        self.return_max_logit, self._max_logit = return_max_logit, None
        assert attn_mask_type in _MASK_TYPES, f"unknown attn_mask_type {attn_mask_type}"
        assert qkv_format in ("sbhd", "bshd", "thd")
        self.qkv_format = qkv_format
        self.attn_mask_type = attn_mask_type
        self.window_size = window_size
        self.tp_size = tp_size if tp_group is None else D.get_world_size(tp_group)
        self.tp_group = tp_group
        self.get_rng_state_tracker = get_rng_state_tracker
        self.layer_number = layer_number
        self.attention_type = attention_type
        self.cp_group, self.cp_global_ranks, self.cp_stream, self.cp_comm_type = cp_group, cp_global_ranks, cp_stream, cp_comm_type
        kv = kv_channels if isinstance(kv_channels, int) else kv_channels[0]
        self.hidden_size_per_attention_head = kv
        self.num_gqa_groups = num_attention_heads if num_gqa_groups is None else num_gqa_groups
        self.num_attention_heads = num_attention_heads
        self.num_heads_per_partition = num_attention_heads // self.tp_size
        self.num_gqa_groups_per_partition = max(self.num_gqa_groups // self.tp_size, 1)
        self.softmax_scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(kv)
        self.attention_dropout = attention_dropout
        self.softmax_type = softmax_type
        self.softmax_offset = None
        if softmax_type == "learnable":
            self.softmax_offset = torch.nn.Parameter(torch.zeros(self.num_heads_per_partition,
                                                                 device="cuda" if torch.cuda.is_available() else "cpu"))
        # reference checkpoints carry an (empty) extra state for the core attention
        self.register_load_state_dict_post_hook(self._ignore_missing_extra_state)

    @staticmethod
    def _ignore_missing_extra_state(module, incompatible):
        for k in list(incompatible.missing_keys):
            if k.endswith("_extra_state"):
                incompatible.missing_keys.remove(k)

    def get_extra_state(self):
        return torch.empty(0, dtype=torch.uint8)

    def set_extra_state(self, state):
        return

    def set_context_parallel_group(self, cp_group, cp_global_ranks, cp_stream, cp_comm_type="p2p") -> None:
        self.cp_group, self.cp_global_ranks, self.cp_stream, self.cp_comm_type = cp_group, cp_global_ranks, cp_stream, cp_comm_type

    # ------------------------------------------------------------------
    def forward(self, query_layer: Optional[torch.Tensor] = None, key_layer: Optional[torch.Tensor] = None,
                value_layer: Optional[torch.Tensor] = None, attention_mask=None, qkv_format: Optional[str] = None, cu_seqlens_q: Optional[torch.Tensor] = None,
                cu_seqlens_kv: Optional[torch.Tensor] = None, cu_seqlens_q_padded=None, cu_seqlens_kv_padded=None,
                max_seqlen_q: Optional[int] = None, max_seqlen_kv: Optional[int] = None,
                attn_mask_type: Optional[str] = None, window_size: Optional[Tuple[int, int]] = None,
                checkpoint_core_attention: bool = False, core_attention_bias_type: str = "no_bias",
                core_attention_bias: Optional[torch.Tensor] = None, alibi_slopes: Optional[torch.Tensor] = None,
                fast_zero_fill: bool = True, inference_params=None, pad_between_seqs: Optional[bool] = None,
                score_mod: Optional[Callable] = None, score_mod_bprop: Optional[Callable] = None,
                score_mod_tensors: Optional[Dict[str, torch.Tensor]] = None,
                score_mod_bprop_tensors: Optional[Dict[str, torch.Tensor]] = None,
                bottom_right_diagonal: Optional[bool] = None, fp8_output: bool = False, bf16_backward: bool = False,
                num_splits: Optional[int] = None, qkv_layer: Optional[torch.Tensor] = None,
                kv_layer: Optional[torch.Tensor] = None, qkv_interleave_dim: int = -3):
        """``bottom_right_diagonal``: corner that the sliding window and the ALiBi diagonal are aligned to when
        ``s_q != s_kv`` (None: top-left for ``causal`` / ``padding_causal``, bottom-right otherwise; the causal
        mask types fix it).  ``qkv_layer`` / ``kv_layer``: one packed buffer holding q, k, v (or k, v) along
        ``qkv_interleave_dim`` (-3: ``...3hd``, -2: ``...h3d``) instead of separate tensors; the pieces are
        zero-copy views.  Under a recipe with ``fp8_dpa`` / ``fp8_mha`` the tensors entering and leaving the
        attention are rounded to FP8 (``attention/fp8_emulation.py``; the kernels stay 16-bit): ``fp8_output`` rounds
        the output too, ``bf16_backward`` keeps the gradients unrounded.  ``num_splits`` is accepted for
        compatibility (the kernels choose their own split of the key sequence)."""
        from .fp8_emulation import plan as _fp8_plan
        fp8 = _fp8_plan(fp8_output, bf16_backward)      # recipe.fp8_dpa / fp8_mha, fp8_output: FP8 rounding at the boundaries
        if qkv_layer is not None or kv_layer is not None:
            query_layer, key_layer, value_layer = _unpack_qkv(query_layer, key_layer, value_layer, qkv_layer,
                                                              kv_layer, qkv_interleave_dim, inference_params)
        fmt = qkv_format or self.qkv_format
        mask_type = attn_mask_type or self.attn_mask_type
        brd = self.bottom_right_diagonal if bottom_right_diagonal is None else bottom_right_diagonal
        if mask_type in ("causal", "padding_causal"):
            brd = False
        if brd is None or mask_type in ("causal_bottom_right", "padding_causal_bottom_right"):
            brd = True
        window = window_size if window_size is not None else self.window_size
        # fast_zero_fill is a hint for a zero-filling strategy of padded outputs that these kernels do not need
        # (they write every row of the output); pad_between_seqs is implied by passing padded cumulative lengths
        if pad_between_seqs and fmt == "thd" and cu_seqlens_q_padded is None:
            raise ValueError("pad_between_seqs=True needs cu_seqlens_q_padded / cu_seqlens_kv_padded")
        if (score_mod_bprop is not None or score_mod_bprop_tensors is not None) and score_mod is None:
            raise ValueError("score_mod_bprop without score_mod")
        if fp8 is not None:
            query_layer, key_layer, value_layer = fp8.inputs(query_layer, key_layer, value_layer)
        if inference_params is not None:
            query_layer, key_layer, value_layer, fmt, mask_type, cu_seqlens_q, cu_seqlens_kv = \
                inference_params.step(self.layer_number, query_layer, key_layer, value_layer, fmt, mask_type)
        # score_mod(score, tensors) -> score edits the scaled scores; autograd differentiates it, so the
        # backward callback of the reference's graph-based interface is accepted and not needed
        score = (score_mod, score_mod_tensors)
        assert score_mod is None or (fmt != "thd" and inference_params is None), \
            "score_mod is supported for sbhd / bshd training inputs"
        thd_extra = (cu_seqlens_q_padded, cu_seqlens_kv_padded, max_seqlen_q, max_seqlen_kv) \
            if inference_params is None else (None, None, None, None)
        if checkpoint_core_attention:
            def run(q, k, v):
                return self._core(q, k, v, fmt, mask_type, window, attention_mask, cu_seqlens_q, cu_seqlens_kv,
                                  core_attention_bias_type, core_attention_bias, alibi_slopes, thd_extra, score, brd)
            out = D.checkpoint(run, query_layer, key_layer, value_layer,
                               get_rng_state_tracker=self.get_rng_state_tracker)
            out = out if fp8 is None else fp8.output(out)
            return (out, self._max_logit) if self.return_max_logit else out
        out = self._core(query_layer, key_layer, value_layer, fmt, mask_type, window, attention_mask, cu_seqlens_q,
                         cu_seqlens_kv, core_attention_bias_type, core_attention_bias, alibi_slopes, thd_extra, score,
                         brd)
        if inference_params is not None:
            out = inference_params.unpack_output(out)
        out = out if fp8 is None else fp8.output(out)
        return (out, self._max_logit) if self.return_max_logit else out

    _logged: set = set()

    def _log_backend(self, q, k, v, fmt, mask_type, window, attention_mask, bias_type, score) -> None:
        """``NVTE_DEBUG=1``: one log line per distinct configuration (every call with ``NVTE_DEBUG_LEVEL=2``) naming
        the path taken; level 1 adds the reasons (reference: ``AttentionLogging`` in
        ``attention/dot_product_attention/utils.py``)."""
        import logging

        from .utils import AttentionParams, get_attention_backend
        cfg = get_config()
        thd = fmt == "thd"
        p = AttentionParams(
            qkv_dtype=q.dtype, qkv_format=fmt, num_heads=q.shape[-2], num_gqa_groups=k.shape[-2], head_dim=q.shape[-1],
            head_dim_v=v.shape[-1], max_seqlen_q=q.shape[0] if thd else q.shape[0 if fmt == "sbhd" else 1],
            max_seqlen_kv=k.shape[0] if thd else k.shape[0 if fmt == "sbhd" else 1], attn_mask_type=mask_type,
            window_size=window, core_attention_bias_type=bias_type, attention_dropout=self.attention_dropout,
            softmax_type=self.softmax_type, has_attention_mask=attention_mask is not None,
            score_mod=score[0] is not None,
            context_parallel=self.cp_group is not None and D.get_world_size(self.cp_group) > 1,
            cp_comm_type=self.cp_comm_type, is_training=self.training, device=q.device.type)
        key = (p.qkv_dtype, fmt, p.num_heads, p.num_gqa_groups, p.head_dim, mask_type, window, bias_type,
               p.has_attention_mask, p.attention_dropout > 0 and p.is_training, p.softmax_type, p.device)
        if cfg.debug_level < 2 and key in DotProductAttention._logged:
            return
        DotProductAttention._logged.add(key)
        backend, why = get_attention_backend(p)
        log = logging.getLogger("DotProductAttention")
        log.info("layer %s: %s (format %s, heads %d/%d, head dim %d, mask %s)", self.layer_number, backend, fmt,
                 p.num_heads, p.num_gqa_groups, p.head_dim, mask_type)
        if cfg.debug_level >= 1:
            for w in why:
                log.debug("  %s", w)

    def _core(self, q, k, v, fmt, mask_type, window, attention_mask, cu_q, cu_kv, bias_type, bias, alibi_slopes,
              thd_extra=(None, None, None, None), score=(None, None), bottom_right_diagonal=None):
        if get_config().debug:
            self._log_backend(q, k, v, fmt, mask_type, window, attention_mask, bias_type, score)
        if fmt == "thd":
            if self.return_max_logit:
                raise NotImplementedError("return_max_logit is implemented for sbhd / bshd inputs")
            return self._thd(q, k, v, mask_type, window, cu_q, cu_kv, *thd_extra)
        # -> [b, h, s, d] views
        if fmt == "sbhd":
            qb, kb, vb = (t.permute(1, 2, 0, 3) for t in (q, k, v))
        else:
            qb, kb, vb = (t.permute(0, 2, 1, 3) for t in (q, k, v))
        b, hq, sq, d = qb.shape
        sk = kb.shape[2]
        causal = "causal" in mask_type
        # 'causal' aligns the diagonal to the top-left corner, '*_bottom_right' to the bottom-right one, for
        # self- and cross-attention alike (reference: dot_product_attention.py:1746-1754)
        bottom_right = "bottom_right" in mask_type
        windowed = window is not None and (window[0] >= 0 or window[1] >= 0)
        if bottom_right_diagonal is not None and not causal and (windowed or bias_type == "alibi"):
            # without a causal mask only the sliding window and the ALiBi diagonal have a corner to align to
            bottom_right = bottom_right_diagonal
        mask = None
        if "padding" in mask_type:
            if attention_mask is not None:
                if isinstance(attention_mask, (tuple, list)):
                    mq, mk = attention_mask
                    mask = mq.reshape(b, 1, sq, 1) | mk.reshape(b, 1, 1, sk)
                else:
                    mask = attention_mask
                    if mask.dim() == 4 and mask.shape[-2] == 1 and sq > 1:
                        mask = mask.reshape(b, 1, 1, sk) | mask.reshape(b, 1, sk, 1)[:, :, :sq]
            elif cu_q is not None:
                mask = _padding_mask_from_cu(cu_q, cu_kv if cu_kv is not None else cu_q, sq, sk, qb.device)
        elif mask_type == "arbitrary":
            mask = attention_mask
        the_bias = None
        if bias_type == "alibi":
            the_bias = _alibi_bias(hq, sq, sk, alibi_slopes, qb.device, bottom_right)
        elif bias_type != "no_bias":
            the_bias = bias
        dropout = self.attention_dropout if self.training else 0.0
        if self.cp_group is not None and D.get_world_size(self.cp_group) > 1:
            from ..parallel.context_parallel import attn_forward_func_with_cp

            # the context-parallel paths implement scale / causal / window only: refuse the rest loudly
            unsupported = [name for name, on in (
                ("a padding or arbitrary attention mask", mask is not None),
                ("core_attention_bias / alibi", the_bias is not None),
                ("attention dropout", dropout > 0.0),
                (f"softmax_type={self.softmax_type!r}", self.softmax_type != "vanilla"),
                ("score_mod", score[0] is not None),
                ("bottom-right causal alignment with sq != sk", causal and bottom_right and sq != sk),
                ("return_max_logit", self.return_max_logit),
            ) if on]
            if unsupported:
                raise NotImplementedError("context parallelism does not support: " + "; ".join(unsupported))
            o = attn_forward_func_with_cp(qb, kb, vb, cp_group=self.cp_group, cp_comm_type=self.cp_comm_type,
                                          scale=self.softmax_scale, causal=causal, window=window,
                                          cp_global_ranks=self.cp_global_ranks, cp_stream=self.cp_stream)
        else:
            ctx = self.get_rng_state_tracker().fork() if (self.get_rng_state_tracker is not None and dropout > 0) \
                else _null()
            if self.return_max_logit:
                if score[0] is not None:
                    raise NotImplementedError("return_max_logit with score_mod")
                from ..ops.attention import max_attention_logit
                self._max_logit = max_attention_logit(qb, kb, scale=self.softmax_scale, causal=causal, window=window,
                                                      attn_mask=mask, bias=the_bias,
                                                      bottom_right=bottom_right or sq == sk)
            with ctx:
                o = ops.attention(qb, kb, vb, scale=self.softmax_scale, causal=causal, window=window, attn_mask=mask,
                                  bias=the_bias, dropout_p=dropout, softmax_type=self.softmax_type,
                                  sink=self.softmax_offset, bottom_right=bottom_right or sq == sk,
                                  out_format=fmt, score_mod=score[0], score_mod_tensors=score[1])
        if fmt == "sbhd":
            return o.permute(2, 0, 1, 3).reshape(sq, b, hq * o.shape[-1])
        return o.permute(0, 2, 1, 3).reshape(b, sq, hq * o.shape[-1])

    def _thd(self, q, k, v, mask_type, window, cu_q, cu_kv, cu_q_padded=None, cu_kv_padded=None, max_sq=None,
             max_skv=None):
        """Packed sequences: one launch of the variable-length attention kernels when they apply,
        else one attention call per sequence.  Tokens outside every sequence give zeros."""
        assert cu_q is not None, "thd format needs cu_seqlens_q"
        cu_kv = cu_kv if cu_kv is not None else cu_q
        if cu_kv_padded is None and cu_q_padded is not None and cu_kv is cu_q:
            cu_kv_padded = cu_q_padded
        causal = "causal" in mask_type
        if self.cp_group is not None and D.get_world_size(self.cp_group) > 1:
            # cu_q holds the lengths of this rank's shard (dual-chunk layout of every sequence)
            from ..parallel.context_parallel_thd import thd_ring_attention

            assert self.cp_comm_type == "p2p", "packed sequences support the ring (p2p) context-parallel mode"
            unsupported = [name for name, on in (
                ("a sliding window", window is not None and tuple(window) not in ((-1, -1), (-1, 0))),
                ("bottom-right causal alignment", "bottom_right" in mask_type),
                ("attention dropout", self.training and self.attention_dropout > 0.0),
                (f"softmax_type={self.softmax_type!r}", self.softmax_type != "vanilla"),
            ) if on]
            if unsupported:
                raise NotImplementedError("context parallelism over packed sequences does not support: "
                                          + "; ".join(unsupported))
            o = thd_ring_attention(q, k, v, cu_q, cp_group=self.cp_group, scale=self.softmax_scale, causal=causal,
                                   cp_global_ranks=self.cp_global_ranks, max_seqlen=max_sq)
            return o.reshape(o.shape[0], -1)
        dropout = self.attention_dropout if self.training else 0.0
        if q.is_cuda and dropout == 0.0 and self.softmax_type == "vanilla" and \
                sys.modules[ops.attention.__module__]._USE_OWN_FLASH and flash.supported_varlen(q, k, v):
            o = flash.flash_attention_varlen(q, k, v, cu_q, cu_kv, scale=self.softmax_scale, causal=causal,
                                             bottom_right="bottom_right" in mask_type, max_seqlen_q=max_sq,
                                             max_seqlen_kv=max_skv, cu_seqlens_q_padded=cu_q_padded,
                                             cu_seqlens_kv_padded=cu_kv_padded, window=window)
            return o.reshape(o.shape[0], -1)
        cq, ck = cu_q.tolist(), cu_kv.tolist()
        oq = cq if cu_q_padded is None else cu_q_padded.tolist()
        ok_ = ck if cu_kv_padded is None else cu_kv_padded.tolist()
        out = None
        for i in range(len(cq) - 1):
            lq, lk = cq[i + 1] - cq[i], ck[i + 1] - ck[i]
            if lq == 0:
                continue
            qi = q[oq[i]:oq[i] + lq].permute(1, 0, 2).unsqueeze(0)
            ki = k[ok_[i]:ok_[i] + lk].permute(1, 0, 2).unsqueeze(0)
            vi = v[ok_[i]:ok_[i] + lk].permute(1, 0, 2).unsqueeze(0)
            o = ops.attention(qi, ki, vi, scale=self.softmax_scale, causal=causal, window=window,
                              softmax_type=self.softmax_type, sink=self.softmax_offset,
                              bottom_right="bottom_right" in mask_type or lq == lk)
            o = o.squeeze(0).permute(1, 0, 2)
            if out is None:
                out = o.new_zeros(q.shape[0], *o.shape[1:])
            out = torch.cat([out[:oq[i]], o, out[oq[i] + lq:]], dim=0)  # differentiable placement
        if out is None:
            out = q.new_zeros(q.shape[0], q.shape[1], v.shape[-1])
        return out.reshape(out.shape[0], -1)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def _unpack_qkv(q, k, v, qkv_layer, kv_layer, dim, inference_params):
    """q, k, v as views of a packed buffer (reference: the ``qkv_layer`` / ``kv_layer`` arguments of
    ``DotProductAttention.forward``)."""
    if qkv_layer is not None and kv_layer is not None:
        raise ValueError("qkv_layer and kv_layer are mutually exclusive")
    if inference_params is not None:
        raise ValueError("packed inputs (qkv_layer / kv_layer) are not supported with KV caching")
    if dim not in (-3, -2):
        raise ValueError(f"qkv_interleave_dim must be -3 (e.g. bs3hd) or -2 (e.g. bsh3d), got {dim}")
    packed = qkv_layer if qkv_layer is not None else kv_layer
    if packed.stride(-1) != 1:
        raise ValueError("the packed tensor must have stride 1 in its last dimension")
    if qkv_layer is not None:
        if q is not None or k is not None or v is not None:
            raise ValueError("qkv_layer already packs q, k and v: pass None for query_layer, key_layer, value_layer")
        if qkv_layer.shape[dim] != 3:
            raise ValueError(f"qkv_layer must have size 3 at dim {dim}, got shape {tuple(qkv_layer.shape)}")
        return tuple(qkv_layer.select(dim, i) for i in range(3))
    if q is None:
        raise ValueError("kv_layer packs only k and v: query_layer is required")
    if k is not None or v is not None:
        raise ValueError("kv_layer already packs k and v: pass None for key_layer and value_layer")
    if kv_layer.dim() != q.dim() + 1 or kv_layer.shape[dim] != 2:
        raise ValueError(f"kv_layer must have one more dimension than query_layer and size 2 at dim {dim}, got "
                         f"shape {tuple(kv_layer.shape)}")
    return (q,) + tuple(kv_layer.select(dim, i) for i in range(2))


def _alibi_bias(h, sq, sk, slopes, device, bottom_right=True):
    if slopes is None:
        n = 2 ** math.floor(math.log2(h))
        m0 = 2.0 ** (-8.0 / n)
        slopes = torch.pow(m0, torch.arange(1, 1 + n))
        if n < h:
            m1 = 2.0 ** (-4.0 / n)
            slopes = torch.cat([slopes, torch.pow(m1, torch.arange(1, 1 + 2 * (h - n), 2))])
    slopes = slopes.to(device).float().reshape(1, h, 1, 1)
    qi = torch.arange(sq, device=device)[:, None] + ((sk - sq) if bottom_right else 0)
    ki = torch.arange(sk, device=device)[None, :]
    return -slopes * (qi - ki).abs().float()[None, None]
