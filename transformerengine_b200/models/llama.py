"""Llama-architecture decoder built from the library's public modules: RMSNorm,
GQA attention with RoPE, SwiGLU MLP, untied embeddings, fused cross entropy.

Parallel layouts: single GPU, data parallel (replicated model, gradient
all-reduce) and tensor parallel with sequence parallelism (Megatron column/row
sharding, vocab-parallel embedding and loss).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..attention.rope import RotaryPositionEmbedding
from ..modules.layernorm_linear import RMSNorm
from ..modules.linear import Linear
from ..parallel import distributed as D
from ..transformer import TransformerLayer


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    ffn_hidden_size: int = 14336
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0
    init_std: float = 0.02
    params_dtype: torch.dtype = torch.bfloat16
    recompute: bool = False  # recompute each layer's activations in backward
    quantize_lm_head: bool = True
    # Variations on the architecture, used by the sibling families (Mistral, Gemma, Qwen3); the defaults are Llama's.
    head_dim: Optional[int] = None            # None: hidden_size // num_heads
    activation: str = "swiglu"                # gated activation of the MLP ("geglu" for Gemma)
    zero_centered_gamma: bool = False         # norm weights stored as (gamma - 1)
    embedding_scale: Optional[float] = None   # multiply the token embeddings (Gemma: sqrt(hidden_size))
    tie_embeddings: bool = False              # the output head shares the embedding table
    sliding_window: Optional[int] = None      # attend to the last N tokens only (Mistral)
    qk_norm: bool = False                     # RMSNorm over each head of q and k, before the rotation (Qwen3)
    qk_norm_eps: float = 1e-6

    @staticmethod
    def llama3_8b(**kw) -> "LlamaConfig":
        return LlamaConfig(**kw)

    @staticmethod
    def llama3_70b(num_layers: int = 80, **kw) -> "LlamaConfig":
        return LlamaConfig(hidden_size=8192, num_layers=num_layers, num_heads=64, num_kv_heads=8,
                           ffn_hidden_size=28672, **kw)

    @staticmethod
    def tiny(**kw) -> "LlamaConfig":
        d = dict(vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, ffn_hidden_size=512)
        d.update(kw)
        return LlamaConfig(**d)

    @property
    def dim_per_head(self) -> int:
        return self.head_dim or self.hidden_size // self.num_heads

    def num_params(self) -> int:
        h, f, v = self.hidden_size, self.ffn_hidden_size, self.vocab_size
        hd = self.dim_per_head
        q = self.num_heads * hd
        per_layer = h * (q + 2 * self.num_kv_heads * hd) + q * h + 3 * h * f + 2 * h + (2 * hd if self.qk_norm else 0)
        return self.num_layers * per_layer + (1 if self.tie_embeddings else 2) * v * h + h

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token (fwd+bwd = 3x forward; causal attention counts half the square)."""
        h, f, v = self.hidden_size, self.ffn_hidden_size, self.vocab_size
        hd = self.dim_per_head
        q = self.num_heads * hd
        gemm = self.num_layers * (h * (q + 2 * self.num_kv_heads * hd) + q * h + 3 * h * f) + v * h
        span = min(seq_len, 2 * self.sliding_window) if self.sliding_window else seq_len
        attn = self.num_layers * 2 * span * q / 2  # QK^T and PV, causal
        return 6.0 * gemm + 6.0 * attn


class VocabParallelEmbedding(torch.nn.Module):
    """Embedding table sharded over the vocabulary; out-of-shard ids contribute zeros and the
    partial results are summed (reduce-scattered along the sequence with sequence parallelism)."""

    def __init__(self, vocab_size, hidden, tp_group=None, sequence_parallel=False, dtype=torch.bfloat16, device=None,
                 init_std=0.02):
        super().__init__()
        self.tp_group = tp_group
        self.tp_size = D.get_world_size(tp_group) if tp_group is not None else 1
        self.rank = D.get_rank(tp_group) if tp_group is not None else 0
        self.sequence_parallel = sequence_parallel and self.tp_size > 1
        assert vocab_size % self.tp_size == 0
        self.per = vocab_size // self.tp_size
        self.start = self.rank * self.per
        self.weight = torch.nn.Parameter(torch.empty(self.per, hidden, dtype=dtype, device=device).normal_(0, init_std))
        if self.tp_size > 1:
            D.set_tensor_model_parallel_attributes(self.weight, True, 0, 1)

    def forward(self, ids_sb: torch.Tensor) -> torch.Tensor:
        """ids [s, b] -> [s(/tp), b, h]"""
        if self.tp_size == 1:
            return torch.nn.functional.embedding(ids_sb, self.weight)
        local = ids_sb - self.start
        oob = (local < 0) | (local >= self.per)
        x = torch.nn.functional.embedding(local.masked_fill(oob, 0), self.weight)
        x = x.masked_fill(oob[..., None], 0)
        return _ReduceFromTP.apply(x, self.tp_group, self.sequence_parallel)


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, sp):  # type: ignore[override]
        ctx.group, ctx.sp = group, sp
        if sp:
            out, _ = D.reduce_scatter_along_first_dim(x, group)
            return out
        out, _ = D.allreduce(x.contiguous(), group)
        return out

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        if ctx.sp:
            out, _ = D.gather_along_first_dim(g.contiguous(), ctx.group)
            return out, None, None
        return g, None, None


class _GatherFromSP(torch.autograd.Function):
    """All-gather along the sequence dim; backward reduce-scatters."""

    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        ctx.group = group
        out, _ = D.gather_along_first_dim(x.contiguous(), group)
        return out

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        out, _ = D.reduce_scatter_along_first_dim(g.contiguous(), ctx.group)
        return out, None


class _FusedCrossEntropy(torch.autograd.Function):
    """Mean token loss over a (possibly vocab-sharded) logits tensor.

    Forward reads the logits once for the per-row max / sum-exp / target logit;
    backward overwrites the logits buffer with the gradient, scaled on the device
    by the incoming gradient, so no separate scaling pass runs.
    """

    @staticmethod
    def forward(ctx, logits, labels, tp_group, vocab_start):  # type: ignore[override]
        valid = (labels != -100).sum().clamp(min=1).float()
        m, s, t = ops.cross_entropy_stats(logits, labels, vocab_start)
        if tp_group is not None and D.get_world_size(tp_group) > 1:
            gm = m.clone()
            dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=tp_group)
            st = torch.stack([s * torch.exp(m - gm), t])
            dist.all_reduce(st, group=tp_group)
            gs, gt = st[0], st[1]
        else:
            gm, gs, gt = m, s, t
        loss_rows = torch.where(labels.reshape(-1) == -100, torch.zeros_like(gs), gm + torch.log(gs) - gt)
        ctx.save_for_backward(logits, labels, gm, gs, valid)
        ctx.vocab_start = vocab_start
        return loss_rows.sum() / valid

    @staticmethod
    def backward(ctx, go):  # type: ignore[override]
        logits, labels, gm, gs, valid = ctx.saved_tensors
        grad = ops.cross_entropy_parallel_grad(logits, labels, gm, gs, ctx.vocab_start, 1.0, inplace_grad=True,
                                               grad_scale_dev=(go.float() / valid))
        return grad, None, None, None


class LlamaModel(torch.nn.Module):
    def __init__(self, cfg: LlamaConfig, tp_group=None, sequence_parallel: bool = True, device=None):
        super().__init__()
        self.cfg = cfg
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.tp_group = tp_group
        self.tp_size = D.get_world_size(tp_group) if tp_group is not None else 1
        self.sp = sequence_parallel and self.tp_size > 1
        init = lambda t: torch.nn.init.normal_(t, 0.0, cfg.init_std)  # noqa: E731
        self.embedding = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, tp_group, self.sp, cfg.params_dtype,
                                                device, cfg.init_std)
        window = (cfg.sliding_window - 1, 0) if cfg.sliding_window else None
        self.layers = torch.nn.ModuleList([
            TransformerLayer(cfg.hidden_size, cfg.ffn_hidden_size, cfg.num_heads, num_gqa_groups=cfg.num_kv_heads,
                             layernorm_epsilon=cfg.rms_eps, hidden_dropout=0.0, attention_dropout=0.0,
                             init_method=init, output_layer_init_method=init, layer_number=i + 1,
                             kv_channels=cfg.head_dim, self_attn_mask_type="causal", window_size=window,
                             tp_group=tp_group, tp_size=self.tp_size,
                             params_dtype=cfg.params_dtype, sequence_parallel=self.sp,
                             set_parallel_mode=self.tp_size > 1, fuse_qkv_params=True, qkv_weight_interleaved=False,
                             zero_centered_gamma=cfg.zero_centered_gamma,
                             bias=False, activation=cfg.activation, normalization="RMSNorm", device=device,
                             attn_input_format="sbhd", qk_norm_type="RMSNorm" if cfg.qk_norm else None,
                             qk_norm_eps=cfg.qk_norm_eps, qk_norm_before_rope=True)
            for i in range(cfg.num_layers)])
        self.final_norm = RMSNorm(cfg.hidden_size, eps=cfg.rms_eps, sequence_parallel=self.sp,
                                  params_dtype=cfg.params_dtype, zero_centered_gamma=cfg.zero_centered_gamma,
                                  device=device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, bias=False, init_method=init,
                              params_dtype=cfg.params_dtype, device=device, tp_group=tp_group, tp_size=self.tp_size,
                              parallel_mode="column" if self.tp_size > 1 else None, sequence_parallel=self.sp)
        if cfg.tie_embeddings:
            # one table for both ends (vocabulary-sharded the same way under tensor parallelism)
            self.lm_head.weight = self.embedding.weight
        self.rope = RotaryPositionEmbedding(cfg.dim_per_head, rotary_base=cfg.rope_theta)
        self._rope_cache = {}

    def _freqs(self, s: int, device):
        f = self._rope_cache.get((s, str(device)))
        if f is None:
            f = self.rope(s).to(device)
            self._rope_cache[(s, str(device))] = f
        return f

    logits_seq_first = True  # forward returns [s, b, vocab]

    def make_inference_params(self, max_batch_size: int, max_sequence_length: int, **kw):
        """Key/value cache for incremental decoding with this model (``is_paged``, ``page_size``,
        ``total_num_pages`` pass through to ``InferenceParams``)."""
        from ..attention.inference import InferenceParams
        cfg = self.cfg
        p = next(self.parameters())
        kw.setdefault("device", p.device)
        return InferenceParams(max_batch_size, max_sequence_length, num_heads_kv=cfg.num_kv_heads // self.tp_size,
                               head_dim_k=cfg.dim_per_head, dtype=cfg.params_dtype,
                               qkv_format="sbhd", **kw)

    def generate(self, prompt: torch.Tensor, max_new_tokens: int, **kw) -> torch.Tensor:
        """Decoding on the key/value cache; see ``models.generation.generate`` for the options."""
        from .generation import generate
        return generate(self, prompt, max_new_tokens, **kw)

    def forward(self, tokens: torch.Tensor, labels: Optional[torch.Tensor] = None, inference_params=None):
        """tokens [b, s] int64.  Returns the mean next-token loss when ``labels`` is given
        (labels are shifted inside), else logits ``[s, b, vocab(/tp)]``.  With ``inference_params`` the tokens
        are the NEW tokens of each sequence (``inference_params.pre_step`` names their counts) and attention
        runs against the key/value cache."""
        b, s = tokens.shape
        ids = tokens.t().contiguous()  # [s, b]
        x = self.embedding(ids)
        if self.cfg.embedding_scale is not None:
            x = x * torch.tensor(self.cfg.embedding_scale, dtype=x.dtype)   # rounded to the activation dtype first
        if inference_params is not None:
            assert not self.sp, "incremental decoding runs without sequence parallelism"
            freqs = self._freqs(inference_params.max_sequence_length, x.device)
        else:
            freqs = self._freqs(s, x.device)
        for layer in self.layers:
            if inference_params is not None:
                x = layer(x, rotary_pos_emb=freqs, inference_params=inference_params)
            elif self.cfg.recompute and torch.is_grad_enabled():
                x = D.checkpoint(layer, x, rotary_pos_emb=freqs)
            else:
                x = layer(x, rotary_pos_emb=freqs)
        x = self.final_norm(x)
        if self.cfg.quantize_lm_head:
            logits = self.lm_head(x)
        else:
            from ..quantization import autocast
            with autocast(enabled=False):
                logits = self.lm_head(x)
        if labels is None:
            return logits
        # next-token targets, [s, b] order to match the logits
        tgt = torch.full_like(ids, -100)
        tgt[:-1] = labels.t()[1:]
        vocab_start = D.get_rank(self.tp_group) * (self.cfg.vocab_size // self.tp_size) if self.tp_size > 1 else 0
        return _FusedCrossEntropy.apply(logits, tgt, self.tp_group if self.tp_size > 1 else None, vocab_start)
