"""Statistics of the debug features as mergeable aggregates.

A statistic is collected as a few partial aggregates (minimum, maximum, sums, counts) kept as device
tensors -- no host synchronisation while the model runs.  At ``debug_api.step()`` the aggregates of all
calls of the iteration are merged, reduced over the reduction group (one all-reduce per reduction kind:
MIN, MAX, SUM) and only then turned into the final numbers, so a tensor-parallel or data-parallel job logs
the statistic of the WHOLE tensor / batch, not of one shard (reference:
``debug/features/utils/stats_buffer.py``, ``debug/features/log_tensor_stats.py``,
``log_fp8_tensor_stats.py``, ``log_nvfp4_tensor_stats.py``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

# aggregate name -> how it merges
_KIND = {"min": "min", "max": "max", "absmax": "max", "absmin_nz": "min", "sum": "sum", "sumsq": "sum",
         "abssum": "sum", "numel": "sum", "underflows": "sum", "overflows": "sum", "sqerr": "sum",
         "simin": "min", "simax": "max", "zeros": "sum", "fp4_max_code": "sum"}

# statistic -> aggregates it needs
TENSOR_STATS = {
    "min": ("min",), "max": ("max",), "mean": ("sum", "numel"), "std": ("sum", "sumsq", "numel"),
    "variance": ("sum", "sumsq", "numel"), "l1_norm": ("abssum",), "l2_norm": ("sumsq",),
    "cur_amax": ("absmax",), "amax": ("absmax",), "dynamic_range": ("absmax", "absmin_nz"),
    "zeros%": ("zeros", "numel"),
}
QUANT_STATS = {
    "underflows%": ("underflows", "numel"), "overflows%": ("overflows", "numel"), "mse": ("sqerr", "numel"),
    "scale_inv_min": ("simin",), "scale_inv_max": ("simax",),
    # NVFP4: share of values that land on the largest magnitude code (6.0), a saturation indicator
    "saturated%": ("fp4_max_code", "numel"),
}


def tensor_aggregates(x: torch.Tensor, names) -> Dict[str, torch.Tensor]:
    xf = x.detach().float()
    out: Dict[str, torch.Tensor] = {}
    for n in names:
        if n == "min":
            out[n] = xf.min()
        elif n == "max":
            out[n] = xf.max()
        elif n == "absmax":
            out[n] = xf.abs().max()
        elif n == "absmin_nz":
            a = xf.abs()
            out[n] = torch.where(a > 0, a, torch.full_like(a, float("inf"))).min()
        elif n == "sum":
            out[n] = xf.sum(dtype=torch.float64).float()
        elif n == "sumsq":
            out[n] = xf.square().sum(dtype=torch.float64).float()
        elif n == "abssum":
            out[n] = xf.abs().sum(dtype=torch.float64).float()
        elif n == "numel":
            out[n] = torch.tensor(float(xf.numel()), device=xf.device)
        elif n == "zeros":
            out[n] = (xf == 0).sum().float()
        else:
            raise ValueError(f"unknown aggregate {n}")
    return out


def _scale_inv_of(q) -> Optional[torch.Tensor]:
    s = getattr(q, "_rowwise_scale_inv", None)
    if s is None:
        s = getattr(q, "_scale_inv", None)
    if s is None:
        return None
    if s.dtype == torch.uint8 and getattr(q, "_amax_rowwise", None) is None:
        return torch.exp2(s.float() - 127.0)       # UE8M0 block scales
    if s.dtype == torch.uint8:
        return s.view(torch.float8_e4m3fn).float()  # NVFP4: E4M3 block scales
    return s.float()


def quant_aggregates(x: torch.Tensor, q, names) -> Dict[str, torch.Tensor]:
    xf = x.detach().float()
    dq = q.dequantize().float().reshape(xf.shape)
    out: Dict[str, torch.Tensor] = {}
    for n in names:
        if n == "underflows":
            out[n] = ((dq == 0) & (xf != 0)).sum().float()
        elif n == "overflows":
            out[n] = (dq.abs() < xf.abs() * 0.5).sum().float()
        elif n == "sqerr":
            out[n] = (dq - xf).square().sum(dtype=torch.float64).float()
        elif n == "numel":
            out[n] = torch.tensor(float(xf.numel()), device=xf.device)
        elif n in ("simin", "simax"):
            s = _scale_inv_of(q)
            if s is None:
                out[n] = torch.tensor(float("nan"), device=xf.device)
            else:
                out[n] = s.min() if n == "simin" else s.max()
        elif n == "fp4_max_code":
            data = getattr(q, "_rowwise_data", None)
            if data is None or getattr(q, "_amax_rowwise", None) is None:
                out[n] = torch.tensor(0.0, device=xf.device)
            else:  # two E2M1 codes per byte; magnitude code 7 = 6.0
                lo, hi = data & 0x7, (data >> 4) & 0x7
                out[n] = ((lo == 7).sum() + (hi == 7).sum()).float()
        else:
            raise ValueError(f"unknown aggregate {n}")
    return out


def finalize(stat: str, agg: Dict[str, float]) -> float:
    g = agg.get
    if stat == "min":
        return g("min")
    if stat == "max":
        return g("max")
    if stat in ("cur_amax", "amax"):
        return g("absmax")
    if stat == "mean":
        return g("sum") / max(g("numel"), 1.0)
    if stat in ("std", "variance"):
        n = max(g("numel"), 1.0)
        var = max(g("sumsq") / n - (g("sum") / n) ** 2, 0.0) * (n / max(n - 1.0, 1.0))
        return var if stat == "variance" else var ** 0.5
    if stat == "l1_norm":
        return g("abssum")
    if stat == "l2_norm":
        return g("sumsq") ** 0.5
    if stat == "dynamic_range":
        import math

        lo, hi = g("absmin_nz"), g("absmax")
        return (math.log2(hi) - math.log2(lo)) if (hi > 0 and lo != float("inf")) else 0.0
    if stat == "zeros%":
        return 100.0 * g("zeros") / max(g("numel"), 1.0)
    if stat == "underflows%":
        return 100.0 * g("underflows") / max(g("numel"), 1.0)
    if stat == "overflows%":
        return 100.0 * g("overflows") / max(g("numel"), 1.0)
    if stat == "saturated%":
        return 100.0 * g("fp4_max_code") / max(g("numel"), 1.0)
    if stat == "mse":
        return g("sqerr") / max(g("numel"), 1.0)
    if stat == "scale_inv_min":
        return g("simin")
    if stat == "scale_inv_max":
        return g("simax")
    raise ValueError(f"unknown statistic {stat}")


class StatsBuffer:
    """Aggregates of one iteration, keyed by (layer, tensor, statistic)."""

    def __init__(self):
        self._agg: Dict[Tuple[str, str, str], Dict[str, torch.Tensor]] = {}

    def __len__(self):
        return len(self._agg)

    def feed(self, layer: str, tensor: str, stat: str, agg: Dict[str, torch.Tensor]) -> None:
        cur = self._agg.get((layer, tensor, stat))
        if cur is None:
            self._agg[(layer, tensor, stat)] = dict(agg)
            return
        for k, v in agg.items():  # several calls in one iteration (micro-batches): merge
            kind = _KIND[k]
            cur[k] = torch.minimum(cur[k], v) if kind == "min" else (torch.maximum(cur[k], v) if kind == "max" else cur[k] + v)

    def drain(self, group=None) -> List[Tuple[Tuple[str, str, str], float]]:
        """Reduce over ``group`` (when it has more than one rank), finalize, clear.  Every rank must hold
        the same keys in the same order, which is the case when all ranks run the same model code."""
        import torch.distributed as dist

        if not self._agg:
            return []
        keys = list(self._agg.keys())
        reduce = group is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        if reduce:
            for kind, op in (("min", dist.ReduceOp.MIN), ("max", dist.ReduceOp.MAX), ("sum", dist.ReduceOp.SUM)):
                slots = [(k, a) for k in keys for a in sorted(self._agg[k]) if _KIND[a] == kind]
                if not slots:
                    continue
                flat = torch.stack([self._agg[k][a].double() for k, a in slots])
                dist.all_reduce(flat, op=op, group=group)
                for (k, a), v in zip(slots, flat):
                    self._agg[k][a] = v
        out = []
        for k in keys:
            vals = {a: float(v.item()) for a, v in self._agg[k].items()}
            out.append((k, finalize(k[2], vals)))
        self._agg = {}
        return out
