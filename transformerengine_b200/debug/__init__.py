"""Numerics debugging: per-layer, per-tensor features that wrap a module's quantizers
(reference: ``transformer_engine/debug/pytorch/debug_quantization.py:43,607``,
``debug/features/api.py:21,102,399`` and the feature files next to it).

Configuration is a dict (or a YAML file with the same content)::

    debug_api.initialize({
        "log_attention": {                      # any section name
            "enabled": True,
            "layers": {"layer_name_regex_pattern": ".*self_attention.*"},
            "features": {
                "LogTensorStats": {"tensors": ["activation", "weight"], "stats": ["min", "max", "l2_norm"]},
                "LogFp8TensorStats": {"tensors": ["activation"], "stats": ["underflows%", "mse"]},
                "FakeQuant": {"tensors": ["gradient"], "gemms": ["wgrad"]},
                "DisableQuantizationGEMM": {"gemms": ["dgrad"]},
                "DisableQuantizationLayer": {},
                "DumpTensors": {"tensors": ["activation"], "dir": "dumps"},
            },
        }
    }, log_dir="debug_logs")

Every feature accepts ``freq`` (collect every n-th iteration), ``start_step`` and ``end_step``, and the
reference's ``tensors_struct`` list form (``[{"tensor": "activation", "stats": [...], "freq": 10}, ...]``).
``LogNvfp4TensorStats`` adds ``saturated%`` (share of values on the largest FP4 code).  Statistics are
buffered as mergeable aggregates and, after ``set_tensor_reduction_group(group)``, reduced over that
group at ``debug_api.step()`` so that sharded tensors report one global value (``debug/stats.py``).

Tensor names: ``activation`` (forward input), ``weight``, ``output``, ``gradient`` (grad output),
``dgrad`` (grad input).  A module takes part when it was built with ``name=...`` and a section's
pattern matches the name.  ``debug_api.step()`` advances the iteration counter used in the logs.
"""
from __future__ import annotations

import json
import os
import re
from typing import Any, Dict, List, Optional

import torch

from ..tensor.base import QuantizedTensorStorage, Quantizer
from .stats import QUANT_STATS, TENSOR_STATS, StatsBuffer, quant_aggregates, tensor_aggregates

_FWD_SLOTS = ("activation", "weight", "output")
_BWD_SLOTS = ("gradient", "dgrad")
_GEMM_OF = {"activation": ("fprop", "wgrad"), "weight": ("fprop", "dgrad"), "output": ("fprop",),
            "gradient": ("dgrad", "wgrad"), "dgrad": ("dgrad",)}


def tensor_name_of_slot(fwd: bool, idx: int) -> str:
    names = _FWD_SLOTS if fwd else _BWD_SLOTS
    return names[idx % len(names)]


class _DebugState:
    def __init__(self):
        self.enabled = False
        self.sections: List[Dict[str, Any]] = []
        self.log_dir: Optional[str] = None
        self.iteration = 0
        self.records: List[Dict[str, Any]] = []
        self.reduction_group = None
        self.buffer = StatsBuffer()

    def finalize(self) -> None:
        """Turn the buffered aggregates of the current iteration into records (reducing over the group)."""
        for (layer, tensor, stat), value in self.buffer.drain(self.reduction_group):
            self.records.append({"stat": stat, "value": value, "layer": layer, "tensor": tensor,
                                 "iteration": self.iteration})

    def features_for(self, layer_name: Optional[str]) -> Dict[str, Dict[str, Any]]:
        out: Dict[str, Dict[str, Any]] = {}
        if not self.enabled or layer_name is None:
            return out
        for sec in self.sections:
            if not sec.get("enabled", True):
                continue
            layers = sec.get("layers", {})
            pat = layers.get("layer_name_regex_pattern")
            names = layers.get("layer_names")
            if (pat and re.search(pat, layer_name)) or (names and layer_name in names) or (not pat and not names):
                out.update(sec.get("features", sec.get("transformer_engine", {})))
        return out


_STATE = _DebugState()


class debug_api:  # noqa: N801  (namespace with the reference's spelling)
    @staticmethod
    def initialize(config=None, feature_dirs=None, log_dir: Optional[str] = None, default_logging_enabled=True):
        if isinstance(config, str):
            import yaml

            with open(config) as f:
                config = yaml.safe_load(f)
        _STATE.sections = list((config or {}).values())
        _STATE.enabled = True
        _STATE.log_dir = log_dir
        _STATE.iteration = 0
        _STATE.records = []
        _STATE.buffer = StatsBuffer()
        if log_dir:
            os.makedirs(log_dir, exist_ok=True)

    @staticmethod
    def step():
        """End of an iteration: reduce and record its statistics, then advance the iteration counter."""
        _STATE.finalize()
        _STATE.iteration += 1

    @staticmethod
    def end_debug():
        debug_api.flush()
        _STATE.enabled = False
        _STATE.sections = []

    @staticmethod
    def set_tensor_reduction_group(group):
        _STATE.reduction_group = group

    @staticmethod
    def flush():
        _STATE.finalize()
        if _STATE.log_dir and _STATE.records:
            with open(os.path.join(_STATE.log_dir, "tensor_stats.jsonl"), "a") as f:
                for r in _STATE.records:
                    f.write(json.dumps(r) + "\n")
            _STATE.records = []

    @staticmethod
    def records() -> List[Dict[str, Any]]:
        _STATE.finalize()
        return _STATE.records


def _active_now(cfg: Dict[str, Any]) -> bool:
    """``freq`` / ``start_step`` / ``end_step`` window of a feature (or of one tensors_struct entry)."""
    it = _STATE.iteration
    if it < int(cfg.get("start_step", 0)):
        return False
    end = cfg.get("end_step")
    if end is not None and it > int(end):
        return False
    freq = int(cfg.get("freq", 1))
    return freq <= 1 or (it - int(cfg.get("start_step", 0))) % freq == 0


def _entries(cfg: Dict[str, Any], tensor: str):
    """The settings that apply to ``tensor`` now: the feature's own (``tensors`` / ``stats``) and every
    matching ``tensors_struct`` entry, each filtered by its time window."""
    out = []
    g = cfg.get("gemms")
    if g is not None and not any(x in g for x in _GEMM_OF[tensor]):
        return out
    struct = cfg.get("tensors_struct")
    if struct:
        for e in struct:
            merged = {k: v for k, v in cfg.items() if k != "tensors_struct"}
            merged.update(e)
            if merged.get("tensor", tensor) == tensor and _active_now(merged):
                out.append(merged)
        return out
    t = cfg.get("tensors")
    if (t is None or tensor in t) and _active_now(cfg):
        out.append(cfg)
    return out


def _wants(cfg: Dict[str, Any], tensor: str) -> bool:
    return bool(_entries(cfg, tensor))


class DebugQuantizer(Quantizer):
    """Wraps a module's quantizer and applies the configured debug features on every call."""

    def __init__(self, parent: Optional[Quantizer], layer_name: str, tensor_name: str, features: Dict[str, Dict]):
        super().__init__(rowwise=True, columnwise=True)
        self.parent, self.layer_name, self.tensor_name, self.features = parent, layer_name, tensor_name, features
        if parent is not None:
            self.rowwise_usage, self.columnwise_usage = parent.rowwise_usage, parent.columnwise_usage

    def set_usage(self, *, rowwise=None, columnwise=None):
        super().set_usage(rowwise=rowwise, columnwise=columnwise)
        if self.parent is not None:
            self.parent.set_usage(rowwise=rowwise, columnwise=columnwise)

    def __getattr__(self, name):  # delegate recipe-specific attributes (dtype, scale, amax ...)
        parent = self.__dict__.get("parent")
        if parent is None:
            raise AttributeError(name)
        return getattr(parent, name)

    def quantize_impl(self, tensor, dtype=None):
        f = self.features
        if "LogTensorStats" in f:
            for e in _entries(f["LogTensorStats"], self.tensor_name):
                for s in e.get("stats", ["min", "max", "mean", "std"]):
                    if s not in TENSOR_STATS:
                        raise ValueError(f"LogTensorStats: unknown statistic {s!r}")
                    _STATE.buffer.feed(self.layer_name, self.tensor_name, s, tensor_aggregates(tensor, TENSOR_STATS[s]))
        if "DumpTensors" in f and _wants(f["DumpTensors"], self.tensor_name) and _STATE.log_dir:
            d = os.path.join(_STATE.log_dir, f["DumpTensors"].get("dir", "dumps"))
            os.makedirs(d, exist_ok=True)
            torch.save(tensor.detach().cpu(), os.path.join(
                d, f"{self.layer_name}.{self.tensor_name}.{_STATE.iteration}.pt".replace("/", "_")))
        q = self.parent.quantize_impl(tensor, dtype) if self.parent is not None else tensor
        for feat in ("LogFp8TensorStats", "LogNvfp4TensorStats"):
            if feat in f and isinstance(q, QuantizedTensorStorage):
                for e in _entries(f[feat], self.tensor_name):
                    for s in e.get("stats", ["underflows%", "mse"]):
                        if s not in QUANT_STATS:
                            raise ValueError(f"{feat}: unknown statistic {s!r}")
                        _STATE.buffer.feed(self.layer_name, self.tensor_name, s,
                                           quant_aggregates(tensor, q, QUANT_STATS[s]))
        return q

    def make_empty(self, shape, *, dtype=torch.float32, device=None, requires_grad=False):
        return self.parent.make_empty(shape, dtype=dtype, device=device, requires_grad=requires_grad)

    def update_quantized(self, src, dst, *, noop_flag=None):
        return self.parent.update_quantized(src, dst, noop_flag=noop_flag)

    def copy(self):
        return DebugQuantizer(self.parent.copy() if self.parent is not None else None, self.layer_name,
                              self.tensor_name, self.features)


class _FakeQuantizer(Quantizer):
    """Quantize-dequantize: the GEMM runs in high precision on values rounded to the low-precision grid."""

    def __init__(self, parent: Quantizer):
        super().__init__(rowwise=True, columnwise=False)
        self.parent = parent

    def quantize_impl(self, tensor, dtype=None):
        p = self.parent.copy()
        p.set_usage(rowwise=True, columnwise=False)
        return p.quantize_impl(tensor, dtype).dequantize().to(tensor.dtype)

    def update_quantized(self, src, dst, *, noop_flag=None):
        dst.copy_(self.quantize_impl(src))
        return dst

    def make_empty(self, shape, *, dtype=torch.float32, device=None, requires_grad=False):
        return torch.empty(tuple(shape), dtype=dtype, device=device, requires_grad=requires_grad)

    def copy(self):
        return _FakeQuantizer(self.parent.copy())


def wrap_quantizer(parent: Optional[Quantizer], layer_name: Optional[str], fwd: bool, idx: int):
    """Called by modules for every quantizer slot; returns the quantizer the module should use."""
    feats = _STATE.features_for(layer_name)
    if not feats:
        return parent
    tname = tensor_name_of_slot(fwd, idx)
    if "DisableQuantizationLayer" in feats or "DisableFP8Layer" in feats:
        return None
    for key in ("DisableQuantizationGEMM", "DisableFP8GEMM"):
        if key in feats and _wants(feats[key], tname):
            return None
    if parent is None:
        return None
    if isinstance(parent, DebugQuantizer):
        return parent
    if "PerTensorScaling" in feats and _wants(feats["PerTensorScaling"], tname):
        # replace the recipe's quantizer by FP8 per-tensor current scaling for the chosen tensors
        # (reference: debug/features/per_tensor_scaling.py:61)
        from ..tensor.float8 import Float8CurrentScalingQuantizer

        fp8_dtype = getattr(parent, "dtype", None)
        if fp8_dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
            fp8_dtype = torch.float8_e4m3fn if fwd else torch.float8_e5m2
        swapped = Float8CurrentScalingQuantizer(fp8_dtype, rowwise=parent.rowwise_usage,
                                                columnwise=parent.columnwise_usage)
        swapped.internal = parent.internal
        parent = swapped
    if "FakeQuant" in feats and _wants(feats["FakeQuant"], tname):
        parent = _FakeQuantizer(parent)
    return DebugQuantizer(parent, layer_name, tname, feats)


def is_enabled() -> bool:
    return _STATE.enabled
