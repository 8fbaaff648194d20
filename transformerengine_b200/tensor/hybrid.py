"""Identity and hybrid quantizers.

``IdentityQuantizer`` keeps the tensor in high precision behind the quantized-tensor interface, so a
custom recipe can leave a role unquantized without special cases in the modules.
``HybridQuantizer`` composes two quantizers: one builds the rowwise copy (read by GEMMs that contract
over the last dim), the other the columnwise copy (GEMMs that contract over the leading dims), e.g.
MXFP8 forward operands with NVFP4 backward operands.  The GEMM front end picks the child that
matches the requested usage (``ops/gemm.py: as_operand``).
(Reference: ``pytorch/tensor/identity_tensor.py:26,172``, ``pytorch/tensor/hybrid_tensor.py:19``.)
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch

from .base import QuantizedTensor, QuantizedTensorStorage, Quantizer


# ------------------------------------------------------------------------------------ identity
class IdentityTensorStorage(QuantizedTensorStorage):
    def __init__(self, *, data: Optional[torch.Tensor], quantizer=None, shape=None, dtype=None):
        self._data = data
        self._quantizer = quantizer
        self._shape = tuple(shape if shape is not None else data.shape)
        self._dtype = dtype if dtype is not None else data.dtype

    def dequantize(self, *, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return self._data.to(dtype or self._dtype)

    def update_usage(self, rowwise_usage=None, columnwise_usage=None) -> None:
        pass  # one copy serves both directions

    def get_usages(self):
        return {"rowwise": self._data is not None, "columnwise": self._data is not None}

    def get_data_tensors(self):
        return (self._data,)

    def prepare_for_saving(self):
        t, self._data = [self._data], None
        return t, self

    def restore_from_saved(self, tensors: list) -> list:
        self._data = tensors[0]
        return tensors[1:]


class IdentityTensor(IdentityTensorStorage, QuantizedTensor):
    def __new__(cls, *, data, quantizer=None, shape=None, dtype=None, requires_grad=False):
        shape = tuple(shape if shape is not None else data.shape)
        dtype = dtype if dtype is not None else data.dtype
        self = QuantizedTensor.__new__(cls, shape=shape, dtype=dtype, requires_grad=requires_grad, device=data.device)
        IdentityTensorStorage.__init__(self, data=data, quantizer=quantizer, shape=shape, dtype=dtype)
        return self

    def __init__(self, *a, **k):
        pass

    def dequantize(self, *, dtype=None):
        return QuantizedTensor.dequantize(self, dtype=dtype)

    def _dequantize_impl(self, dtype):
        return IdentityTensorStorage.dequantize(self, dtype=dtype)

    def _new_like(self, requires_grad=None, clone=False, dtype=None):
        return IdentityTensor(data=self._data.clone() if clone else self._data, quantizer=self._quantizer,
                              shape=self._shape, dtype=dtype or self._dtype,
                              requires_grad=self.requires_grad if requires_grad is None else requires_grad)

    def __reduce_ex__(self, protocol):
        return (_make_identity_tensor_in_reduce_ex, (self._data, self._dtype, self._shape))


def _make_identity_tensor_in_reduce_ex(data, dtype, shape):
    return IdentityTensor(data=data, dtype=dtype, shape=shape)


class IdentityQuantizer(Quantizer):
    """Keeps values as they are (optionally cast to ``dtype``)."""

    def __init__(self, *, dtype: Optional[torch.dtype] = None, rowwise: bool = True, columnwise: bool = True):
        super().__init__(rowwise=rowwise, columnwise=columnwise)
        self.dtype = dtype

    def _cast(self, t: torch.Tensor) -> torch.Tensor:
        return t if self.dtype is None or t.dtype == self.dtype else t.to(self.dtype)

    def quantize_impl(self, tensor: torch.Tensor, dtype=None):
        data = self._cast(tensor.detach())
        if self.internal:
            return IdentityTensorStorage(data=data, quantizer=self, shape=tensor.shape, dtype=dtype or tensor.dtype)
        return IdentityTensor(data=data, quantizer=self, shape=tensor.shape, dtype=dtype or tensor.dtype)

    def update_quantized(self, src: torch.Tensor, dst, *, noop_flag=None):
        if isinstance(src, QuantizedTensorStorage):
            src = src.dequantize()
        new = self._cast(src.detach())
        if noop_flag is not None:  # keep the old values where the flag is set (CUDA-graph weight caching)
            new = torch.where(noop_flag.reshape(()).bool(), dst._data, new.to(dst._data.dtype))
        if dst._data is not None and dst._data.shape == new.shape and dst._data.dtype == new.dtype:
            dst._data.copy_(new)
        else:
            dst._data = new.clone()
        return dst

    def make_empty(self, shape: Iterable[int], *, dtype=torch.float32, device=None, requires_grad=False,
                   pin_memory: bool = False):
        data = torch.empty(tuple(shape), dtype=self.dtype or dtype, device=device, pin_memory=pin_memory)
        return IdentityTensor(data=data, quantizer=self, shape=tuple(shape), dtype=dtype, requires_grad=requires_grad)

    def is_requantization_safe(self) -> bool:
        return True


# ------------------------------------------------------------------------------------ hybrid
class HybridQuantizedTensorStorage(QuantizedTensorStorage):
    """Two quantized tensors of the same logical matrix: ``_rowwise`` carries the rowwise copy,
    ``_columnwise`` the columnwise copy (possibly in another format)."""

    def __init__(self, *, rowwise, columnwise, quantizer=None, shape=None, dtype=torch.float32):
        self._rowwise, self._columnwise = rowwise, columnwise
        self._quantizer = quantizer
        ref = rowwise if rowwise is not None else columnwise
        self._shape = tuple(shape if shape is not None else ref.logical_shape)
        self._dtype = dtype

    def dequantize(self, *, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        src = self._rowwise if self._rowwise is not None else self._columnwise
        assert src is not None, "hybrid tensor holds no data"
        return src.dequantize(dtype=dtype or self._dtype)

    def update_usage(self, rowwise_usage=None, columnwise_usage=None) -> None:
        if rowwise_usage is False:
            self._rowwise = None
        if columnwise_usage is False:
            self._columnwise = None

    def get_usages(self):
        return {"rowwise": self._rowwise is not None, "columnwise": self._columnwise is not None}

    def get_data_tensors(self):
        out = ()
        for child in (self._rowwise, self._columnwise):
            if child is not None:
                out += tuple(child.get_data_tensors())
        return out

    def prepare_for_saving(self):
        tensors = []
        self._saved_counts = []
        for child in (self._rowwise, self._columnwise):
            if child is None:
                self._saved_counts.append(0)
                continue
            ts, _ = child.prepare_for_saving()
            tensors.extend(ts)
            self._saved_counts.append(len(ts))
        return tensors, self

    def restore_from_saved(self, tensors: list) -> list:
        for child, n in zip((self._rowwise, self._columnwise), self._saved_counts):
            if child is not None:
                rest = child.restore_from_saved(list(tensors[:n]))
                assert not rest
            tensors = tensors[n:]
        return list(tensors)


class HybridQuantizedTensor(HybridQuantizedTensorStorage, QuantizedTensor):
    def __new__(cls, *, rowwise, columnwise, quantizer=None, shape=None, dtype=torch.float32, requires_grad=False):
        ref = rowwise if rowwise is not None else columnwise
        shape = tuple(shape if shape is not None else ref.logical_shape)
        self = QuantizedTensor.__new__(cls, shape=shape, dtype=dtype, requires_grad=requires_grad, device=ref.device)
        HybridQuantizedTensorStorage.__init__(self, rowwise=rowwise, columnwise=columnwise, quantizer=quantizer,
                                              shape=shape, dtype=dtype)
        return self

    def __init__(self, *a, **k):
        pass

    def dequantize(self, *, dtype=None):
        return QuantizedTensor.dequantize(self, dtype=dtype)

    def _dequantize_impl(self, dtype):
        return HybridQuantizedTensorStorage.dequantize(self, dtype=dtype)

    def _new_like(self, requires_grad=None, clone=False, dtype=None):
        def dup(c):
            if c is None or not clone:
                return c
            return c.clone() if isinstance(c, torch.Tensor) else c

        return HybridQuantizedTensor(rowwise=dup(self._rowwise), columnwise=dup(self._columnwise),
                                     quantizer=self._quantizer, shape=self._shape, dtype=dtype or self._dtype,
                                     requires_grad=self.requires_grad if requires_grad is None else requires_grad)

    def __reduce_ex__(self, protocol):
        return (_make_hybrid_tensor_in_reduce_ex, (self._rowwise, self._columnwise, self._dtype, self._shape))


def _make_hybrid_tensor_in_reduce_ex(rowwise, columnwise, dtype, shape):
    return HybridQuantizedTensor(rowwise=rowwise, columnwise=columnwise, dtype=dtype, shape=shape)


class HybridQuantizer(Quantizer):
    """``rowwise_quantizer`` builds the rowwise copy, ``columnwise_quantizer`` the columnwise one.

    ``columnwise_source="rowwise_dequantized"`` quantizes the columnwise copy from the dequantized
    rowwise copy (double quantization: both directions see the same rounded values).  The quantizer
    takes ownership of its children and pins each to its direction."""

    _SOURCES = ("original", "rowwise_dequantized")

    def __init__(self, *, rowwise_quantizer: Quantizer, columnwise_quantizer: Quantizer,
                 columnwise_source: str = "original"):
        super().__init__(rowwise=True, columnwise=True)
        for name, q in (("rowwise", rowwise_quantizer), ("columnwise", columnwise_quantizer)):
            if not isinstance(q, Quantizer) and not getattr(q, "_is_quantizer_request", False):
                raise TypeError(f"the {name} quantizer must be a Quantizer (or a QuantizerRequest that the recipe "
                                f"state resolves), got {type(q).__name__}")
        if rowwise_quantizer is columnwise_quantizer and isinstance(rowwise_quantizer, Quantizer):
            raise ValueError("the rowwise and columnwise quantizers must be distinct objects")
        if columnwise_source not in self._SOURCES:
            raise ValueError(f"columnwise_source must be one of {self._SOURCES}")
        self.columnwise_source = columnwise_source
        self.set_child("rowwise_quantizer", rowwise_quantizer)
        self.set_child("columnwise_quantizer", columnwise_quantizer)

    def set_child(self, side: str, q) -> None:
        """Install a child and pin it to its direction.  A ``QuantizerRequest`` is kept as a placeholder until the
        recipe state that owns this quantizer replaces it (``CustomRecipeState.make_quantizers``)."""
        assert side in ("rowwise_quantizer", "columnwise_quantizer")
        setattr(self, side, q)
        if isinstance(q, Quantizer):
            q.set_usage(rowwise=side == "rowwise_quantizer", columnwise=side == "columnwise_quantizer")

    def _resolved(self) -> None:
        for side in ("rowwise_quantizer", "columnwise_quantizer"):
            if not isinstance(getattr(self, side), Quantizer):
                raise RuntimeError(f"HybridQuantizer.{side} is an unresolved {type(getattr(self, side)).__name__}: "
                                   "requests are resolved when a CustomRecipe factory returns the quantizer to a module")

    def copy(self) -> "HybridQuantizer":
        self._resolved()
        q = HybridQuantizer(rowwise_quantizer=self.rowwise_quantizer.copy(),
                            columnwise_quantizer=self.columnwise_quantizer.copy(),
                            columnwise_source=self.columnwise_source)
        q.set_usage(rowwise=self.rowwise_usage, columnwise=self.columnwise_usage)
        q.internal = self.internal
        return q

    def _children(self, tensor: torch.Tensor):
        self._resolved()
        need_row = self.rowwise_usage or (self.columnwise_usage and self.columnwise_source == "rowwise_dequantized")
        row = col = None
        for q in (self.rowwise_quantizer, self.columnwise_quantizer):
            q.internal = True
        if need_row:
            row = self.rowwise_quantizer.quantize_impl(tensor)
        if self.columnwise_usage:
            src = tensor if self.columnwise_source == "original" else row.dequantize(dtype=tensor.dtype)
            col = self.columnwise_quantizer.quantize_impl(src)
        if not self.rowwise_usage:
            row = None
        return row, col

    def quantize_impl(self, tensor: torch.Tensor, dtype=None):
        tensor = tensor.detach()
        row, col = self._children(tensor)
        cls = HybridQuantizedTensorStorage if self.internal else HybridQuantizedTensor
        return cls(rowwise=row, columnwise=col, quantizer=self, shape=tensor.shape, dtype=dtype or tensor.dtype)

    def update_quantized(self, src: torch.Tensor, dst, *, noop_flag=None):
        if isinstance(src, QuantizedTensorStorage):
            src = src.dequantize()
        row, col = self._children(src.detach())
        if noop_flag is not None and bool(noop_flag.reshape(-1)[0]):
            return dst
        dst._rowwise, dst._columnwise = row, col
        return dst

    def make_empty(self, shape: Iterable[int], *, dtype=torch.float32, device=None, requires_grad=False,
                   pin_memory: bool = False):
        shape = tuple(shape)
        for q in (self.rowwise_quantizer, self.columnwise_quantizer):
            q.internal = True
        self._resolved()
        kw = dict(dtype=dtype, device=device, pin_memory=pin_memory)
        row = self.rowwise_quantizer.make_empty(shape, **kw) if self.rowwise_usage else None
        col = self.columnwise_quantizer.make_empty(shape, **kw) if self.columnwise_usage else None
        return HybridQuantizedTensor(rowwise=row, columnwise=col, quantizer=self, shape=shape, dtype=dtype,
                                     requires_grad=requires_grad)

    def calibrate(self, tensor: torch.Tensor) -> None:
        self.rowwise_quantizer.calibrate(tensor)
        self.columnwise_quantizer.calibrate(tensor)

    def is_requantization_safe(self) -> bool:
        if self.rowwise_usage and not self.rowwise_quantizer.is_requantization_safe():
            return False
        if self.columnwise_usage and not self.columnwise_quantizer.is_requantization_safe():
            return False
        # a column-wise copy derived from the dequantized row-wise copy inherits the row-wise quantizer's determinism
        return not (self.columnwise_usage and self.columnwise_source == "rowwise_dequantized"
                    and not self.rowwise_quantizer.is_requantization_safe())

    # amax reduction over a process group is a property of the children that compute an amax (current scaling,
    # NVFP4); setting it here sets it on every child that has the notion
    @property
    def with_amax_reduction(self) -> bool:
        return any(getattr(q, "with_amax_reduction", False) for q in (self.rowwise_quantizer, self.columnwise_quantizer))

    @with_amax_reduction.setter
    def with_amax_reduction(self, value: bool) -> None:
        for q in (self.rowwise_quantizer, self.columnwise_quantizer):
            if hasattr(q, "with_amax_reduction"):
                q.with_amax_reduction = value

    @property
    def amax_reduction_group(self):
        for q in (self.rowwise_quantizer, self.columnwise_quantizer):
            if getattr(q, "amax_reduction_group", None) is not None:
                return q.amax_reduction_group
        return None

    @amax_reduction_group.setter
    def amax_reduction_group(self, group) -> None:
        for q in (self.rowwise_quantizer, self.columnwise_quantizer):
            if hasattr(q, "amax_reduction_group"):
                q.amax_reduction_group = group

    def supports_only_rowwise_all_gather(self) -> bool:
        return True
