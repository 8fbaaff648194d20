"""Quantizer / quantized-tensor base classes.

A :class:`Quantizer` is a builder that turns a high-precision tensor into a
quantized one.  A quantized tensor carries up to two physical copies of the
logical matrix: a *rowwise* copy (scales along the last dim, used when the
tensor is contracted over its last dim) and a *columnwise* copy (scales along
the flattened leading dims, used when the tensor is contracted over those).
In this library every columnwise copy is stored transposed ``[C, R]`` so that
all GEMM operands are contraction-dim contiguous for the tcgen05 kernels.

``*Storage`` classes are plain containers without autograd; the ``*Tensor``
classes wrap them as ``torch.Tensor`` subclasses so that quantized parameters
behave like tensors (reference: ``pytorch/quantized_tensor.py:53-1083``).
"""
from __future__ import annotations

import abc
import copy
from typing import Any, Dict, Iterable, Optional, Tuple

import torch
from torch.utils._pytree import tree_map


class QuantizedTensorStorage:
    """Container of quantized data.  Sub-classes define the fields."""

    _quantizer: Optional["Quantizer"] = None
    _dtype: torch.dtype = torch.float32
    _shape: Tuple[int, ...] = ()

    # -- interface ----------------------------------------------------------
    def dequantize(self, *, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        raise NotImplementedError

    def update_usage(self, rowwise_usage: Optional[bool] = None, columnwise_usage: Optional[bool] = None) -> None:
        """Drop the copy that is no longer needed (frees memory)."""
        raise NotImplementedError

    def get_usages(self) -> Dict[str, bool]:
        raise NotImplementedError

    def get_data_tensors(self) -> Tuple[Optional[torch.Tensor], ...]:
        raise NotImplementedError

    def prepare_for_saving(self):
        """Return (tensors, self) with the tensor fields detached from ``self``,
        for ``ctx.save_for_backward``."""
        raise NotImplementedError

    def restore_from_saved(self, tensors: list) -> list:
        raise NotImplementedError

    @property
    def logical_shape(self) -> Tuple[int, ...]:
        return tuple(self._shape)

    @property
    def device(self):  # type: ignore[override]
        for t in self.get_data_tensors():
            if t is not None:
                return t.device
        raise RuntimeError("quantized tensor holds no data")

    def size(self, dim: Optional[int] = None):
        return torch.Size(self._shape) if dim is None else self._shape[dim]

    def numel(self) -> int:
        n = 1
        for s in self._shape:
            n *= s
        return n

    def _rows_cols(self) -> Tuple[int, int]:
        c = self._shape[-1]
        return self.numel() // max(c, 1), c

    # -- conveniences shared by all formats (reference: quantized_tensor.py, QuantizedTensorStorage) -------------
    def update_quantizer(self, quantizer: "Quantizer") -> None:
        """Bind another quantizer (of the same kind) to this tensor: later in-place updates use it."""
        if self._quantizer is not None and type(quantizer) is not type(self._quantizer):
            raise TypeError(f"cannot replace a {type(self._quantizer).__name__} by a {type(quantizer).__name__}")
        self._quantizer = quantizer

    def copy_from_storage(self, src: "QuantizedTensorStorage") -> None:
        """Copy the payload of ``src`` (same class, shape and set of copies) into this object's buffers."""
        if type(src) is not type(self) and not (isinstance(src, type(self)) or isinstance(self, type(src))):
            raise TypeError(f"cannot copy a {type(src).__name__} into a {type(self).__name__}")
        if tuple(src._shape) != tuple(self._shape):
            raise ValueError(f"shape mismatch: {tuple(src._shape)} vs {tuple(self._shape)}")
        for name, val in vars(src).items():
            mine = getattr(self, name, None)
            if isinstance(val, torch.Tensor) and name.startswith("_") and name not in ("_quantizer",):
                if isinstance(mine, torch.Tensor) and mine.shape == val.shape:
                    mine.copy_(val)
                elif mine is None:
                    raise ValueError(f"the destination lacks the buffer {name}")
            elif isinstance(mine, torch.Tensor) and val is None and name.startswith("_"):
                raise ValueError(f"the source lacks the buffer {name}")

    def clear(self) -> None:
        """Release the payload (the object stays, its buffers become empty tensors)."""
        for name, val in list(vars(self).items()):
            if isinstance(val, QuantizedTensorStorage):
                val.clear()                      # per-direction children of a hybrid tensor
            elif isinstance(val, torch.Tensor) and name.startswith("_"):
                setattr(self, name, torch.empty(0, dtype=val.dtype, device=val.device))


class Quantizer(abc.ABC):
    """Builder of quantized tensors.

    ``rowwise_usage`` / ``columnwise_usage`` select which copies are produced;
    ``internal=True`` produces a bare Storage object (cheaper, no autograd).
    """

    def __init__(self, *, rowwise: bool = True, columnwise: bool = True) -> None:
        self.rowwise_usage = rowwise
        self.columnwise_usage = columnwise
        self.internal = False
        self.optimize_for_gemm = True

    def set_usage(self, *, rowwise: Optional[bool] = None, columnwise: Optional[bool] = None) -> None:
        if rowwise is not None:
            self.rowwise_usage = rowwise
        if columnwise is not None:
            self.columnwise_usage = columnwise

    def copy(self) -> "Quantizer":
        return copy.copy(self)

    def __call__(self, tensor: torch.Tensor) -> Any:
        return self.quantize(tensor)

    def quantize(self, tensor: torch.Tensor, *, out: Optional[QuantizedTensorStorage] = None, dtype=None):
        if out is not None:
            return self.update_quantized(tensor, out)
        if isinstance(tensor, QuantizedTensorStorage):
            tensor = tensor.dequantize()
        return self.quantize_impl(tensor.detach() if self.internal else tensor, dtype=dtype)

    @abc.abstractmethod
    def quantize_impl(self, tensor: torch.Tensor, dtype=None):
        ...

    @abc.abstractmethod
    def update_quantized(self, src: torch.Tensor, dst: QuantizedTensorStorage, *, noop_flag=None):
        ...

    @abc.abstractmethod
    def make_empty(self, shape: Iterable[int], *, dtype=torch.float32, device=None, requires_grad=False,
                   pin_memory: bool = False):
        ...

    def calibrate(self, tensor: torch.Tensor) -> None:
        """Record statistics without quantizing (``autocast(calibrating=True)``)."""

    def is_quantizable(self, inp: torch.Tensor) -> bool:
        """Whether ``inp`` can be quantized by this quantizer as it is (shape constraints of the format)."""
        return True

    def is_requantization_safe(self) -> bool:
        """Whether quantizing the same input again reproduces the same payload (False for quantizers with state
        that moves, such as delayed scaling, or with random rounding): callers may then drop a quantized value and
        rebuild it later."""
        return False

    def multi_quantize(self, tensors) -> list:
        """Quantize a list of tensors with this quantizer's settings."""
        return [self.quantize(t) for t in tensors]

    def get_columnwise_shape(self, shape: Iterable[int]) -> Tuple[int, ...]:
        """Shape of the column-wise copy of a tensor of ``shape``: stored transposed, ``[last dim, product of the
        leading dims]``."""
        shape = tuple(shape)
        if not shape:
            return ()
        rows = 1
        for d in shape[:-1]:
            rows *= d
        return (shape[-1], rows)

    def supports_only_rowwise_all_gather(self) -> bool:
        return False

    def get_usages(self) -> Dict[str, bool]:
        return {"rowwise": self.rowwise_usage, "columnwise": self.columnwise_usage}


def pin_payload(obj):
    """Move the payload tensors of a quantized tensor on the host into page-locked memory (``make_empty(...,
    pin_memory=True)``: staging buffers of asynchronous host <-> device copies)."""
    for name, val in list(vars(obj).items()):
        if isinstance(val, torch.Tensor) and name.startswith("_") and val.device.type == "cpu" and not val.is_pinned():
            setattr(obj, name, val.pin_memory())
        elif isinstance(val, QuantizedTensorStorage):
            pin_payload(val)
    return obj


def _stride_for(shape) -> Tuple[int, ...]:
    st, acc = [], 1
    for s in reversed(tuple(shape)):
        st.append(acc)
        acc *= max(int(s), 1)
    return tuple(reversed(st))


class _QuantizeFunc(torch.autograd.Function):
    """Differentiable quantize: straight-through gradient."""

    @staticmethod
    def forward(ctx, tensor, quantizer):  # type: ignore[override]
        return quantizer.quantize_impl(tensor.detach())

    @staticmethod
    def backward(ctx, grad):  # type: ignore[override]
        return grad, None


class _DequantizeFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, dtype):  # type: ignore[override]
        return tensor._dequantize_impl(dtype)

    @staticmethod
    def backward(ctx, grad):  # type: ignore[override]
        return grad, None


class QuantizedTensor(torch.Tensor):
    """``torch.Tensor`` wrapper over a quantized payload.

    Generic torch ops see the dequantized values (``__torch_dispatch__``);
    in-place ops re-quantize into the payload.  Library kernels read the
    payload fields directly.
    """

    @staticmethod
    def __new__(cls, *args, shape, dtype, requires_grad=False, device=None, **kwargs):
        shape = tuple(int(s) for s in shape)
        return torch.Tensor._make_wrapper_subclass(
            cls,
            shape,
            strides=_stride_for(shape),
            storage_offset=0,
            dtype=dtype,
            layout=torch.strided,
            requires_grad=requires_grad,
            device=torch.device("cpu") if device is None else device,
        )

    # sub-classes implement
    def _dequantize_impl(self, dtype: Optional[torch.dtype]) -> torch.Tensor:
        raise NotImplementedError

    def _new_like(self, **overrides):
        raise NotImplementedError

    def quantize_(self, tensor: torch.Tensor, *, noop_flag=None) -> "QuantizedTensor":
        """Overwrite the payload with a quantization of ``tensor``."""
        q = self._quantizer
        assert q is not None, "in-place update needs the quantizer that built this tensor"
        if isinstance(tensor, QuantizedTensor):
            tensor = tensor.dequantize()
        q.update_quantized(tensor, self, noop_flag=noop_flag)
        return self

    def dequantize(self, *, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        if torch.is_grad_enabled() and self.requires_grad:
            return _DequantizeFunc.apply(self, dtype)
        return self._dequantize_impl(dtype)

    def detach(self):  # type: ignore[override]
        return self._new_like(requires_grad=False)

    def clone(self, *a, **k):  # type: ignore[override]
        return self._new_like(clone=True)

    def float(self):  # type: ignore[override]
        return self.dequantize(dtype=torch.float32)

    def bfloat16(self):  # type: ignore[override]
        return self.dequantize(dtype=torch.bfloat16)

    def half(self):  # type: ignore[override]
        return self.dequantize(dtype=torch.float16)

    def cpu(self, *a, **k):  # type: ignore[override]
        return self.dequantize().cpu()

    def __repr__(self, *, tensor_contents=None):  # type: ignore[override]
        return f"{self.__class__.__name__}(shape={tuple(self.shape)}, dtype={self.dtype}, data={self.dequantize()})"

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func in (torch.ops.aten.detach.default, torch.ops.aten.alias.default):
            return args[0]._new_like(requires_grad=False)
        if func == torch.ops.aten.clone.default:
            return args[0]._new_like(clone=True)
        if func == torch.ops.aten.copy_.default:
            dst, src = args[0], args[1]
            if isinstance(dst, QuantizedTensor):
                dst.quantize_(src.dequantize() if isinstance(src, QuantizedTensor) else src)
                return dst
            dst.copy_(src.dequantize(dtype=dst.dtype))
            return dst
        if func == torch.ops.aten.view.default and tuple(args[1]) == tuple(args[0].shape):
            return args[0]._new_like(requires_grad=False)

        def unwrap(t):
            return t._dequantize_impl(None) if isinstance(t, QuantizedTensor) else t

        # in-place ops on a quantized destination: compute in high precision, requantize
        schema = getattr(func, "_schema", None)
        if schema is not None and schema.is_mutable and len(args) and isinstance(args[0], QuantizedTensor):
            dst = args[0]
            hp = dst._dequantize_impl(None)
            rest = tree_map(unwrap, args[1:])
            func(hp, *rest, **tree_map(unwrap, kwargs))
            dst.quantize_(hp)
            return dst
        return func(*tree_map(unwrap, args), **tree_map(unwrap, kwargs))

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    # parameters of quantized type must survive .data assignment and state_dict
    def contiguous(self, memory_format=torch.contiguous_format):  # type: ignore[override]
        return self

    def to_dtype(self, dtype: torch.dtype):
        return self._new_like(dtype=dtype)

    def get_metadata(self) -> Dict[str, Any]:
        """Everything but shape / dtype / requires_grad that ``type(self)(...)`` needs to rebuild this tensor: the
        payload tensors and the format fields, by constructor keyword."""
        import inspect

        out: Dict[str, Any] = {}
        params = inspect.signature(type(self).__new__).parameters
        alias = {"fp8_scale_inv": "_scale_inv", "data_transpose": "_transpose"}
        for name in params:
            if name in ("cls", "shape", "dtype", "requires_grad", "device"):
                continue
            attr = alias.get(name, "_" + name)
            if hasattr(self, attr):
                out[name] = getattr(self, attr)
        return out

    @classmethod
    def make_like(cls, tensor: "QuantizedTensor", *, shape=None, dtype=None,
                  requires_grad: bool = False) -> "QuantizedTensor":
        """A tensor that shares ``tensor``'s payload and quantizer under another logical dtype / requires_grad
        (``shape`` must describe the same number of elements)."""
        if shape is not None and tuple(shape) != tuple(tensor._shape):
            raise ValueError(f"make_like keeps the payload, whose shape is {tuple(tensor._shape)}; reshape the source "
                             f"to {tuple(shape)} first")
        return tensor._new_like(requires_grad=requires_grad, dtype=dtype)


def prepare_for_saving(*tensors):
    """Split a mix of plain and quantized tensors into (saveable tensors, objects)."""
    flat, objs = [], []
    for t in tensors:
        if t is None or isinstance(t, torch.Tensor) and not isinstance(t, QuantizedTensorStorage):
            flat.append(t)
            objs.append(None)
        else:
            ts, obj = t.prepare_for_saving()
            flat.extend(ts)
            objs.append(obj)
    return flat, objs


def restore_from_saved(objs, saved):
    saved = list(saved)
    out = []
    for o in objs:
        if o is None:
            out.append(saved.pop(0))
        else:
            saved = o.restore_from_saved(saved)
            out.append(o)
    return out


def restore_from_func_ctx(ctx, return_saved_tensors: bool = False):
    """Rebuild the tensors that ``prepare_for_saving`` split, from an autograd context that kept the objects in
    ``ctx.tensor_objects`` and the raw tensors in ``ctx.saved_tensors``; the objects are dropped from the context."""
    if getattr(ctx, "tensor_objects", None) is None:
        raise AttributeError("ctx must have .tensor_objects to restore saved tensors")
    saved = list(ctx.saved_tensors)
    out = restore_from_saved(ctx.tensor_objects, list(saved))
    ctx.tensor_objects = None
    return (out, saved) if return_saved_tensors else out
