"""Grouped tensor: a collection of 2-D tensors (experts' weights, per-expert token blocks) that live
in one packed buffer and are described by per-member shapes, so that grouped GEMMs and grouped
quantization take one object instead of a Python list.

High-precision members are views of one flat buffer.  Quantized members are built by the group's
quantizer; their payloads are kept per member (every format of this library stores block scales in
the GEMM tile layout, which is defined per matrix), while ``rowwise_data`` still exposes the packed
bytes for checkpointing.
(Reference: ``pytorch/tensor/storage/grouped_tensor_storage.py:24,444,629,947,1306``,
``pytorch/tensor/grouped_tensor.py:68``.)
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .base import QuantizedTensorStorage, Quantizer


class GroupedTensorStorage:
    """``num_tensors`` members of shapes ``(first_dims[i], last_dims[i])``; ``None`` dims mean uniform."""

    def __init__(self, *, num_tensors: int, shapes: Sequence[Tuple[int, int]], quantizer: Optional[Quantizer],
                 dtype: torch.dtype, device, logical_shape: Tuple[int, int], first_dims=None, last_dims=None):
        self.num_tensors = num_tensors
        self.tensor_shapes: List[Tuple[int, int]] = [tuple(int(x) for x in s) for s in shapes]
        self.quantizer = quantizer
        self.fake_dtype = dtype
        self.logical_shape = tuple(logical_shape)
        self.first_dims, self.last_dims = first_dims, last_dims
        sizes = [a * b for a, b in self.tensor_shapes]
        offs = [0]
        for n in sizes:
            offs.append(offs[-1] + n)
        self.tensor_offsets = torch.tensor(offs, dtype=torch.int64, device=device)
        self._offsets_host = offs
        self.data: Optional[torch.Tensor] = None          # packed high-precision values (no quantizer)
        self.members: List = []                            # per-member tensors (views or quantized)
        if quantizer is None:
            self.data = torch.empty(offs[-1], dtype=dtype, device=device)
            self.members = [self.data[offs[i]:offs[i + 1]].view(*self.tensor_shapes[i]) for i in range(num_tensors)]
        else:
            from .hybrid import HybridQuantizer, IdentityQuantizer

            if isinstance(quantizer, (HybridQuantizer, IdentityQuantizer)):
                raise NotImplementedError("grouped storage of identity / hybrid members is not supported; "
                                          "keep separate tensors (GroupedLinear(single_grouped_weight=False))")
            self.members = [quantizer.make_empty(s, dtype=dtype, device=device) for s in self.tensor_shapes]

    # ---- factories
    @staticmethod
    def make_grouped_tensor_with_shapes(num_tensors: int, shapes: Sequence[Tuple[int, int]],
                                        quantizer: Optional[Quantizer] = None, device=None,
                                        dtype: Optional[torch.dtype] = None, cls=None) -> "GroupedTensorStorage":
        assert len(shapes) == num_tensors
        f, l = [s[0] for s in shapes], [s[1] for s in shapes]
        uf, ul = len(set(f)) <= 1, len(set(l)) <= 1
        first = None if uf else torch.tensor(f, dtype=torch.int64, device=device)
        last = None if ul else torch.tensor(l, dtype=torch.int64, device=device)
        if not uf and not ul:
            logical = (1, sum(a * b for a, b in shapes))
        else:
            logical = (f[0] if (uf and not ul) else sum(f), l[0] if ul else sum(l))
        return (cls or GroupedTensorStorage)(num_tensors=num_tensors, shapes=shapes, quantizer=quantizer,
                                             dtype=dtype or torch.float32, device=device, logical_shape=logical,
                                             first_dims=first, last_dims=last)

    @staticmethod
    def make_grouped_tensor(num_tensors: int, first_dims: Optional[torch.Tensor], last_dims: Optional[torch.Tensor],
                            logical_first_dim: int, logical_last_dim: int, quantizer: Optional[Quantizer] = None,
                            device=None, dtype: Optional[torch.dtype] = None, cls=None) -> "GroupedTensorStorage":
        f = first_dims.tolist() if first_dims is not None else None
        l = last_dims.tolist() if last_dims is not None else None
        if f is None and l is None:
            assert logical_first_dim % num_tensors == 0
            shapes = [(logical_first_dim // num_tensors, logical_last_dim)] * num_tensors
        elif l is None:
            shapes = [(a, logical_last_dim) for a in f]
        elif f is None:
            shapes = [(logical_first_dim, b) for b in l]
        else:
            shapes = list(zip(f, l))
        return (cls or GroupedTensorStorage)(num_tensors=num_tensors, shapes=shapes, quantizer=quantizer,
                                             dtype=dtype or torch.float32, device=device,
                                             logical_shape=(logical_first_dim, logical_last_dim),
                                             first_dims=first_dims, last_dims=last_dims)

    @staticmethod
    def make_grouped_tensor_from_rowwise_data(*, num_tensors: int, tensor_shape: Tuple[int, ...],
                                              rowwise_data: torch.Tensor, dtype: Optional[torch.dtype] = None,
                                              cls=None) -> "GroupedTensorStorage":
        """Wrap existing packed values (no allocation, no copy)."""
        rows = 1
        for s in tensor_shape[:-1]:
            rows *= s
        shapes = [(rows, tensor_shape[-1])] * num_tensors
        g = (cls or GroupedTensorStorage).__new__(cls or GroupedTensorStorage)
        GroupedTensorStorage.__init__(g, num_tensors=0, shapes=[], quantizer=None, dtype=dtype or rowwise_data.dtype,
                                      device=rowwise_data.device, logical_shape=(rows * num_tensors, tensor_shape[-1]))
        g.num_tensors, g.tensor_shapes = num_tensors, shapes
        n = rows * tensor_shape[-1]
        g._offsets_host = [i * n for i in range(num_tensors + 1)]
        g.tensor_offsets = torch.tensor(g._offsets_host, dtype=torch.int64, device=rowwise_data.device)
        g.data = rowwise_data.reshape(-1)
        g.members = [g.data[i * n:(i + 1) * n].view(rows, tensor_shape[-1]) for i in range(num_tensors)]
        return g

    # ---- shape queries
    def all_same_first_dim(self) -> bool:
        return len({s[0] for s in self.tensor_shapes}) <= 1

    def all_same_last_dim(self) -> bool:
        return len({s[1] for s in self.tensor_shapes}) <= 1

    def all_same_shape(self) -> bool:
        return self.all_same_first_dim() and self.all_same_last_dim()

    def varying_both_dims(self) -> bool:
        return not self.all_same_first_dim() and not self.all_same_last_dim()

    def get_common_first_dim(self) -> int:
        assert self.all_same_first_dim(), "members differ in their first dim"
        return self.tensor_shapes[0][0]

    def get_common_last_dim(self) -> int:
        assert self.all_same_last_dim(), "members differ in their last dim"
        return self.tensor_shapes[0][1]

    def get_dtype(self) -> torch.dtype:
        return self.fake_dtype

    def has_data(self) -> bool:
        if self.quantizer is None:
            return self.data is not None
        return all(m.get_usages().get("rowwise", False) for m in self.members)

    def has_columnwise_data(self) -> bool:
        return self.quantizer is not None and all(m.get_usages().get("columnwise", False) for m in self.members)

    @property
    def rowwise_data(self) -> Optional[torch.Tensor]:
        """Packed payload: the flat buffer, or the members' rowwise bytes concatenated."""
        if self.quantizer is None:
            return self.data
        parts = [m.get_data_tensors()[0] for m in self.members]
        if any(p is None for p in parts):
            return None
        return torch.cat([p.reshape(-1).view(torch.uint8) for p in parts])

    # ---- members
    def split_into_quantized_tensors(self) -> List:
        """The members, as views of the packed buffer (high precision) or quantized tensors."""
        return list(self.members)

    def quantize(self, tensors: Sequence[torch.Tensor], noop_flag: Optional[torch.Tensor] = None) -> List:
        """(Re)fill the group from high-precision tensors, one per member."""
        assert len(tensors) == self.num_tensors
        for i, t in enumerate(tensors):
            assert tuple(t.reshape(-1, t.shape[-1]).shape) == self.tensor_shapes[i], "member shape mismatch"
            if self.quantizer is None:
                self.members[i].copy_(t.reshape(self.tensor_shapes[i]))
            else:
                self.quantizer.update_quantized(t.reshape(self.tensor_shapes[i]), self.members[i], noop_flag=noop_flag)
        return self.split_into_quantized_tensors()

    def dequantize(self, *, dtype: Optional[torch.dtype] = None) -> List[torch.Tensor]:
        dt = dtype or self.fake_dtype
        return [m.dequantize(dtype=dt) if isinstance(m, QuantizedTensorStorage) else m.to(dt) for m in self.members]

    def get_data_tensors(self):
        if self.quantizer is None:
            return (self.data,)
        out = ()
        for m in self.members:
            out += tuple(m.get_data_tensors())
        return out

    def prepare_for_saving(self):
        if self.quantizer is None:
            t, self.data = [self.data], None
            self.members = []
            return t, self
        tensors, self._saved_counts = [], []
        for m in self.members:
            ts, _ = m.prepare_for_saving()
            tensors.extend(ts)
            self._saved_counts.append(len(ts))
        return tensors, self

    def restore_from_saved(self, tensors: list) -> list:
        if self.quantizer is None:
            self.data = tensors[0]
            o = self._offsets_host
            self.members = [self.data[o[i]:o[i + 1]].view(*self.tensor_shapes[i]) for i in range(self.num_tensors)]
            return list(tensors[1:])
        for m, n in zip(self.members, self._saved_counts):
            m.restore_from_saved(list(tensors[:n]))
            tensors = tensors[n:]
        return list(tensors)

    def clear(self) -> None:
        self.data, self.members = None, []

    def copy(self) -> "GroupedTensorStorage":
        g = GroupedTensorStorage.__new__(type(self))
        g.__dict__.update(self.__dict__)
        g.members = list(self.members)
        return g

    def __repr__(self) -> str:
        return (f"{type(self).__name__}(num_tensors={self.num_tensors}, shapes={self.tensor_shapes}, "
                f"logical_shape={self.logical_shape}, quantizer={type(self.quantizer).__name__}, dtype={self.fake_dtype})")


class GroupedTensor(GroupedTensorStorage):
    """Grouped tensor that also acts as ONE parameter-like object: ``stacked()`` gives the members as
    a single ``[num_tensors, rows, cols]`` tensor when their shapes agree (what a module registers
    when it keeps all experts' weights in one parameter)."""

    @staticmethod
    def make_grouped_tensor_with_shapes(*a, **k):  # type: ignore[override]
        return GroupedTensorStorage.make_grouped_tensor_with_shapes(*a, cls=GroupedTensor, **k)

    @staticmethod
    def make_grouped_tensor(*a, **k):  # type: ignore[override]
        return GroupedTensorStorage.make_grouped_tensor(*a, cls=GroupedTensor, **k)

    @staticmethod
    def make_grouped_tensor_from_rowwise_data(**k):  # type: ignore[override]
        return GroupedTensorStorage.make_grouped_tensor_from_rowwise_data(cls=GroupedTensor, **k)

    def stacked(self, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        assert self.all_same_shape(), "stacking needs members of one shape"
        if self.quantizer is None:
            r, c = self.tensor_shapes[0]
            t = self.data.view(self.num_tensors, r, c)
            return t if dtype is None else t.to(dtype)
        return torch.stack(self.dequantize(dtype=dtype))
