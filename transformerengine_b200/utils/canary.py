"""Guard bands around kernel outputs: catches writes outside a tensor without a memory checker.

A guarded tensor is a view into a larger allocation whose bytes before and after the view hold a known
pattern; after the kernels under test have run, ``check()`` verifies the pattern.  The guard is sized in
bytes, so it also catches a kernel that treats a 1-byte tensor as wider elements.  Used by the GPU tests of
the kernels that compute their own addresses (quantizers with swizzled scale layouts, TMA-store epilogues,
strided RoPE): an out-of-range store that stays inside the caching allocator's block is silent otherwise.
(The reference relies on ``compute-sanitizer`` runs for this; there is no counterpart module.)
"""
from __future__ import annotations

import contextlib
from typing import List, Sequence, Tuple

import torch

_PATTERN = 0xA5


class GuardedAllocation:
    """Hands out tensors with guard bands and checks all of them at once."""

    def __init__(self, guard_bytes: int = 4096):
        assert guard_bytes % 256 == 0, "keep the payload 256-byte aligned"
        self.guard_bytes = guard_bytes
        self._allocs: List[Tuple[str, torch.Tensor, int]] = []   # (name, raw bytes, payload bytes)

    def empty(self, shape: Sequence[int], dtype: torch.dtype, device="cuda", name: str = "", fill=None) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        padded = (nbytes + 255) // 256 * 256
        raw = torch.full((self.guard_bytes + padded + self.guard_bytes,), _PATTERN, dtype=torch.uint8, device=device)
        self._allocs.append((name or f"tensor{len(self._allocs)}", raw, nbytes))
        view = raw[self.guard_bytes:self.guard_bytes + nbytes].view(dtype).reshape(tuple(shape))
        if fill is not None:
            view.fill_(fill)
        return view

    def empty_like(self, t: torch.Tensor, name: str = "") -> torch.Tensor:
        return self.empty(t.shape, t.dtype, t.device, name)

    def violations(self) -> List[str]:
        """Names (with the first bad offset) of the allocations whose guard bands were written."""
        bad = []
        for name, raw, nbytes in self._allocs:
            g = self.guard_bytes
            head = raw[:g]
            tail = raw[g + nbytes:]
            for side, band, base in (("before", head, -g), ("after", tail, nbytes)):
                wrong = (band != _PATTERN).nonzero()
                if wrong.numel():
                    bad.append(f"{name}: byte {base + int(wrong[0])} relative to the tensor ({side} it) was overwritten")
        return bad

    def check(self) -> None:
        bad = self.violations()
        if bad:
            raise AssertionError("out-of-bounds writes detected:\n  " + "\n  ".join(bad))

    @contextlib.contextmanager
    def intercept(self, device_type: str = "cuda"):
        """Inside the block ``torch.empty`` / ``torch.zeros`` calls for ``device_type`` return guarded tensors, so
        the outputs that the library's Python wrappers allocate for their kernels are covered without changing the
        wrappers.  Calls that name no device, or use layouts / pinning, pass through."""
        real_empty, real_zeros = torch.empty, torch.zeros

        def shape_of(args):
            if len(args) == 1 and isinstance(args[0], (tuple, list, torch.Size)):
                return tuple(int(v) for v in args[0])
            return tuple(int(v) for v in args)

        def make(real, fill):
            def fn(*args, **kw):
                dev = kw.get("device")
                simple = set(kw) <= {"dtype", "device"} and dev is not None and torch.device(dev).type == device_type
                if not simple or not all(isinstance(a, (int, tuple, list, torch.Size)) for a in args):
                    return real(*args, **kw)
                return self.empty(shape_of(args), kw.get("dtype") or torch.get_default_dtype(), dev,
                                  name=f"alloc{len(self._allocs)}{shape_of(args)}", fill=fill)
            return fn

        torch.empty, torch.zeros = make(real_empty, None), make(real_zeros, 0)
        try:
            yield self
        finally:
            torch.empty, torch.zeros = real_empty, real_zeros
