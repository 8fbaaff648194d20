"""Small helpers that training frameworks import from the reference's ``pytorch/utils.py``: weight initialisers,
divisibility checks, tensor splitting, dtype / device canonicalisation, NVTX ranges.  Everything here is a few lines
of plain PyTorch; nothing depends on the extension."""
from __future__ import annotations

import contextlib
import math
import os
from typing import Callable, List, Optional, Sequence, Tuple, Union

import torch

# ------------------------------------------------------------------------------------------- initialisers


def init_method_constant(val: float) -> Callable:
    def init_(tensor: torch.Tensor) -> torch.Tensor:
        return torch.nn.init.constant_(tensor, val)
    return init_


def init_method_normal(sigma: float) -> Callable:
    """Normal(0, sigma) initialiser."""
    def init_(tensor: torch.Tensor) -> torch.Tensor:
        return torch.nn.init.normal_(tensor, mean=0.0, std=sigma)
    return init_


def scaled_init_method_normal(sigma: float, num_layers: int) -> Callable:
    """Normal(0, sigma / sqrt(2 * num_layers)): the output projections of a residual stack of ``num_layers`` blocks."""
    std = sigma / math.sqrt(2.0 * num_layers)

    def init_(tensor: torch.Tensor) -> torch.Tensor:
        return torch.nn.init.normal_(tensor, mean=0.0, std=std)
    return init_


def get_default_init_method() -> Callable:
    """Normal(0, 0.023), the library's default weight initialiser."""
    return init_method_normal(0.023)


# ------------------------------------------------------------------------------------------- arithmetic
def ensure_divisibility(numerator: int, denominator: int) -> None:
    if numerator % denominator != 0:
        raise ValueError(f"{numerator} is not divisible by {denominator}")


def divide(numerator: int, denominator: int) -> int:
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def round_up_to_nearest_multiple(value: int, multiple: int) -> int:
    if multiple == 0:
        raise ValueError("multiple cannot be zero")
    return ceil_div(value, multiple) * multiple


# ------------------------------------------------------------------------------------------- tensors
def requires_grad(*tensors: Optional[torch.Tensor]) -> bool:
    return any(t is not None and t.requires_grad for t in tensors)


def clear_tensor_data(*tensors: Optional[torch.Tensor]) -> None:
    """Free the memory of tensors that are no longer needed although references to them remain (saved activations
    after their last use): plain tensors get an empty storage, quantized tensors drop their payload."""
    for t in tensors:
        if t is None:
            continue
        if hasattr(t, "clear") and hasattr(t, "get_data_tensors"):
            t.clear()
        elif isinstance(t, torch.Tensor):
            t.data = torch.empty(0, dtype=t.dtype, device=t.device)


def cast_if_needed(tensor: Optional[torch.Tensor], dtype: torch.dtype) -> Optional[torch.Tensor]:
    if tensor is None or tensor.dtype == dtype:
        return tensor
    return tensor.to(dtype)


def split_tensor_along_dim(tensor: torch.Tensor, dim: int, num_partitions: int,
                           contiguous_split_chunks: bool = False) -> Tuple[torch.Tensor, ...]:
    size = divide(tensor.size(dim), num_partitions)
    parts = torch.split(tensor, size, dim=dim)
    return tuple(p.contiguous() for p in parts) if contiguous_split_chunks else parts


def combine_tensors(tensors: Sequence[torch.Tensor], dim: int) -> torch.Tensor:
    """Stack tensors along a NEW dimension ``dim`` (the inverse of ``SplitAlongDim`` with ``squeeze=True``)."""
    return torch.stack(list(tensors), dim=dim)


class SplitAlongDim(torch.autograd.Function):
    """``torch.split`` whose backward writes the pieces' gradients into one buffer (no concatenation when the
    incoming gradients already are adjacent views of one tensor)."""

    @staticmethod
    def forward(ctx, mixed: torch.Tensor, split_dim: int, split_size_or_sections, squeeze: bool = False):  # type: ignore[override]
        ctx.split_dim, ctx.sizes, ctx.squeeze = split_dim, split_size_or_sections, squeeze
        parts = torch.split(mixed, split_size_or_sections, dim=split_dim)
        if squeeze:
            parts = tuple(p.squeeze(split_dim) for p in parts)
        return parts

    @staticmethod
    def backward(ctx, *grads):  # type: ignore[override]
        if ctx.squeeze:
            grads = tuple(g.unsqueeze(ctx.split_dim) for g in grads)
        return torch.cat(grads, dim=ctx.split_dim), None, None, None


def attention_mask_func(attention_scores: torch.Tensor, attention_mask: torch.Tensor) -> torch.Tensor:
    """Put a large negative number where the boolean mask is True."""
    return attention_scores.masked_fill(attention_mask, -10000.0)


def assert_viewless_tensor(tensor, extra_msg: Optional[str] = None):
    """Tensors that are views keep their base alive; code that swaps ``.data`` needs tensors that own their memory."""
    if isinstance(tensor, (list, tuple)):
        return type(tensor)(assert_viewless_tensor(t, extra_msg) for t in tensor)
    if isinstance(tensor, torch.Tensor) and tensor._base is not None:
        raise AssertionError("the tensor is a view of another tensor" + (f": {extra_msg}" if extra_msg else ""))
    return tensor


def safely_set_viewless_tensor_data(tensor: torch.Tensor, new_data_tensor: torch.Tensor) -> None:
    assert_viewless_tensor(tensor, f"cannot set .data of a view (shape {tuple(tensor.shape)})")
    tensor.data = new_data_tensor


_ONES: dict = {}


def get_cached_ones_tensor(num_elements: int, dtype: torch.dtype, device) -> torch.Tensor:
    """A tensor of ones kept alive by a cache, so that its address is stable across CUDA-graph replays."""
    key = (int(num_elements), dtype, str(device))
    t = _ONES.get(key)
    if t is None:
        t = _ONES[key] = torch.ones(num_elements, dtype=dtype, device=device)
    return t


def all_close(a: torch.Tensor, b: torch.Tensor) -> bool:
    return bool(torch.all(torch.isclose(a, b)))


def print_rank_0(*args) -> None:
    if not torch.distributed.is_available() or not torch.distributed.is_initialized() \
            or torch.distributed.get_rank() == 0:
        print(*args)


def compare_tensors(a: torch.Tensor, b: torch.Tensor) -> None:
    """Print the largest difference between two tensors (debugging aid)."""
    if a.shape != b.shape:
        print_rank_0("Tensors have different shape")
        return
    print_rank_0(f"max err={float((a.float() - b.float()).abs().max())}, max a={float(a.max())}, max b={float(b.max())}")


# ------------------------------------------------------------------------------------------- checks
def check_dim_for_fp8_exec(tensor: torch.Tensor) -> bool:
    """Whether a matrix can be an operand of the FP8 GEMMs: 2-D, rows a multiple of 8, columns of 16."""
    return tensor.dim() == 2 and tensor.size(0) % 8 == 0 and tensor.size(1) % 16 == 0


def assert_dim_for_fp8_exec(*tensors: torch.Tensor) -> None:
    for t in tensors:
        rows = math.prod(t.shape[:-1])
        if rows % 8 != 0 or t.shape[-1] % 16 != 0:
            raise ValueError("FP8 execution requires the product of all dimensions except the last to be divisible by "
                             f"8 and the last dimension by 16, got dims={list(t.shape)}")


def needs_quantized_gemm(obj, rowwise: bool = True) -> bool:
    """Whether ``obj`` is a quantized tensor (a plain tensor / parameter goes to the 16-bit GEMM)."""
    return type(obj) not in (torch.Tensor, torch.nn.Parameter)


def validate_ctx_manager(ctx: Callable) -> None:
    try:
        with ctx():
            pass
    except Exception as e:  # noqa: BLE001
        raise ValueError("Object must be a valid ctx manager") from e


def validate_rng_states_func(get_rng_tracker: Callable) -> None:
    """The tracker a module is given must offer ``get_states``, ``set_states`` and a ``fork`` context manager."""
    if not callable(get_rng_tracker):
        raise TypeError(f"get_rng_tracker must be callable, got {type(get_rng_tracker).__name__}")
    try:
        tracker = get_rng_tracker()
    except Exception as e:  # noqa: BLE001
        raise RuntimeError("Cannot call get_rng_tracker function") from e
    for name in ("get_states", "set_states", "fork"):
        if not callable(getattr(tracker, name, None)):
            raise TypeError(f"rng tracker ({type(tracker).__name__}) lacks a callable '{name}'")


# ------------------------------------------------------------------------------------------- device / dtype
def is_bf16_compatible() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] >= 8


def is_non_tn_fp8_gemm_supported() -> bool:
    """Whether FP8 GEMMs take operands in layouts other than TN.  The tcgen05 kernels of this library read both
    operands K-major and keep a transposed copy where a layout needs one, so callers never depend on this."""
    if not torch.cuda.is_available():
        return False
    cap = torch.cuda.get_device_capability()
    return (10, 0) <= cap < (12, 0) or cap >= (13, 0)


def get_sm_count() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


def canonicalize_device(device: Optional[Union[torch.device, str]]) -> torch.device:
    if device is None:
        device = torch.get_default_device() if hasattr(torch, "get_default_device") else torch.device("cpu")
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def canonicalize_dtype(dtype: Optional[torch.dtype]) -> torch.dtype:
    return torch.get_default_dtype() if dtype is None else dtype


def devices_match(device1: torch.device, device2: torch.device) -> bool:
    d1, d2 = torch.device(device1), torch.device(device2)
    if d1.type != d2.type:
        return False
    if d1.type == "cuda":
        i1 = torch.cuda.current_device() if d1.index is None else d1.index
        i2 = torch.cuda.current_device() if d2.index is None else d2.index
        return i1 == i2
    return d1 == d2


def canonicalize_process_group(group):
    """``None`` means the default process group."""
    if group is None:
        return torch.distributed.distributed_c10d._get_default_group()
    return group


def torch_get_autocast_gpu_dtype() -> torch.dtype:
    return torch.get_autocast_dtype("cuda") if hasattr(torch, "get_autocast_dtype") else torch.get_autocast_gpu_dtype()


# ------------------------------------------------------------------------------------------- NVTX
def _nvtx_enabled() -> bool:
    return os.getenv("NVTE_NVTX_ENABLED", "0") == "1" and torch.cuda.is_available()


_NVTX_STACK: List[str] = []


def nvtx_range_push(msg: str) -> None:
    """Open a named range in profiler timelines (only with ``NVTE_NVTX_ENABLED=1`` and a GPU)."""
    if _nvtx_enabled():
        _NVTX_STACK.append(msg)
        torch.cuda.nvtx.range_push(msg)


def nvtx_range_pop(msg: Optional[str] = None) -> None:
    if not _nvtx_enabled():
        return
    if not _NVTX_STACK:
        raise RuntimeError("nvtx_range_pop without a matching push")
    last = _NVTX_STACK.pop()
    if msg is not None and msg != last:
        raise ValueError(f"closing NVTX range {msg!r} but the innermost open one is {last!r}")
    torch.cuda.nvtx.range_pop()


@contextlib.contextmanager
def get_nvtx_range_context(msg: str):
    nvtx_range_push(msg)
    try:
        yield
    finally:
        nvtx_range_pop(msg)


__all__ = [n for n in dir() if not n.startswith("_") and n not in (
    "annotations", "contextlib", "math", "os", "torch", "Callable", "List", "Optional", "Sequence", "Tuple", "Union")]
