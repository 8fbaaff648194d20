"""One typed configuration object for the library's runtime switches.

Every switch has a field with a default, an environment variable that overrides it (read once, at first
use) and a docstring line.  Code asks ``get_config().fused_ep`` instead of calling ``os.environ.get`` at
the point of use; tests and applications change a switch for a region with ``override(fused_ep=False)``.
(The reference reads about eighty ``NVTE_*`` variables ad hoc across Python and C++; the recipe
dataclasses keep their own ``NVTE_*`` names for compatibility, see ``common/recipe.py``.)

The native kernels read three variables of their own at first launch (``TEB200_GEMM_2CTA``,
``TEB200_GEMM_BN``, ``TEB200_ATTN_GSPLIT``/``TEB200_ATTN_PAIR``); they are mirrored here so that
``describe()`` lists every switch in one place.
"""
from __future__ import annotations

import contextlib
import dataclasses
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, Optional


def _env_bool(v: str) -> bool:
    return v.strip().lower() in ("1", "true", "yes", "on")


@dataclass
class Config:
    # name of the environment variable and a help line live in the field metadata
    attention_backend: str = field(default="own", metadata=dict(
        env="TEB200_ATTN", help="'own': tcgen05 attention kernels of this library; 'library': torch SDPA for A/B "
                                "timing; 'reference': fp32 reference math everywhere (numerics debugging; also chosen "
                                "by NVTE_FUSED_ATTN=0 together with NVTE_FLASH_ATTN=0)"))
    fused_context_parallel: bool = field(default=True, metadata=dict(
        env="TEB200_FUSED_CP", help="attention kernels read peer K/V over NVLink instead of an NCCL ring"))
    fused_ep: bool = field(default=True, metadata=dict(
        env="TEB200_FUSED_EP", help="MoE dispatch/combine through the peer-memory kernels instead of NCCL all-to-all"))
    dp_overlap: bool = field(default=True, metadata=dict(
        env="TEB200_DP_OVERLAP", help="start data-parallel gradient reductions during the backward pass"))
    nvtx: bool = field(default=False, metadata=dict(env="TEB200_NVTX", help="emit NVTX ranges"))
    fused_mla_q_uproj: bool = field(default=True, metadata=dict(
        env="NVTE_FUSED_MLA_Q_UPROJ", help="use the composed-kernel latent-attention query projection"))
    allow_unsafe_pickle_extra_state: bool = field(default=False, metadata=dict(
        env="NVTE_ALLOW_UNSAFE_PICKLE_EXTRA_STATE", help="load _extra_state with the unrestricted unpickler"))
    wait_limit_cycles: int = field(default=0, metadata=dict(
        env="TEB200_WAIT_LIMIT_CYCLES", help="limit of host-launched flag waits in SM clock cycles (0: about one second)"))
    copy_ctas: int = field(default=0, metadata=dict(
        env="TEB200_COPY_CTAS", help="SMs that copy instead of computing in a fused collective GEMM (0: automatic)"))
    fused_qkv_rope: bool = field(default=True, metadata=dict(
        env="TEB200_FUSED_QKV_ROPE", help="rotate the query and key heads of a packed QKV projection with one launch"))
    debug: bool = field(default=False, metadata=dict(
        env="NVTE_DEBUG", help="log which attention path every configuration takes (logger 'DotProductAttention')"))
    debug_level: int = field(default=0, metadata=dict(
        env="NVTE_DEBUG_LEVEL", help="0: the chosen path; 1: also the conditions that ruled the others out; 2: every call"))
    fp8_dpa_bwd: bool = field(default=True, metadata=dict(
        env="NVTE_FP8_DPA_BWD", help="with recipe.fp8_dpa: also round the attention gradients to FP8 (0: 16-bit backward)"))
    # mirrored switches of the native kernels (read there at first launch)
    gemm_cta_pairs: bool = field(default=True, metadata=dict(
        env="TEB200_GEMM_2CTA", help="dense GEMMs on cta_group::2 pairs (0: single-CTA kernels)"))
    gemm_tile_n: int = field(default=0, metadata=dict(
        env="TEB200_GEMM_BN", help="force the single-CTA GEMM tile width (0: automatic)"))
    nvfp4_one_pass: bool = field(default=True, metadata=dict(
        env="TEB200_NVFP4_FUSED", help="NVFP4 row-wise and column-wise copies from one read of the input"))
    attention_group_split: bool = field(default=True, metadata=dict(
        env="TEB200_ATTN_GSPLIT", help="split dK/dV head groups over CTAs when few heads underfill the GPU"))

    @classmethod
    def from_env(cls, environ: Optional[Dict[str, str]] = None) -> "Config":
        environ = os.environ if environ is None else environ
        cfg = cls()
        for f in fields(cls):
            raw = environ.get(f.metadata["env"])
            if raw is None:
                continue
            if f.type in (bool, "bool"):
                val: Any = _env_bool(raw)
            elif f.type in (int, "int"):
                try:
                    val = int(raw)
                except ValueError:
                    raise ValueError(f"{f.metadata['env']}={raw!r} is not an integer") from None
            else:
                val = raw
            setattr(cfg, f.name, val)
        # the reference's switches: with both of its fused backends off only its unfused PyTorch path is left
        if environ.get("TEB200_ATTN") is None and environ.get("NVTE_FUSED_ATTN") == "0" \
                and environ.get("NVTE_FLASH_ATTN") == "0":
            cfg.attention_backend = "reference"
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.attention_backend not in ("own", "library", "reference"):
            raise ValueError(f"attention_backend must be 'own', 'library' or 'reference', got {self.attention_backend!r}")
        if self.gemm_tile_n not in (0, 128, 256):
            raise ValueError("gemm_tile_n must be 0, 128 or 256")
        if self.wait_limit_cycles < 0:
            raise ValueError("wait_limit_cycles must be >= 0")

    def describe(self) -> str:
        """One line per switch: field, environment variable, current value, meaning."""
        return "\n".join(f"{f.name:34s} {f.metadata['env']:38s} = {getattr(self, f.name)!r:10}  {f.metadata['help']}"
                         for f in fields(self))


_CONFIG: Optional[Config] = None


def get_config() -> Config:
    global _CONFIG
    if _CONFIG is None:
        _CONFIG = Config.from_env()
    return _CONFIG


def set_config(cfg: Config) -> None:
    global _CONFIG
    cfg.validate()
    _CONFIG = cfg


def reload_from_env() -> Config:
    """Read the environment again (tests that change ``os.environ``)."""
    global _CONFIG
    _CONFIG = Config.from_env()
    return _CONFIG


@contextlib.contextmanager
def override(**kw):
    """Change switches for the duration of a ``with`` block."""
    old = get_config()
    new = dataclasses.replace(old, **kw)
    set_config(new)
    try:
        yield new
    finally:
        set_config(old)
