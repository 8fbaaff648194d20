"""Run code written against ``transformer_engine`` unchanged.

    import transformerengine_b200.compat as compat
    compat.install_as_transformer_engine()

    import transformer_engine.pytorch as te                       # this library
    from transformer_engine.common.recipe import DelayedScaling   # this library's recipes
    from transformer_engine.pytorch.distributed import checkpoint

After ``install_as_transformer_engine()`` the names ``transformer_engine``, ``transformer_engine.pytorch`` (and every
submodule below it that has a counterpart here: ``distributed``, ``module.linear``, ``tensor.float8_tensor``,
``optimizers``, ``cpu_offload``, ...), and ``transformer_engine.common.recipe`` resolve to this package's modules.
Nothing is copied: the module objects are the same, so ``isinstance`` checks and pickles agree between the two
spellings.  The alias is opt-in (this call, or ``TEB200_ALIAS_TRANSFORMER_ENGINE=1`` in the environment at import of
this package) and refuses to shadow a real ``transformer_engine`` installation.  The compiled extension of the
reference (``transformer_engine_torch``) has no counterpart: code that calls it directly has to be ported.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys
import types

_OURS = "transformerengine_b200"
_INSTALLED = [False]


# reference modules whose counterpart here sits at another place
_RENAMED = {
    "transformer_engine.pytorch.attention.dot_product_attention.utils": _OURS + ".attention.utils",
    "transformer_engine.pytorch.attention.dot_product_attention.context_parallel": _OURS + ".parallel.context_parallel",
    "transformer_engine.pytorch.attention.dot_product_attention.dot_product_attention":
        _OURS + ".attention.dot_product_attention",
    "transformer_engine.pytorch.ops": _OURS + ".fusible",
    "transformer_engine.pytorch.utils": _OURS + ".utils",
}


def _target(fullname: str):
    """Name of this package's module behind a ``transformer_engine...`` name, or None."""
    if fullname in _RENAMED:
        return _RENAMED[fullname]
    if fullname == "transformer_engine.pytorch":
        return _OURS
    if fullname.startswith("transformer_engine.pytorch."):
        return _OURS + fullname[len("transformer_engine.pytorch"):]
    if fullname == "transformer_engine.common":
        return _OURS + ".common"
    if fullname.startswith("transformer_engine.common."):
        return _OURS + ".common" + fullname[len("transformer_engine.common"):]
    if fullname == "transformer_engine.debug" or fullname.startswith("transformer_engine.debug."):
        return _OURS + fullname[len("transformer_engine"):]
    return None


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        return importlib.import_module(self.target)       # the SAME module object under a second name

    def exec_module(self, module):
        return None


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        t = _target(fullname)
        if t is None:
            return None
        try:
            if importlib.util.find_spec(t) is None:
                return None
        except (ImportError, ValueError):
            return None
        real = importlib.import_module(t)
        spec = importlib.machinery.ModuleSpec(fullname, _AliasLoader(t), is_package=hasattr(real, "__path__"))
        return spec


def is_installed() -> bool:
    return _INSTALLED[0]


def install_as_transformer_engine() -> None:
    """Make ``import transformer_engine...`` resolve to this package (see the module docstring)."""
    if _INSTALLED[0]:
        return
    existing = sys.modules.get("transformer_engine")
    if existing is not None and getattr(existing, "__file__", None):
        raise RuntimeError("a real transformer_engine package is already imported; the alias would shadow it")
    try:
        spec = importlib.util.find_spec("transformer_engine") if existing is None else None
    except (ImportError, ValueError):
        spec = None
    if spec is not None and spec.origin:
        raise RuntimeError(f"transformer_engine is installed ({spec.origin}); refusing to shadow it")
    ours = importlib.import_module(_OURS)
    root = existing if existing is not None else types.ModuleType("transformer_engine")
    root.__doc__ = "Alias of transformerengine_b200 (transformerengine_b200.compat.install_as_transformer_engine)."
    root.__path__ = []                      # a package, so that submodule imports reach the finder
    root.__version__ = getattr(ours, "__version__", "0")
    sys.modules["transformer_engine"] = root
    sys.meta_path.insert(0, _AliasFinder())
    # importing through the finder sets the attributes on the parents as the import system always does
    root.pytorch = importlib.import_module("transformer_engine.pytorch")
    root.common = importlib.import_module("transformer_engine.common")
    importlib.import_module("transformer_engine.common.recipe")
    # names below a parent that is a plain module here (the reference's dot_product_attention is a package) cannot go
    # through the finder: register them directly
    for alias, target in _RENAMED.items():
        sys.modules.setdefault(alias, importlib.import_module(target))
    _INSTALLED[0] = True
