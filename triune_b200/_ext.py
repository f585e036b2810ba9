"""Loader of the native torch extension ``triune_b200._C``.

The extension is built in-tree by :mod:`triune_b200._build`. On a machine with a GPU the ops refuse to
run without it (no silent PyTorch fall-back on CUDA tensors); on a CPU-only machine the pure-PyTorch
reference ops are used and the extension is never touched.
"""

from __future__ import annotations

import importlib
import os
from functools import lru_cache

_FORCE_REFERENCE = os.environ.get("TRIUNE_REFERENCE_OPS", "0") == "1"


@lru_cache(maxsize=1)
def _load():
    try:
        return importlib.import_module("triune_b200._C")
    except ImportError as e:  # pragma: no cover - depends on build state
        return e


def ext():
    """Return the extension module or raise a clear error."""
    m = _load()
    if isinstance(m, Exception):
        raise RuntimeError(
            "triune_b200._C is not built; run `python -m triune_b200._build` (needs nvcc). "
            f"Import error was: {m}"
        )
    return m


def ext_available() -> bool:
    return not isinstance(_load(), Exception)


def use_kernels(*tensors) -> bool:
    """True when the sm_100a kernels must handle these tensors (all CUDA, reference mode off)."""
    if _FORCE_REFERENCE:
        return False
    if not tensors or not all(t is None or t.is_cuda for t in tensors):
        return False
    ext()  # raises loudly if a CUDA tensor arrives and the extension is missing
    return True


def set_reference_ops(flag: bool) -> None:
    """Route every op through the PyTorch reference (oracle mode for tests)."""
    global _FORCE_REFERENCE
    _FORCE_REFERENCE = bool(flag)


def reference_ops_enabled() -> bool:
    return _FORCE_REFERENCE
