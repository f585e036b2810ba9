"""Precision recipes: callables that return the context a training / inference forward runs under, with a
``description`` attribute saying what will actually execute.

Parity: ``triune/recipes/{bf16,fp8,mxfp8,nvfp4}.py``. The reference leans on autocast and Transformer Engine; this
framework stores parameters in the compute dtype and quantised paths are module conversions
(``convert_to_fp8`` / ``convert_to_nvfp4``), so a recipe = (optional conversion) + a context that is normally empty.
"""

from __future__ import annotations

from contextlib import nullcontext
from typing import Callable

import torch

from ..models.quant_linear import convert_to_fp8, convert_to_nvfp4
from ..runtime.capabilities import PrecisionCapabilities

__all__ = ["bf16_autocast", "build_fp8_precision_context", "build_mxfp8_precision_context", "build_precision_context",
           "apply_precision", "convert_to_fp8", "convert_to_nvfp4"]


def bf16_autocast(device_type: str = "cuda"):
    """Autocast for foreign fp32 models; native models are already bf16 and need no context."""
    return torch.amp.autocast(device_type, dtype=torch.bfloat16) if device_type == "cuda" else nullcontext()


def _ctx(factory, description: str) -> Callable:
    fn = lambda: factory()  # noqa: E731
    fn.description = description
    return fn


def build_fp8_precision_context(*, device, use_te: bool = False) -> Callable:
    if torch.device(device).type != "cuda":
        raise RuntimeError("FP8 requires CUDA")
    caps = PrecisionCapabilities.detect(device)
    if caps.fp8_gemm:
        return _ctx(nullcontext, "block-scaled E4M3 GEMM (tcgen05 kind::f8f6f4, 1x128 / 128x128 scales) in FP8Linear modules")
    return _ctx(lambda: bf16_autocast("cuda"), "FP8 kernels unavailable on SM%d.%d; BF16" % caps.compute_capability)


def build_mxfp8_precision_context(*, device) -> Callable:
    if torch.device(device).type != "cuda":
        raise RuntimeError("MXFP8 requires CUDA")
    caps = PrecisionCapabilities.detect(device)
    if caps.fp8_gemm:  # 1x32 power-of-two scales are not implemented; the 1x128 fp32-scaled path serves the request
        return _ctx(nullcontext, "MXFP8 requested: served by the 1x128 / 128x128 fp32-scaled E4M3 GEMM")
    return _ctx(lambda: bf16_autocast("cuda"), "Fallback BF16 autocast")


def build_precision_context(*, use_fp4: bool, device) -> Callable:
    dev = torch.device(device)
    if not use_fp4:
        return _ctx(lambda: bf16_autocast(dev.type) if dev.type != "cuda" else nullcontext(), "BF16 parameters and compute")
    if dev.type != "cuda":
        raise RuntimeError("NVFP4 requires CUDA")
    caps = PrecisionCapabilities.detect(dev)
    if not caps.fp4_gemm:
        raise RuntimeError("NVFP4 requires the sm_100a kernels of this framework; found SM%d.%d" % caps.compute_capability)
    return _ctx(nullcontext, "NVFP4 weights (E2M1 + E4M3/16 scales), W4A16 tensor-core GEMM / packed GEMV")


def apply_precision(model, precision: str, device=None, fallback: bool = True) -> str:
    """Convert ``model`` in place for 'fp8' / 'fp4' serving; returns the precision that was applied."""
    dev = torch.device(device) if device is not None else next(model.parameters()).device
    p = PrecisionCapabilities.detect(dev).resolve_precision(precision, fallback) if dev.type == "cuda" else precision
    if p == "fp8":
        convert_to_fp8(model)
    elif p == "fp4":
        convert_to_nvfp4(model)
    return p
