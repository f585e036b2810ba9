"""Precision capabilities of the device, probed by running this framework's own kernels.

Parity (``triune/runtime/capabilities.py:17-194``): ``PrecisionCapabilities.detect`` and ``resolve_precision`` with
fallback. The reference asks whether cuBLAS ``_scaled_mm`` or Transformer Engine can run; here the question is whether
the in-tree sm_100a kernels can: each probe runs one tiny problem and compares it with the PyTorch oracle, once per
device, so a mis-built extension shows up as "unsupported" instead of as wrong numbers later.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

log = logging.getLogger(__name__)
_PROBES: Dict[Tuple[int, str], bool] = {}


def _probe(device: torch.device, name: str, fn) -> bool:
    key = (device.index if device.index is not None else torch.cuda.current_device(), name)
    if key not in _PROBES:
        try:
            _PROBES[key] = bool(fn())
        except Exception as e:  # extension missing, wrong architecture, launch failure
            log.debug("capability probe %s failed: %s", name, e)
            _PROBES[key] = False
    return _PROBES[key]


def _probe_bf16_gemm(dev) -> bool:
    from .. import ops

    a = torch.randn(128, 64, device=dev).bfloat16()
    b = torch.randn(128, 64, device=dev).bfloat16()
    return torch.allclose(ops.gemm(a, b).float(), a.float() @ b.float().t(), atol=0.5, rtol=5e-2)


def _probe_fp8_gemm(dev) -> bool:
    from ..ops import quant_cuda, reference as ref

    x = torch.randn(128, 128, device=dev).bfloat16()
    wq, ws = ref.fp8_block_quantize_weight(torch.randn(128, 128, device=dev) * 0.05)
    xq, xs = quant_cuda.fp8_quantize_act(x)
    y = quant_cuda.fp8_block_gemm(xq, xs, wq, ws).float()
    want = ref.fp8_block_gemm(xq, xs, wq, ws, 128, torch.float32)
    return bool((y - want).abs().max() <= 2e-2 * want.abs().max())


def _probe_nvfp4(dev) -> bool:
    from ..ops import quant_cuda, reference as ref

    w = torch.randn(64, 128, device=dev) * 0.1
    p, s, t = quant_cuda.nvfp4_quantize(w)
    return torch.equal(quant_cuda.nvfp4_dequant(p, s, t).float(), ref.nvfp4_dequantize(p, s, t, torch.bfloat16).float())


@dataclass
class PrecisionCapabilities:
    device: torch.device
    compute_capability: Tuple[int, int]
    fp8_gemm: bool
    fp4_gemm: bool
    transformer_engine: bool
    native_scaled_mm: bool
    bf16_supported: bool
    mxfp8_gemm: bool = False
    tcgen05: bool = False  # the tensor-core GEMM of this framework runs and matches the oracle

    @classmethod
    def detect(cls, device=None) -> "PrecisionCapabilities":
        dev = torch.device(device) if device is not None else torch.device("cuda:0" if torch.cuda.is_available() else "cpu")
        if dev.type != "cuda" or not torch.cuda.is_available():
            return cls(dev, (0, 0), False, False, False, False, False)
        from .. import _ext

        major, minor = torch.cuda.get_device_capability(dev)
        have_ext = major == 10 and _ext.ext_available()
        tc = have_ext and _probe(dev, "bf16", lambda: _probe_bf16_gemm(dev))
        fp8 = have_ext and _probe(dev, "fp8", lambda: _probe_fp8_gemm(dev))
        fp4 = have_ext and _probe(dev, "nvfp4", lambda: _probe_nvfp4(dev))
        try:
            import transformer_engine.pytorch  # noqa: F401

            te = True
        except Exception:
            te = False
        return cls(dev, (major, minor), fp8, fp4, te, hasattr(torch, "_scaled_mm") and (major, minor) >= (8, 9),
                   major >= 8 and torch.cuda.is_bf16_supported(), mxfp8_gemm=False, tcgen05=tc)

    def resolve_precision(self, requested: str, fallback: bool = True) -> str:
        """'fp4' | 'nvfp4' | 'fp8' | 'mxfp8' | 'bf16' | 'bfloat16' | 'fp16' | 'fp32' | 'float32' -> what will actually run."""
        req = requested.lower().strip()
        alias = {"bfloat16": "bf16", "float32": "fp32", "float16": "fp16", "nvfp4": "fp4"}
        req = alias.get(req, req)
        base = "bf16" if self.bf16_supported else "fp32"
        ok = {"fp4": self.fp4_gemm, "fp8": self.fp8_gemm, "mxfp8": self.mxfp8_gemm, "bf16": self.bf16_supported, "fp16": True,
              "fp32": True}
        if req not in ok:
            raise ValueError(f"unknown precision {requested!r}")
        if ok[req]:
            return req
        major, minor = self.compute_capability
        msg = f"{req.upper()} requested but unsupported on {self.device} (SM{major}.{minor})"
        if not fallback:
            raise RuntimeError(msg)
        if req == "fp4" and self.fp8_gemm:
            log.warning("%s; falling back to FP8.", msg)
            return "fp8"
        log.warning("%s; falling back to %s.", msg, base.upper())
        return base

    def summary(self) -> Dict[str, object]:
        return {"device": str(self.device), "sm": "%d.%d" % self.compute_capability, "tcgen05_gemm": self.tcgen05,
                "fp8_block_gemm": self.fp8_gemm, "nvfp4": self.fp4_gemm, "bf16": self.bf16_supported}
