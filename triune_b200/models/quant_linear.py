"""Quantised linear layers and model converters for the serving path.

Parity: ``FP8Linear`` / ``convert_to_fp8`` (``triune/model/fp8.py:126-195``), ``FP4Linear`` /
``convert_to_nvfp4`` (``triune/model/fp4.py:25-114``) and ``NVFP4Linear`` (``triune/kernels/fast_nvfp4.py:543-696``).

Formats
  * FP8: E4M3 weights with one fp32 scale per 128x128 block; activations are quantised per 1x128 row segment at
    run time (the reference used a single per-tensor scale).
  * NVFP4: packed E2M1 (two codes per byte) with one E4M3 scale per 16 elements and one fp32 per-tensor scale;
    optional 16-point Hadamard rotation of the weight rows folded into the activation path. ``from_reference``
    reads the reference's legacy layout (bf16 block scales, tensor scale 1).
Sensitive layers (router, exit heads, final head, embeddings, small gates) are left in bf16 by the converters.
"""

from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import reference as ref

PROTECTED = ("router", "exit_head", "final_head", "lm_head", "embed")


class FP8Linear(nn.Module):
    """Linear with a bf16/fp32 master weight; the forward runs the block-scaled E4M3 GEMM."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, block: int = 128, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features, self.block = in_features, out_features, block
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, std=0.02)
        self._q = None  # (version, wq, ws)
        self._mx = None  # (version, E4M3 weight, blocked power-of-two scales per 1x32) for the block-scaled tensor-core GEMM
        self.mx = True   # inference on CUDA: MXFP8 (scales applied by the tensor core); False: fp32 128-block scales

    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, std=0.02)
        if self.bias is not None:
            nn.init.zeros_(self.bias)
        self._q = self._mx = None

    def quantized_mx(self):
        from ..ops import quant_cuda

        v = self.weight._version
        if self._mx is None or self._mx[0] != v or self._mx[1].device != self.weight.device:
            wq, sf = quant_cuda.mxfp8_quantize(self.weight.detach().to(torch.bfloat16))
            self._mx = (v, wq, sf)
        return self._mx[1], self._mx[2]

    @classmethod
    def from_linear(cls, lin: nn.Linear, block: int = 128) -> "FP8Linear":
        m = cls(lin.in_features, lin.out_features, lin.bias is not None, block)
        m.weight = nn.Parameter(lin.weight.detach().clone(), requires_grad=lin.weight.requires_grad)
        if lin.bias is not None:
            m.bias = nn.Parameter(lin.bias.detach().clone(), requires_grad=lin.bias.requires_grad)
        return m

    def quantized(self):
        v = self.weight._version
        if self._q is None or self._q[0] != v or self._q[1].device != self.weight.device:
            wq, ws = ref.fp8_block_quantize_weight(self.weight.detach(), self.block)
            self._q = (v, wq, ws)
        return self._q[1], self._q[2]

    fused_gelu = True  # forward(x, gelu=True) applies tanh-GELU (in the GEMM epilogue on the block-scaled path)

    def forward(self, x: torch.Tensor, gelu: bool = False) -> torch.Tensor:
        if self.training and torch.is_grad_enabled() and self.weight.requires_grad:
            # straight-through: quantisation error enters the forward, gradients flow to the master weight
            wq, ws = self.quantized()
            w_dq = (wq.float() * ws.repeat_interleave(self.block, 0).repeat_interleave(self.block, 1)
                    [: self.out_features, : self.in_features]).to(self.weight.dtype)
            w = self.weight + (w_dq - self.weight).detach()
            y = F.linear(x, w, self.bias)
            return ops.gelu_tanh(y) if gelu else y
        x2 = x.reshape(-1, self.in_features)
        from ..ops import quant_cuda

        if self.mx and quant_cuda.mxfp8_supported(x2, self.in_features, self.out_features) and self.weight.is_cuda:
            wq, sf = self.quantized_mx()
            y = quant_cuda.mxfp8_linear(x2, wq, sf, x.dtype, bias=self.bias, gelu=gelu)  # bias / GELU in the epilogue
            return y.view(*x.shape[:-1], self.out_features)
        wq, ws = self.quantized()
        y = ops.fp8_linear(x2, wq, ws, self.block, out_dtype=x.dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        if gelu:
            y = ops.gelu_tanh(y)
        return y.view(*x.shape[:-1], self.out_features)


class NVFP4Linear(nn.Module):
    """Inference linear over packed NVFP4 weights (buffers only; ~4.5 bits per weight)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, hadamard: bool = False,
                 scale_dtype=torch.float8_e4m3fn):
        super().__init__()
        assert in_features % 16 == 0, "NVFP4 needs in_features to be a multiple of 16"
        self.in_features, self.out_features, self.hadamard = in_features, out_features, hadamard
        self.register_buffer("packed_weight", torch.zeros(out_features, in_features // 2, dtype=torch.uint8))
        self.register_buffer("block_scales", torch.zeros(out_features, in_features // 16, dtype=scale_dtype))
        self.register_buffer("tensor_scale", torch.ones((), dtype=torch.float32))
        self.bias = nn.Parameter(torch.zeros(out_features), requires_grad=False) if bias else None
        self._dq = None
        self.w4a4 = True          # prefer the block-scaled E2M1 x E2M1 tensor-core GEMM where it applies
        self._sf_blocked = None   # block scales in the GEMM's layout (derived, not saved)
        self._alpha = 1.0

    @classmethod
    def empty_skeleton(cls, in_features, out_features, bias=False, hadamard=False, device=None):
        m = cls(in_features, out_features, bias, hadamard)
        return m.to(device) if device is not None else m

    @classmethod
    def from_linear(cls, lin: nn.Linear, hadamard: bool = False) -> "NVFP4Linear":
        m = cls(lin.in_features, lin.out_features, lin.bias is not None, hadamard)
        m.load_weight(lin.weight.detach())
        if lin.bias is not None:
            m.bias.data.copy_(lin.bias.detach())
        return m.to(lin.weight.device)

    @classmethod
    def from_reference(cls, packed: torch.Tensor, scales_bf16: torch.Tensor, hadamard: bool = False) -> "NVFP4Linear":
        """Adopt the reference's layout (E2M1 + bf16 scale per 16 elements)."""
        out_f, half = packed.shape
        m = cls(half * 2, out_f, False, hadamard, scale_dtype=torch.bfloat16)
        m.packed_weight.copy_(packed)
        m.block_scales.copy_(scales_bf16)
        return m

    @torch.no_grad()
    def load_weight(self, w: torch.Tensor):
        # the rotation of each group of 16 input features is folded into the quantiser; activations get the same one
        if w.is_cuda and self.block_scales.dtype == torch.float8_e4m3fn:
            p, s, t = ops.nvfp4_quantize(w, hadamard=self.hadamard)
        else:
            wf = ref.fwht16(w.float()) if self.hadamard else w.float()
            p, s, t = ref.nvfp4_quantize(wf, self.block_scales.dtype)
        self.packed_weight = p.to(self.packed_weight.device)
        self.block_scales = s.to(self.block_scales.device)
        self.tensor_scale = t.to(self.tensor_scale.device)
        self._dq = None
        self._sf_blocked = None

    def dequantized(self, dtype=torch.bfloat16) -> torch.Tensor:
        return ref.nvfp4_dequantize(self.packed_weight, self.block_scales, self.tensor_scale, dtype)

    def bits_per_weight(self) -> float:
        n = self.out_features * self.in_features
        return 8.0 * (self.packed_weight.numel() + self.block_scales.numel() * self.block_scales.element_size()) / n

    def _w4a4_ready(self, x2: torch.Tensor) -> bool:
        """Block-scaled tensor-core path (activations quantised to E2M1 on the fly, both scale sets applied by the
        tensor core): CUDA bf16 activations, E4M3 block scales, more rows than the GEMV path serves."""
        from ..ops import quant_cuda

        return (self.w4a4 and quant_cuda.nvfp4_supported(x2, self.packed_weight) and x2.shape[0] > 8
                and self.block_scales.dtype == torch.float8_e4m3fn and self.in_features % 32 == 0
                and self.out_features % 8 == 0)

    fused_gelu = True  # forward(x, gelu=True) applies tanh-GELU (in the GEMM epilogue on the block-scaled path)

    def forward(self, x: torch.Tensor, gelu: bool = False) -> torch.Tensor:
        x2 = x.reshape(-1, self.in_features)
        if self._w4a4_ready(x2):
            from ..ops import quant_cuda

            if self._sf_blocked is None or self._sf_blocked.device != x2.device:
                self._sf_blocked = quant_cuda.nvfp4_block_scales(self.block_scales, self.in_features)
                self._alpha = float(self.tensor_scale)  # one host read, at the first call
            y = quant_cuda.nvfp4_w4a4_linear(x2, self.packed_weight, self._sf_blocked, self._alpha, self.hadamard, x.dtype,
                                             bias=self.bias, gelu=gelu)
            return y.view(*x.shape[:-1], self.out_features)
        else:
            if self.hadamard:
                x2 = ops.fwht16(x2)
            y = ops.nvfp4_linear(x2, self.packed_weight, self.block_scales, self.tensor_scale, out_dtype=x.dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        if gelu:
            y = ops.gelu_tanh(y)
        return y.view(*x.shape[:-1], self.out_features)


class FP4Linear(nn.Module):
    """Training-time 4-bit linear: quantise-dequantise forward with a straight-through estimator, master-weight
    backward (the reference used Transformer Engine when present, else this STE form)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def to_nvfp4_inference(self) -> "NVFP4Linear":
        """This layer as packed 4-bit inference storage (E2M1 values, one scale per 16 inputs)."""
        if self.in_features % 16 != 0:
            raise ValueError(f"NVFP4 packed format requires in_features % 16 == 0, got {self.in_features}")
        return NVFP4Linear.from_linear(self)

    def forward(self, x):
        w = self.weight
        if w.shape[1] % 16 == 0:
            p, s, t = ref.nvfp4_quantize(w.detach().float())
            w = w + (ref.nvfp4_dequantize(p, s, t, w.dtype) - w).detach()
        return F.linear(x, w, self.bias)


def _protected(name: str, mod: nn.Linear, extra: Iterable[str]) -> bool:
    low = name.lower()
    if any(k in low for k in tuple(PROTECTED) + tuple(extra)):
        return True
    return "gate" in low and mod.out_features * mod.in_features < 65536


def _convert(model: nn.Module, make, protect: Iterable[str], min_features: int):
    n = 0
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if type(child) is nn.Linear and not _protected(full, child, protect) and child.in_features % 16 == 0 \
                    and min(child.in_features, child.out_features) >= min_features:
                setattr(mod, child_name, make(child))
                n += 1
    return n


def convert_to_fp8(model: nn.Module, protect: Iterable[str] = (), min_features: int = 16) -> int:
    """Replace eligible ``nn.Linear`` modules by :class:`FP8Linear`; returns the number converted."""
    return _convert(model, FP8Linear.from_linear, protect, min_features)


def convert_to_nvfp4(model: nn.Module, hadamard: bool = False, protect: Iterable[str] = (), min_features: int = 16,
                     w4a4: bool = True) -> int:
    """Replace eligible ``nn.Linear`` modules by packed :class:`NVFP4Linear`; returns the number converted. ``w4a4``
    (default) lets prefill-sized calls quantise their activations too and run on the block-scaled tensor-core GEMM;
    ``w4a4=False`` keeps activations in bf16 (weights decoded in front of the bf16 GEMM)."""

    def make(l):
        m = NVFP4Linear.from_linear(l, hadamard)
        m.w4a4 = bool(w4a4)
        return m

    return _convert(model, make, protect, min_features)
