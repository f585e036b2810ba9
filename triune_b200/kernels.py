"""The kernel-level functions of the reference under their own names, on this framework's operators.

Code written against ``triune.kernels`` (``fast_rmsnorm``, ``fast_chunk_gla``, ``chunked_cross_entropy_from_hidden``,
``fast_zeropower_via_newtonschulz5``, ``nvfp4_linear`` ...; ``triune/kernels/__init__.py``) keeps working after
``from triune_b200 import kernels``: same names, same argument order, same tensor layouts, same return shapes. Behind
them are the sm_100a CUDA kernels on a GPU and the PyTorch reference operators elsewhere (``triune_b200/ops``); there
is no Triton here, so ``is_triton_available()`` is False and the backend reports itself as ``cuda-sm100a`` or ``pytorch``.

Layout notes where the two projects differ inside: ``fast_rope`` takes head-major ``[B, H, T, D]`` tensors (this
framework's operator takes ``[B, T, H, D]``); ``nvfp4_quantize`` returns ``(packed, scale)`` with bf16 block scales and no
tensor-level scale, the reference's legacy layout, and ``NVFP4Linear`` here is constructed like the reference's
(``in_features, out_features, bias, dtype, hadamard``).
"""

from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _ext, ops
from .ops import reference as _ref

_TURBO = {"on": True}


# ---------------------------------------------------------------------------------------------------- dispatcher facts
def is_triton_available() -> bool:
    return False


def get_triton_error() -> Optional[str]:
    return "this framework does not use Triton: its GPU kernels are hand-written CUDA for sm_100a"


def is_turbo_mode_enabled() -> bool:
    return _TURBO["on"]


def set_turbo_mode(enabled: bool) -> bool:
    """Turbo on: CUDA tensors go to the sm_100a kernels (the default). Off: everything runs on the PyTorch reference
    operators, which is what the numerics tests compare the kernels against. Returns the new state."""
    _TURBO["on"] = bool(enabled)
    _ext.set_reference_ops(not _TURBO["on"])
    return _TURBO["on"]


def get_kernel_backend() -> str:
    return "cuda-sm100a" if (_TURBO["on"] and torch.cuda.is_available() and _ext.ext_available()) else "pytorch"


def get_kernel_telemetry() -> Dict[str, Any]:
    return {"backend": get_kernel_backend(), "turbo_mode": _TURBO["on"], "triton": False, "extension_built": _ext.ext_available(),
            "kernel_launches": ops.launch_count(), "cuda_available": torch.cuda.is_available()}


# ---------------------------------------------------------------------------------------------------- norms, activations
def fast_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return ops.rmsnorm(x, weight.to(x.dtype) if weight.dtype != x.dtype else weight, eps)


def fast_fused_add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (rmsnorm(x + residual) * weight, x + residual)."""
    w = weight.to(x.dtype) if weight.dtype != x.dtype else weight
    if residual is None:
        return ops.rmsnorm(x, w, eps), x
    return ops.add_rmsnorm(x, residual, w, eps)


class FastRMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        if residual is not None:
            return fast_fused_add_rmsnorm(x, residual, self.weight, self.eps)
        return fast_rmsnorm(x, self.weight, self.eps)


def fast_swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return ops.swiglu(gate, up)


def fast_gelu(x: torch.Tensor) -> torch.Tensor:
    return ops.gelu_tanh(x)


class FastSwiGLU(nn.Module):
    def forward(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        return fast_swiglu(gate, up)


class FastGELU(nn.GELU):
    def __init__(self, approximate: str = "tanh"):
        super().__init__(approximate=approximate)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return fast_gelu(x) if self.approximate == "tanh" else super().forward(x)


def fast_rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rotary embedding of head-major ``q, k [B, H, T, D]`` (half-split pairs ``(x[i], x[i + D/2])``) with ``cos / sin`` of
    ``[T, D/2]`` or ``[T, D]`` (leading singleton dimensions allowed)."""
    D, T = q.shape[-1], q.shape[-2]
    c, s = cos.reshape(-1, cos.shape[-1])[:T], sin.reshape(-1, sin.shape[-1])[:T]
    if c.shape[-1] == D // 2:
        c, s = torch.cat((c, c), dim=-1), torch.cat((s, s), dim=-1)
    qt, kt = q.transpose(1, 2), k.transpose(1, 2)  # the operator's layout is [B, T, H, D]
    return ops.apply_rope(qt, c, s).transpose(1, 2), ops.apply_rope(kt, c, s).transpose(1, 2)


# ---------------------------------------------------------------------------------------------------- cross entropy
def fast_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, chunk_size: int = 2048, ignore_index: int = -100) -> torch.Tensor:
    """Mean cross entropy over the targets that are not ``ignore_index`` (``chunk_size`` is accepted for compatibility: the
    kernel works row by row and needs no chunking)."""
    return ops.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), ignore_index)


def chunked_cross_entropy_from_hidden(hidden_states: torch.Tensor, lm_head, targets: torch.Tensor, chunk_size: int = 1024,
                                      ignore_index: int = -100, force_chunked: bool = False) -> torch.Tensor:
    """Cross entropy straight from the hidden states: the head GEMM and the loss run chunk by chunk, so ``[N, V]`` logits
    never exist as a whole. ``lm_head`` is an ``nn.Linear`` or a weight ``[V, d]``."""
    weight = lm_head.weight if isinstance(lm_head, nn.Linear) else lm_head
    bias = lm_head.bias if isinstance(lm_head, nn.Linear) else None
    h = hidden_states.reshape(-1, hidden_states.shape[-1])
    return ops.linear_cross_entropy(h, weight, targets.reshape(-1), bias=bias, ignore_index=ignore_index)


class FastChunkedCrossEntropyLoss(nn.Module):
    def __init__(self, chunk_size: int = 1024, ignore_index: int = -100):
        super().__init__()
        self.chunk_size, self.ignore_index = chunk_size, ignore_index

    def forward(self, logits_or_hidden: torch.Tensor, targets: torch.Tensor, lm_head=None) -> torch.Tensor:
        if lm_head is not None:
            return chunked_cross_entropy_from_hidden(logits_or_hidden, lm_head, targets, self.chunk_size, self.ignore_index)
        return fast_cross_entropy(logits_or_hidden, targets, self.chunk_size, self.ignore_index)


# ---------------------------------------------------------------------------------------------------- sequence mixers
def fast_chunk_gla(q, k, v, g, initial_state=None, chunk_size: int = 64, out: Optional[torch.Tensor] = None):
    """Gated linear attention over ``[B, T, H, D]`` with log-decay gates ``g``; -> (output [B, T, H, Dv], final state
    [B, H, Dk, Dv])."""
    o, s = ops.gla(q, k, v, g, initial_state=initial_state, chunk_size=chunk_size)
    if out is not None:
        out.copy_(o)
        o = out
    return o, s


def fast_chunk_gated_deltanet(q, k, v, g, beta=None, initial_state=None, chunk_size: int = 64):
    return ops.gated_deltanet(q, k, v, g, beta=beta, initial_state=initial_state)


def fast_recurrent_gated_deltanet(q, k, v, g, beta=None, initial_state=None):
    """Token-by-token delta rule (decode, or an oracle for the chunked form)."""
    if _ext.use_kernels(q):
        return ops.gated_deltanet(q, k, v, g, beta=beta, initial_state=initial_state)
    return _ref.gated_deltanet_recurrent(q, k, v, g, beta, initial_state)


# ---------------------------------------------------------------------------------------------------- optimizer, LoRA
def fast_zeropower_via_newtonschulz5(G: torch.Tensor, steps: int = 5, eps: float = 1e-7, scratch_buffer=None, return_scratch: bool = False):
    """Quintic Newton-Schulz orthogonalisation of ``G [.., m, n]`` (``scratch_buffer`` is accepted and handed back: the
    kernels here keep their own workspace)."""
    X = ops.muon_ns(G, steps)
    return (X, scratch_buffer) if return_scratch else X


NS5_COEFFS = (1.875, -1.25, 0.375)  # quintic Newton-Schulz polynomial X <- aX + b(XX^T)X + c(XX^T)^2 X
NVFP4_GROUP_SIZE = 16  # elements per E4M3 block scale
HAS_TRITON = False  # no kernel of this framework goes through Triton; the name answers scripts that ask


def compute_muon_update_scale(d_out: int, d_in: int, rms_target: Optional[float] = None) -> float:
    """Scale of an orthogonalised update so that its per-element size does not depend on the matrix's aspect ratio:
    sqrt(max(1, d_out / d_in)), times ``rms_target`` when one is given (``triune/kernels/fast_muon.py:8-12``)."""
    aspect = max(1.0, float(d_out) / float(d_in)) ** 0.5
    return aspect * float(rms_target) if rms_target is not None and rms_target > 0 else aspect


def fast_zeropower_via_newtonschulz5_batched(G_batch: torch.Tensor, steps: int = 5, eps: float = 1e-7, scratch_buffer=None,
                                             return_scratch: bool = False):
    """``fast_zeropower_via_newtonschulz5`` for a stack ``[B, m, n]`` (one launch per Newton-Schulz step for the whole
    stack on the GPU)."""
    if G_batch.ndim != 3:
        raise ValueError(f"Batched orthogonalization requires 3D tensor [B, M, N], got ndim={G_batch.ndim}")
    X = ops.muon_ns(G_batch, steps)
    return (X, scratch_buffer) if return_scratch else X


def fast_triangular_adamw(R_batch: torch.Tensor, batch_mom: torch.Tensor, batch_var: torch.Tensor, batch_delta: torch.Tensor,
                          step_vals: torch.Tensor, beta1: float, beta2: float, eps: float = 1e-8, mask_mode: str = "triu") -> torch.Tensor:
    """Adam direction of a stack of small core matrices ``[N, DR, DR]``: moments updated in place, the bias-corrected
    direction written to ``batch_delta``; ``mask_mode="triu"`` zeroes the direction below the diagonal, ``"full"`` keeps
    it dense. ``step_vals`` holds one step count per matrix. Where all counts agree and the stack is fp32 on the GPU the
    fused kernel of the optimizer runs; otherwise the same arithmetic in PyTorch
    (``triune/kernels/fast_triangular.py:91-170`` of the reference)."""
    if mask_mode not in ("triu", "full"):
        raise ValueError(f"Unknown mask_mode={mask_mode!r}; expected 'triu' or 'full'")
    N = R_batch.shape[0]
    steps = step_vals.reshape(-1)
    if steps.numel() == 1 and N > 1:
        steps = steps.expand(N)
    if (_ext.use_kernels(R_batch) and mask_mode == "full" and R_batch.dtype == torch.float32 and R_batch.is_contiguous()
            and batch_mom.dtype == torch.float32 and batch_var.dtype == torch.float32 and batch_mom.is_contiguous()
            and batch_var.is_contiguous() and N > 0 and bool((steps == steps[0]).all())):
        # the kernel masks its INPUT when asked for a triangle (moments of the lower part stay zero); the reference keeps
        # dense moments and masks the direction only, so only the dense mode maps onto it one to one
        delta = _ext.ext().triangular_adamw(R_batch, batch_mom, batch_var, beta1, beta2, eps, int(steps[0]), False, None)
        batch_delta.copy_(delta)
        return batch_delta
    R = R_batch.float()
    batch_mom.lerp_(R, 1.0 - beta1)
    batch_var.mul_(beta2).addcmul_(R, R, value=1.0 - beta2)
    t = steps.to(torch.float32).view(N, 1, 1)
    c1 = 1.0 - beta1 ** t
    c2 = (1.0 - beta2 ** t).clamp_min(1e-7)
    delta = (batch_mom / c1) / ((batch_var / c2).sqrt() + eps)
    if mask_mode == "triu":
        delta = delta.triu()
    batch_delta.copy_(delta)
    return batch_delta


def fast_lora_forward(x: torch.Tensor, lora_A: torch.Tensor, lora_B: torch.Tensor, scaling: float = 2.0) -> torch.Tensor:
    """scaling * (x A^T) B^T with A [r, in], B [out, r]."""
    return ops.linear(ops.linear(x, lora_A), lora_B, alpha=float(scaling))


def fast_lora_linear(x, weight, bias, lora_A, lora_B, scaling: float = 2.0) -> torch.Tensor:
    return ops.lora_linear(x, weight, bias, lora_A, lora_B, scaling)


def fast_qkv_lora_linear(x, W_q, b_q, W_k, b_k, W_v, b_v, A_q, B_q, A_k, B_k, A_v, B_v, scaling: float = 2.0) -> torch.Tensor:
    """The three projections with their adapters, concatenated along the feature dimension: [.., q | k | v]."""
    return torch.cat((ops.lora_linear(x, W_q, b_q, A_q, B_q, scaling), ops.lora_linear(x, W_k, b_k, A_k, B_k, scaling),
                      ops.lora_linear(x, W_v, b_v, A_v, B_v, scaling)), dim=-1)


def fast_gate_up_lora_linear(x, W_g, b_g, W_u, b_u, A_g, B_g, A_u, B_u, scaling: float = 2.0) -> torch.Tensor:
    """silu(gate) * up with adapters on both projections."""
    return ops.swiglu(ops.lora_linear(x, W_g, b_g, A_g, B_g, scaling), ops.lora_linear(x, W_u, b_u, A_u, B_u, scaling))


# ---------------------------------------------------------------------------------------------------- FP8, NVFP4
def is_fp8_available(device: Optional[torch.device] = None) -> bool:
    """E4M3 tensor-core GEMMs exist where the sm_100a extension runs; elsewhere the FP8 layers compute in bf16 from
    de-quantised weights."""
    dev = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    return dev.type == "cuda" and torch.cuda.is_available() and _ext.ext_available()


def fast_fp8_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T + b with the weight rounded to block-scaled E4M3 on the way (one-off use; keep a ``FastFP8Linear`` for a
    weight that is used more than once, so that it is quantised once)."""
    from .models.quant_linear import FP8Linear

    return FP8Linear.from_linear(_as_linear(weight, bias)).to(weight.device).eval()(x)


def _as_linear(weight: torch.Tensor, bias: Optional[torch.Tensor]) -> nn.Linear:
    lin = nn.Linear(weight.shape[1], weight.shape[0], bias=bias is not None, device="meta")
    lin.weight = nn.Parameter(weight.detach(), requires_grad=False)
    if bias is not None:
        lin.bias = nn.Parameter(bias.detach(), requires_grad=False)
    return lin


class FastFP8Linear(nn.Module):
    """A linear layer that holds its weight in fp32 / bf16 for training and serves through the block-scaled E4M3 path once
    ``quantize()`` has been called (or on the first evaluation-mode forward)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype: torch.dtype = torch.float32):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        self._q = None

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        if self.bias is not None:
            nn.init.zeros_(self.bias)
        self._q = None

    def quantize(self):
        from .models.quant_linear import FP8Linear

        self._q = FP8Linear.from_linear(_as_linear(self.weight, self.bias)).to(self.weight.device).eval()
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.training:
            self._q = None
            return F.linear(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))
        if self._q is None:
            self.quantize()
        return self._q(x)


def fwht_16(x: torch.Tensor) -> torch.Tensor:
    return ops.fwht16(x)


def nvfp4_quantize(tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[N, K] -> (packed E2M1 [N, K/2] uint8, bf16 block scales [N, K/16]): the layout without a tensor-level scale."""
    packed, scales, _ = _ref.nvfp4_quantize(tensor, torch.bfloat16)
    return packed, scales


def nvfp4_dequantize(packed: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    return _ref.nvfp4_dequantize(packed, scale, 1.0, dtype)


def nvfp4_linear(x: torch.Tensor, packed_weight: torch.Tensor, scale: torch.Tensor, bias: Optional[torch.Tensor] = None, hadamard: bool = False) -> torch.Tensor:
    """y = x W^T + b from a packed weight; with ``hadamard`` the weight was quantised in the rotated basis, so groups of 16
    input features are rotated the same way first."""
    xin = ops.fwht16(x) if hadamard else x
    ts = torch.ones((), device=x.device, dtype=torch.float32)
    y = ops.nvfp4_linear(xin.reshape(-1, xin.shape[-1]), packed_weight, scale, ts, out_dtype=x.dtype).reshape(*x.shape[:-1], packed_weight.shape[0])
    return y if bias is None else y + bias.to(y.dtype)


class NVFP4Linear(nn.Module):
    """The reference's constructor (``in_features, out_features, bias, dtype, hadamard``) over this framework's layer: weights
    live packed (E2M1 + block scales); ``from_linear`` quantises an existing layer."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, dtype: torch.dtype = torch.bfloat16, hadamard: bool = False):
        super().__init__()
        from .models.quant_linear import NVFP4Linear as _Impl

        self.impl = _Impl(in_features, out_features, bias=bias, hadamard=hadamard)
        self.in_features, self.out_features, self.hadamard, self.dtype = in_features, out_features, hadamard, dtype

    @classmethod
    def from_linear(cls, linear: nn.Linear, hadamard: bool = False) -> "NVFP4Linear":
        from .models.quant_linear import NVFP4Linear as _Impl

        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.impl = _Impl.from_linear(linear, hadamard=hadamard)
        self.in_features, self.out_features, self.hadamard, self.dtype = linear.in_features, linear.out_features, hadamard, linear.weight.dtype
        return self

    @classmethod
    def empty_skeleton(cls, in_features: int, out_features: int, bias: bool = False, hadamard: bool = False, device=None) -> "NVFP4Linear":
        """A layer with packed storage of the right shape and no values yet, to be filled by a checkpoint loader."""
        self = cls(in_features, out_features, bias=bias, hadamard=hadamard)
        return self.to(device) if device is not None else self

    @property
    def weight(self) -> torch.Tensor:
        """The de-quantised weight ``[out, in]`` (a copy; the storage stays packed)."""
        return self.impl.dequantized()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.impl(x)


__all__ = ["is_triton_available", "get_kernel_backend", "get_triton_error", "is_turbo_mode_enabled", "set_turbo_mode", "get_kernel_telemetry",
           "fast_rmsnorm", "fast_fused_add_rmsnorm", "FastRMSNorm", "fast_rope", "fast_swiglu", "fast_gelu", "FastSwiGLU", "FastGELU",
           "fast_cross_entropy", "chunked_cross_entropy_from_hidden", "FastChunkedCrossEntropyLoss", "fast_chunk_gla", "fast_chunk_gated_deltanet",
           "fast_recurrent_gated_deltanet", "fast_zeropower_via_newtonschulz5", "fast_lora_forward", "fast_lora_linear", "fast_qkv_lora_linear",
           "fast_gate_up_lora_linear", "is_fp8_available", "fast_fp8_linear", "FastFP8Linear", "nvfp4_quantize", "nvfp4_dequantize", "nvfp4_linear",
           "fwht_16", "NVFP4Linear"]
