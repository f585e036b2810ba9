"""Dispatch of the quantised serving ops to the sm_100a kernels (``csrc/quant/quant_kernels.cu``)."""

from __future__ import annotations

import torch

from .. import _ext
from . import _tick


def fp8_supported(x2, wq) -> bool:
    return _ext.use_kernels(x2, wq) and x2.dtype == torch.bfloat16 and x2.shape[1] % 16 == 0 and wq.shape[0] % 8 == 0


def fp8_quantize_act(x2: torch.Tensor):
    _tick()
    return _ext.ext().fp8_quantize_act(x2.contiguous())


def fp8_block_gemm(xq, xs, wq, ws):
    _tick()
    return _ext.ext().fp8_block_gemm(xq, xs.contiguous(), wq, ws.contiguous())


def fp8_block_linear(x2, wq, ws, block, out_dtype):
    assert block == 128, "the tensor-core path uses 128-wide scale blocks"
    xq, xs = fp8_quantize_act(x2)
    y = fp8_block_gemm(xq, xs, wq, ws)
    return y if out_dtype == torch.bfloat16 else y.to(out_dtype)


def nvfp4_supported(x2, packed) -> bool:
    return _ext.use_kernels(x2, packed) and x2.dtype == torch.bfloat16 and packed.shape[0] % 8 == 0


def nvfp4_quantize(w: torch.Tensor, hadamard: bool = False):
    """[N,K] bf16/fp32 on the GPU -> (packed uint8 [N,K/2], E4M3 scales [N,K/16], fp32 tensor scale)."""
    _tick(3)
    return tuple(_ext.ext().nvfp4_quantize(w.contiguous(), bool(hadamard)))


def nvfp4_dequant(packed, scales, tscale):
    _tick()
    return _ext.ext().nvfp4_dequant(packed, scales, tscale)


def fwht16(x: torch.Tensor) -> torch.Tensor:
    _tick()
    return _ext.ext().fwht16(x.contiguous())


def nvfp4_linear(x2, packed, scales, tscale, out_dtype):
    """Decode (M <= 8): GEMV straight from the packed weights. Prefill: decode the weights to bf16 once per call
    (4.5 -> 16 bits, a small fraction of the GEMM's traffic at large M) and run the tcgen05 GEMM."""
    from . import gemm

    e = _ext.ext()
    x2 = x2.contiguous()
    if x2.shape[0] <= 8:
        _tick()
        y = e.nvfp4_gemv(x2, packed, scales, tscale)
    else:
        y = gemm(x2, nvfp4_dequant(packed, scales, tscale))
    return y if out_dtype == torch.bfloat16 else y.to(out_dtype)


def nvfp4_block_scales(scales: torch.Tensor, K: int) -> torch.Tensor:
    """Row-major E4M3 block scales [N, K/16] -> the blocked layout the tensor-core GEMM loads."""
    _tick()
    return _ext.ext().nvfp4_block_scales(scales.contiguous().view(torch.uint8), int(K))


def nvfp4_quantize_act(x2: torch.Tensor, hadamard: bool = False):
    """bf16 [M, K] -> (packed E2M1 [M, K/2], blocked unsigned-E4M3 scales); optional folded 16-point Hadamard rotation."""
    _tick()
    return tuple(_ext.ext().nvfp4_quantize_act(x2, bool(hadamard)))


last_gemm_status = None


def _bias16(bias):
    """The GEMM epilogue adds a contiguous bf16 bias; anything else is converted once per call (tiny)."""
    if bias is None:
        return None
    b = bias.detach()
    return b if (b.dtype == torch.bfloat16 and b.is_contiguous() and b.data_ptr() % 16 == 0) else b.to(torch.bfloat16).contiguous().clone()


def nvfp4_w4a4_linear(x2, packed, sf_blocked, alpha: float, hadamard: bool, out_dtype, bias=None, gelu: bool = False):
    """y = alpha * dequant(quant(x)) @ dequant(W)^T with both operands E2M1 and both scale sets applied by the tensor
    core (``tcgen05.mma.kind::mxf4nvf4``); nothing is decoded to bf16."""
    global last_gemm_status
    e = _ext.ext()
    x2 = x2 if (x2.stride(1) == 1 and x2.stride(0) % 8 == 0 and x2.data_ptr() % 16 == 0) else x2.contiguous()
    a_p, a_sf = e.nvfp4_quantize_act(x2, bool(hadamard))
    y, last_gemm_status = e.nvfp4_gemm(a_p, a_sf, packed, sf_blocked, float(alpha), 0, _bias16(bias), bool(gelu))
    _tick(2)
    return y if out_dtype == torch.bfloat16 else y.to(out_dtype)


def mxfp8_supported(x2, K: int, N: int) -> bool:
    return _ext.use_kernels(x2) and x2.dtype == torch.bfloat16 and K % 32 == 0 and N % 8 == 0


def mxfp8_quantize(x2: torch.Tensor):
    """bf16 [R, K] -> (E4M3 [R, K], blocked power-of-two scales per 32 elements) for the block-scaled FP8 GEMM."""
    _tick()
    x2 = x2 if (x2.stride(1) == 1 and x2.stride(0) % 8 == 0 and x2.data_ptr() % 16 == 0) else x2.contiguous()
    return tuple(_ext.ext().mxfp8_quantize(x2))


def mxfp8_gemm(a, sfa, b, sfb, alpha: float = 1.0, tile_n: int = 0, bias=None, gelu: bool = False):
    global last_gemm_status
    _tick()
    y, last_gemm_status = _ext.ext().mxfp8_gemm(a, sfa, b, sfb, float(alpha), int(tile_n), _bias16(bias), bool(gelu))
    return y


def mxfp8_linear(x2, wq, w_sf, out_dtype, bias=None, gelu: bool = False):
    """y = dequant(quant(x)) @ dequant(W)^T, both E4M3 with 1x32 power-of-two scales applied by the tensor core
    (``tcgen05.mma.kind::mxf8f6f4.block_scale``): no promotion of partial sums out of TMEM per K block."""
    xq, x_sf = mxfp8_quantize(x2)
    y = mxfp8_gemm(xq, x_sf, wq, w_sf, bias=bias, gelu=gelu)  # bias and tanh-GELU ride in the GEMM epilogue
    return y if out_dtype == torch.bfloat16 else y.to(out_dtype)
