"""Dispatch of the quantised GEMMs to the sm_100a kernels."""

from __future__ import annotations

import torch

from .. import _ext


def fp8_supported(x2, wq) -> bool:
    return _ext.use_kernels(x2, wq) and hasattr(_ext.ext(), "fp8_block_gemm") and x2.dtype == torch.bfloat16 \
        and x2.shape[1] % 128 == 0 and wq.shape[0] % 8 == 0


def fp8_block_linear(x2, wq, ws, block, out_dtype):
    e = _ext.ext()
    xq, xs = e.fp8_quantize_act(x2.contiguous())
    return e.fp8_block_gemm(xq, xs, wq, ws).to(out_dtype)


def nvfp4_supported(x2, packed) -> bool:
    return _ext.use_kernels(x2, packed) and hasattr(_ext.ext(), "nvfp4_dequant") and x2.dtype == torch.bfloat16 \
        and packed.shape[0] % 8 == 0


def nvfp4_linear(x2, packed, scales, tscale, out_dtype):
    from . import gemm

    e = _ext.ext()
    w = e.nvfp4_dequant(packed, scales, tscale)  # bf16 [N, K], decoded by the dequant kernel
    return gemm(x2.contiguous(), w).to(out_dtype)
