"""Operator API.

Each op has one meaning and two executors: the sm_100a kernels of ``triune_b200._C`` for CUDA bf16
tensors, and the PyTorch statements in :mod:`triune_b200.ops.reference` for CPU tensors (and as test
oracles). There is no silent fall-back on a GPU: a CUDA tensor without the built extension raises.

Parity: this is the role of the reference's ``triune/ops/__init__.py:1-84`` facade and
``triune/kernels/__init__.py:10-68``; the autograd functions below replace
``triune/kernels/fast_rmsnorm.py``, ``fast_rope.py``, ``fast_swiglu.py``, ``fast_cross_entropy.py``,
``fast_gla.py`` and the expert GEMM path of ``triune/model/moe.py:385-437``.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .. import _ext
from . import reference as ref

GEMM_DENSE, GEMM_GROUPED_M, GEMM_GROUPED_K = 0, 1, 2
GF_OUT_F32, GF_ACCUMULATE, GF_GELU, GF_DGELU, GF_PAIRED_GROUPS, GF_ADDAUX = 1, 2, 4, 8, 16, 128

# kernel launch accounting (used by bench.py's ``gpu_launches``)
_LAUNCHES = {"count": 0}


def launch_count() -> int:
    return _LAUNCHES["count"]


def reset_launch_count() -> None:
    _LAUNCHES["count"] = 0


def _tick(n: int = 1) -> None:
    _LAUNCHES["count"] += n


# ----------------------------------------------------------------------------
# GEMM
# ----------------------------------------------------------------------------
def _tma_ok(t: torch.Tensor) -> bool:
    return (
        t.is_cuda
        and t.dtype == torch.bfloat16
        and t.stride(-1) == 1
        and t.stride(-2) % 8 == 0
        and t.data_ptr() % 16 == 0
        and (t.dim() == 2 or (t.dim() == 3 and t.stride(0) % 8 == 0))
    )


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    out: Optional[torch.Tensor] = None,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: Optional[torch.Tensor] = None,
    gelu: bool = False,
    aux_out: Optional[torch.Tensor] = None,
    dgelu_aux: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    alpha: float = 1.0,
    out_dtype: torch.dtype = torch.bfloat16,
    row_scale: Optional[torch.Tensor] = None,
    mode: int = GEMM_DENSE,
    tile_group: Optional[torch.Tensor] = None,
    group_offsets: Optional[torch.Tensor] = None,
    num_groups: int = 0,
    paired_groups: bool = False,
    add_aux: Optional[torch.Tensor] = None,
    beta: float = 1.0,
    k_runs: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """out = alpha * A @ B^T with a fused epilogue, on tcgen05 tensor cores.

    ``a`` is [.., M, K] (``a_mn``: stored [.., K, M]); ``b`` is [.., N, K] (``b_mn``: stored [.., K, N]).
    ``mode``: dense/batched, rows grouped by expert (``tile_group``), or reduction grouped by expert
    (``group_offsets``; then ``a`` [R, M], ``b`` [R, N] and out is [G, M, N]).
    ``gelu`` applies tanh-GELU after the bias; ``aux_out`` (bf16, out's layout) then receives GELU'(pre-activation),
    which a later call takes as ``dgelu_aux`` to form ``out = alpha * (A @ B^T) * dgelu_aux`` in its epilogue.
    ``add_aux`` (bf16, out's layout) forms ``out = alpha * A @ B^T + beta * add_aux`` in the epilogue.
    ``paired_groups`` (rows grouped by expert only) promises that every expert's rows are padded to a multiple of 256,
    which lets long reductions run on CTA pairs.
    ``k_runs`` (reduction grouped by expert only; int32 [runs, 2] = first row, number of 64-row blocks): the rows each
    group reduces over as a list of runs, ``group_offsets`` then indexing runs instead of rows, so partly filled
    segments of a fixed-capacity buffer cost only the blocks that hold rows.
    """
    assert _tma_ok(a) and _tma_ok(b), "gemm operands must be CUDA bf16 with 16-byte aligned rows"
    if mode == GEMM_GROUPED_K:
        M, N = a.shape[-1], b.shape[-1]
        shape = (num_groups, M, N)
    else:
        M = a.shape[-1] if a_mn else a.shape[-2]
        N = b.shape[-1] if b_mn else b.shape[-2]
        batch = a.shape[0] if a.dim() == 3 else (b.shape[0] if (b.dim() == 3 and mode == GEMM_DENSE) else None)
        shape = (M, N) if batch is None else (batch, M, N)
    if out is None:
        out = torch.empty(shape, device=a.device, dtype=out_dtype)
    flags = (GF_ACCUMULATE if accumulate else 0) | (GF_GELU if gelu else 0) | (GF_DGELU if dgelu_aux is not None else 0)
    if paired_groups and mode == GEMM_GROUPED_M:
        flags |= GF_PAIRED_GROUPS
    aux_in = dgelu_aux
    if add_aux is not None:
        assert dgelu_aux is None and not gelu and not accumulate and out_dtype == torch.bfloat16
        flags |= GF_ADDAUX
        aux_in = add_aux
    _ext.ext().tc_gemm(
        a, b, out, a_mn, b_mn, mode, flags, float(alpha), bias, aux_in, aux_out, row_scale, tile_group,
        group_offsets, None, float(beta), k_runs,
    )
    _tick()
    return out


def _accumulate_weight_grad(w: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor, alpha: float = 1.0):
    """dW = alpha * dy^T x. Accumulates into ``w.main_grad`` (fp32) when the parameter has one, else returns bf16."""
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        gemm(dy2, x2, mg, a_mn=True, b_mn=True, accumulate=True, alpha=alpha)
        return None
    return gemm(dy2, x2, a_mn=True, b_mn=True, alpha=alpha)


def _accumulate_bias_grad(b: Optional[torch.Tensor], dy2: torch.Tensor):
    if b is None:
        return None
    mg = getattr(b, "main_grad", None)
    fast = _tma_ok(dy2) and dy2.dim() == 2 and dy2.shape[1] % 8 == 0 and _ext.use_kernels(dy2)
    if mg is not None:
        if fast and mg.dtype == torch.float32 and mg.is_contiguous():
            _ext.ext().colsum(dy2, mg)  # column sums added into the fp32 gradient arena
            _tick(2)
        else:
            mg.add_(dy2.sum(0, dtype=torch.float32))
        return None
    if fast:
        db = _ext.ext().colsum(dy2, None)
        _tick(2)
        return db.to(b.dtype)
    return dy2.sum(0, dtype=torch.float32).to(b.dtype)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, alpha=1.0):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if not _tma_ok(x2):
            x2 = x2.contiguous()
        y = gemm(x2, w, bias=bias, alpha=alpha)  # alpha scales the product, not the bias
        ctx.save_for_backward(x2, w, bias if bias is not None else torch.empty(0))
        ctx.has_bias = bias is not None
        ctx.in_shape = x.shape
        ctx.alpha = float(alpha)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, bias = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.shape[0])
        if not _tma_ok(dy2):
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True, alpha=ctx.alpha).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            dw = _accumulate_weight_grad(w, dy2, x2, ctx.alpha)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _accumulate_bias_grad(bias, dy2)
        return dx, dw, db, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, alpha: float = 1.0) -> torch.Tensor:
    """y = alpha * x @ w^T + bias (the scale rides in the GEMM epilogues of the forward and both gradients)."""
    if _ext.use_kernels(x, w) and x.dtype == torch.bfloat16 and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0:
        return _LinearFn.apply(x, w, bias, alpha)
    if alpha != 1.0:
        y = F.linear(x, w) * alpha
        return y if bias is None else y + bias
    return F.linear(x, w, bias)


class _MLPFn(torch.autograd.Function):
    """Linear -> GELU(tanh) -> Linear with the activation and its derivative fused into GEMM epilogues."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if not _tma_ok(x2):
            x2 = x2.contiguous()
        M, Hd = x2.shape[0], w1.shape[0]
        dact = torch.empty(M, Hd, device=x.device, dtype=x.dtype)  # GELU'(x w1^T + b1), written by the same epilogue
        h = gemm(x2, w1, bias=b1, gelu=True, aux_out=dact)
        y = gemm(h, w2, bias=b2)
        ctx.save_for_backward(x2, w1, b1, w2, b2, dact, h)
        ctx.in_shape = x.shape
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, b1, w2, b2, dact, h = ctx.saved_tensors
        dy2 = dy.reshape(-1, w2.shape[0])
        if not _tma_ok(dy2):
            dy2 = dy2.contiguous()
        dpre = gemm(dy2, w2, b_mn=True, dgelu_aux=dact)
        dw2 = _accumulate_weight_grad(w2, dy2, h)
        db2 = _accumulate_bias_grad(b2, dy2)
        dx = gemm(dpre, w1, b_mn=True).view(ctx.in_shape) if ctx.needs_input_grad[0] else None
        dw1 = _accumulate_weight_grad(w1, dpre, x2)
        db1 = _accumulate_bias_grad(b1, dpre)
        return dx, dw1, db1, dw2, db2


def _wants_grad(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


def mlp_gelu(x, w1, b1, w2, b2):
    """Dense FFN: gelu_tanh(x w1^T + b1) w2^T + b2."""
    if _ext.use_kernels(x, w1, w2) and x.dtype == torch.bfloat16 and b1 is not None and b2 is not None:
        if not _wants_grad(x, w1, b1, w2, b2):
            # inference: the GELU epilogue skips the derivative tile (half the bytes written by the first GEMM)
            K = x.shape[-1]
            x2 = x.reshape(-1, K)
            if not _tma_ok(x2):
                x2 = x2.contiguous()
            return gemm(gemm(x2, w1, bias=b1, gelu=True), w2, bias=b2).view(*x.shape[:-1], w2.shape[0])
        return _MLPFn.apply(x, w1, b1, w2, b2)
    return F.linear(ref.gelu_tanh(F.linear(x, w1, b1)), w2, b2)


def gelu_tanh(x):
    return ref.gelu_tanh(x)


class _SwiGLUFn(torch.autograd.Function):
    """silu(gate) * up for separate [.., width] tensors (either may be a column slice of a wider matrix)."""

    @staticmethod
    def forward(ctx, gate, up):
        w = gate.shape[-1]
        g2, u2 = gate.reshape(-1, w), up.reshape(-1, w)
        ctx.save_for_backward(g2, u2)
        ctx.shape = gate.shape
        out = _ext.ext().swiglu_fwd(g2, u2)
        _tick()
        return out.view(gate.shape)

    @staticmethod
    def backward(ctx, dh):
        g2, u2 = ctx.saved_tensors
        d2 = dh.reshape(-1, g2.shape[-1])
        if not _rows_ok(d2):
            d2 = d2.contiguous()
        dg, du, _ = _ext.ext().swiglu_bwd(g2, u2, d2)
        _tick()
        return dg.view(ctx.shape), du.view(ctx.shape)


def _rows_ok(t: torch.Tensor) -> bool:
    return (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


def swiglu(gate, up):
    """silu(gate) * up (``triune/kernels/fast_swiglu.py:19-45``)."""
    if (_ext.use_kernels(gate, up) and gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16
            and gate.shape == up.shape and gate.shape[-1] % 8 == 0
            and _rows_ok(gate.reshape(-1, gate.shape[-1])) and _rows_ok(up.reshape(-1, up.shape[-1]))):
        return _SwiGLUFn.apply(gate, up)
    return ref.swiglu(gate, up)


class _SwiGLUMLPFn(torch.autograd.Function):
    """down( silu(x Wg^T) * (x Wu^T) ) with w13 = [Wg ; Wu] ([2H, d]) and w2 = [d, H].

    Forward: ONE GEMM over the fused weight whose epilogue forms silu(gate) * up from the two halves of its accumulator
    tile (the [M, 2H] pre-activations go out once, for the backward pass), then the down projection. Backward: the GEMM
    that forms d(hidden) = dy w2 applies the SwiGLU derivative in its epilogue and writes d(gate | up) directly, which
    feeds the input-gradient and weight-gradient GEMMs of the fused weight. No stand-alone elementwise pass remains."""

    @staticmethod
    def forward(ctx, x, w13, w2):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if not _tma_ok(x2):
            x2 = x2.contiguous()
        M, H = x2.shape[0], w13.shape[0] // 2
        train = any(ctx.needs_input_grad)  # (grad mode is off inside forward: ask the context, not torch)
        h = torch.empty(M, H, device=x.device, dtype=x.dtype)
        gu = torch.empty(M, 2 * H, device=x.device, dtype=x.dtype) if train else None
        _ext.ext().tc_gemm_swiglu(x2, w13, h, gu)
        _tick()
        y = gemm(h, w2)
        if train:
            ctx.save_for_backward(x2, w13, w2, gu, h)
        ctx.in_shape = x.shape
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w13, w2, gu, h = ctx.saved_tensors
        dy2 = dy.reshape(-1, w2.shape[0])
        if not _tma_ok(dy2):
            dy2 = dy2.contiguous()
        dgu = torch.empty_like(gu)
        _ext.ext().tc_gemm_dswiglu(dy2, w2, True, gu, dgu)   # d(hidden) = dy @ w2, w2 stored [d, H] = [K, N]
        _tick()
        dw2 = _accumulate_weight_grad(w2, dy2, h)
        dx = gemm(dgu, w13, b_mn=True).view(ctx.in_shape) if ctx.needs_input_grad[0] else None
        dw13 = _accumulate_weight_grad(w13, dgu, x2)
        return dx, dw13, dw2


def swiglu_mlp(x, w13, w2):
    """SwiGLU feed-forward over a fused gate/up weight: ``down(silu(x Wg^T) * (x Wu^T))``."""
    H = w13.shape[0] // 2
    if (_ext.use_kernels(x, w13, w2) and x.dtype == torch.bfloat16 and H % 32 == 0 and w13.shape[1] % 8 == 0
            and w2.shape[0] % 8 == 0 and w13.is_contiguous() and w2.is_contiguous()):
        return _SwiGLUMLPFn.apply(x, w13, w2)
    gu = F.linear(x, w13)
    return F.linear(ref.swiglu(gu[..., :H], gu[..., H:]), w2)


# ----------------------------------------------------------------------------
# RMSNorm
# ----------------------------------------------------------------------------
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        xc = x.contiguous()
        y, rstd, _ = _ext.ext().rmsnorm_fwd(xc, None, w, eps)
        _tick()
        ctx.save_for_backward(xc, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx, dw = _ext.ext().rmsnorm_bwd(x, w, dy, rstd, None)
        _tick()
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            mg.add_(dw)
            dw = None
        else:
            dw = dw.to(w.dtype)
        return dx, dw, None


class _AddRMSNormFn(torch.autograd.Function):
    """(y, s) = (rmsnorm(x + r), x + r); one pass over x and r."""

    @staticmethod
    def forward(ctx, x, r, w, eps):
        y, rstd, s = _ext.ext().rmsnorm_fwd(x.contiguous(), r.contiguous(), w, eps)
        _tick()
        ctx.save_for_backward(s, w, rstd)
        return y, s

    @staticmethod
    def backward(ctx, dy, ds):
        s, w, rstd = ctx.saved_tensors
        if dy is None:
            dy = torch.zeros_like(s)
        dx, dw = _ext.ext().rmsnorm_bwd(s, w, dy, rstd, ds)
        _tick()
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            mg.add_(dw)
            dw = None
        else:
            dw = dw.to(w.dtype)
        return dx, dx, dw, None


def _norm_kernel_ok(x, w):
    return (
        _ext.use_kernels(x, w)
        and x.dtype == torch.bfloat16
        and w.dtype == torch.bfloat16
        and x.shape[-1] % 8 == 0
        and x.shape[-1] <= 2048
    )


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if _norm_kernel_ok(x, w):
        return _RMSNormFn.apply(x, w, eps)
    return ref.rmsnorm(x, w, eps)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float = 1e-6):
    """Returns (rmsnorm(x + residual), x + residual)."""
    if _norm_kernel_ok(x, w) and residual.is_cuda:
        return _AddRMSNormFn.apply(x, residual, w, eps)
    return ref.add_rmsnorm(x, residual, w, eps)


# ----------------------------------------------------------------------------
# RoPE + GLA feature map
# ----------------------------------------------------------------------------
def rope_tables(seq_len, head_dim, base=10000.0, offset=0, device=None):
    return ref.rope_tables(seq_len, head_dim, base, offset, device)


class _RoPEFn(torch.autograd.Function):
    """Half-split rotation of [B, T, H, D] by [T, D/2] tables; the gradient is the inverse rotation."""

    @staticmethod
    def forward(ctx, x, cos_half, sin_half):
        B, T, H, D = x.shape
        x2 = x.reshape(B * T, H * D)
        if not _rows_ok(x2):
            x2 = x2.contiguous()
        y = _ext.ext().rope_apply(x2, cos_half, sin_half, T, H, D, False)
        _tick()
        ctx.save_for_backward(cos_half, sin_half)
        ctx.dims = (B, T, H, D)
        return y.view(B, T, H, D)

    @staticmethod
    def backward(ctx, dy):
        cos_half, sin_half = ctx.saved_tensors
        B, T, H, D = ctx.dims
        d2 = dy.reshape(B * T, H * D)
        if not _rows_ok(d2):
            d2 = d2.contiguous()
        dx = _ext.ext().rope_apply(d2, cos_half, sin_half, T, H, D, True)
        _tick()
        return dx.view(B, T, H, D), None, None


def apply_rope(x, cos, sin):
    """Rotary embedding of ``x [B, T, H, D]`` with ``cos/sin [T, D]`` tables in the half-split convention
    (``triune/kernels/fast_rope.py:16-80``)."""
    if (_ext.use_kernels(x) and x.dtype == torch.bfloat16 and x.dim() == 4 and x.shape[-1] % 16 == 0
            and cos.shape[0] == x.shape[1] and cos.shape[-1] == x.shape[-1]):
        D = x.shape[-1]
        ch = cos[:, : D // 2].float().contiguous()
        sh = sin[:, : D // 2].float().contiguous()
        return _RoPEFn.apply(x, ch, sh)
    return ref.apply_rope(x, cos, sin)


class _EmbeddingFn(torch.autograd.Function):
    """Row gather whose gradient is scattered straight into the fp32 gradient arena (``weight.main_grad``): no dense
    [V, d] bf16 gradient, no sort, no second pass to fold it into the arena."""

    @staticmethod
    def forward(ctx, ids, weight):
        flat = ids.reshape(-1).contiguous()
        ctx.save_for_backward(flat, weight)
        return F.embedding(ids, weight)

    @staticmethod
    def backward(ctx, dy):
        flat, weight = ctx.saved_tensors
        d = weight.shape[1]
        dy2 = dy.reshape(-1, d)
        if dy2.dtype != torch.bfloat16 or dy2.stride(1) != 1 or dy2.stride(0) % 4 != 0:
            dy2 = dy2.to(torch.bfloat16).contiguous()
        mg = getattr(weight, "main_grad", None)
        if mg is not None and mg.is_contiguous() and mg.dtype == torch.float32 and mg.data_ptr() % 16 == 0:
            _ext.ext().embedding_bwd(dy2, flat, mg)
            _tick()
            return None, None
        g = torch.zeros(weight.shape, device=weight.device, dtype=torch.float32)
        _ext.ext().embedding_bwd(dy2, flat, g)
        _tick()
        return None, g.to(weight.dtype)


def embedding(ids, weight):
    """``weight[ids]``; on the kernel path the gradient is a scatter-add into the fp32 arena."""
    if (_ext.use_kernels(weight) and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0
            and ids.is_cuda and ids.dtype == torch.int64 and _wants_grad(weight)):
        return _EmbeddingFn.apply(ids, weight)
    return F.embedding(ids, weight)


class _QKPrepFn(torch.autograd.Function):
    """qkvg [tokens, 4*H*D] -> (q~, k~) = rope(normalize(elu(.)+1)); reads the q and k column blocks in place."""

    @staticmethod
    def forward(ctx, qkvg, cos_half, sin_half, T, H, D):
        out = _ext.ext().qk_prep_fwd(qkvg, H * D, cos_half, sin_half, T, H, D)
        _tick()
        ctx.save_for_backward(qkvg, cos_half if cos_half is not None else torch.empty(0),
                              sin_half if sin_half is not None else torch.empty(0))
        ctx.dims = (T, H, D, cos_half is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkvg, cs, sn = ctx.saved_tensors
        T, H, D, has_rope = ctx.dims
        d_in = torch.zeros_like(qkvg)
        _ext.ext().qk_prep_bwd(qkvg, H * D, dout.contiguous(), d_in, cs if has_rope else None,
                               sn if has_rope else None, T, H, D)
        _tick()
        return d_in, None, None, None, None, None


def qk_feature_map(qkvg: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], B: int, T: int,
                   H: int, D: int):
    """From the fused projection output [B*T, 4*H*D] return (q~, k~, v, g_logits), each [B, T, H, D].

    q~, k~ are feature-mapped, normalised and rotated; v and the raw gate logits are strided views of
    the projection output (no copy). cos/sin are [T, D] tables (half-split convention).
    """
    HD = H * D
    if _ext.use_kernels(qkvg) and qkvg.dtype == torch.bfloat16 and D in (64, 128):
        ch = cos[:, : D // 2].float().contiguous() if cos is not None else None
        sh = sin[:, : D // 2].float().contiguous() if sin is not None else None
        qk = _QKPrepFn.apply(qkvg, ch, sh, T, H, D)  # [tokens, 2, H, D]
        qk = qk.view(B, T, 2, H, D)
        q, k = qk[:, :, 0], qk[:, :, 1]
    else:
        qr = qkvg[:, :HD].reshape(B, T, H, D)
        kr = qkvg[:, HD : 2 * HD].reshape(B, T, H, D)
        qf = F.normalize(F.elu(qr.float()) + 1.0, p=2.0, dim=-1, eps=1e-6)
        kf = F.normalize(F.elu(kr.float()) + 1.0, p=2.0, dim=-1, eps=1e-6)
        if cos is not None:
            qf = ref.apply_rope(qf, cos.float(), sin.float())
            kf = ref.apply_rope(kf, cos.float(), sin.float())
        q, k = qf.to(qkvg.dtype), kf.to(qkvg.dtype)
    v = qkvg[:, 2 * HD : 3 * HD].view(B, T, H, D)
    g = qkvg[:, 3 * HD :].view(B, T, H, D)
    return q, k, v, g


# ----------------------------------------------------------------------------
# GLA / Gated DeltaNet
# ----------------------------------------------------------------------------
def gla(q, k, v, g, initial_state=None, scale: float = 1.0, gate_logits: bool = False, chunk_size: int = 64):
    """Gated linear attention over [B,T,H,D] tensors; returns (out [B,T,H,Dv], final_state [B,H,Dk,Dv] fp32).

    ``g`` is the per-dimension log decay (<= 0), or the raw gate logits when ``gate_logits`` (then
    log-sigmoid is applied in fp32 inside the op, avoiding a bf16 round trip of the decays).
    """
    from . import gla_cuda

    if gla_cuda.supported(q, k, v, g, initial_state):
        return gla_cuda.gla_chunk(q, k, v, g, initial_state, scale, gate_logits)
    gl = F.logsigmoid(g.float()) if gate_logits else g
    if q.shape[1] == 1 and initial_state is not None and not torch.is_grad_enabled():
        o, s = ref.gla_decode_step(q[:, 0], k[:, 0], v[:, 0], gl[:, 0], initial_state, scale)
        return o.unsqueeze(1), s
    return ref.gla_chunk(q, k, v, gl, initial_state, scale, chunk_size)


def gla_recurrent(q, k, v, g, initial_state=None, scale: float = 1.0):
    return ref.gla_recurrent(q, k, v, g, initial_state, scale)


class _FinalStateGradFn(torch.autograd.Function):
    """Attaches the gradient of a GLA final state to a state that was computed without one.

    S_T = sum_t diag(e^{R_t}) k_t v_t^T + diag(e^{R_0'}) S_0 with R_t = sum_{s>t} g_s (the decay from token t to the end)
    and R_0' = sum_s g_s. For an incoming gradient G = dL/dS_T:

        dk_t = e^{R_t} * (G v_t)        dv_t = G^T (e^{R_t} * k_t)        dS_0 = diag(e^{R_0'}) G
        dg_s = sum_{t<s} k_t * dk_t  +  e^{R_0'} * rowsum(S_0 * G)

    which is two batched products and two cumulative sums over the sequence: small next to the attention itself.
    """

    @staticmethod
    def forward(ctx, k, v, gl, s0, s_final):
        ctx.save_for_backward(k, v, gl, s0 if s0 is not None else torch.empty(0, device=k.device))
        ctx.has_s0 = s0 is not None
        return s_final.detach().clone()

    @staticmethod
    def backward(ctx, G):
        k, v, gl, s0 = ctx.saved_tensors
        dt = torch.float64 if gl.dtype == torch.float64 else torch.float32
        G, kf, vf = G.to(dt), k.to(dt), v.to(dt)
        bcum = torch.cumsum(gl.to(dt), dim=1)                      # [B, T, H, Dk]
        w = torch.exp(bcum[:, -1:] - bcum)                           # e^{R_t}
        dk = w * torch.einsum("bhkv,bthv->bthk", G, vf)
        dv = torch.einsum("bhkv,bthk->bthv", G, w * kf)
        c = kf * dk
        dg = torch.cumsum(c, dim=1) - c                              # exclusive prefix sum over t < s
        ds0 = None
        if ctx.has_s0:
            tot = torch.exp(bcum[:, -1])                             # [B, H, Dk]
            ds0 = (tot.unsqueeze(-1) * G).to(s0.dtype)
            dg = dg + (tot * (s0.to(dt) * G).sum(-1)).unsqueeze(1)
        return dk.to(k.dtype), dv.to(v.dtype), dg.to(gl.dtype), ds0, None


def gla_final_state_with_grad(k, v, log_decay, initial_state, final_state):
    """``final_state`` (as returned by the kernels, which carry no gradient for it) with its dependence on ``k``, ``v``,
    the per-step log decay ``[B, T, H, Dk]`` (already clamped the way the kernel clamps it) and ``initial_state``
    restored for autograd. Used where the state itself is trained through: context parallelism, truncated
    back-propagation across segments."""
    return _FinalStateGradFn.apply(k, v, log_decay, initial_state, final_state)


def gated_deltanet(q, k, v, g, beta=None, initial_state=None, scale: float = 1.0, gate_logits: bool = False,
                   chunk_size: int = 64):
    """Gated DeltaNet over [B,T,H,D] tensors; returns (out, final_state [B,H,Dk,Dv]).

    Without gradients (prefill, decode) CUDA bf16 inputs run the exact token recurrence in one kernel; with gradients
    they run the chunk-parallel tcgen05 kernels (UT transform per chunk, sequential state pass, chunk outputs, and the
    stage-wise backward of ``csrc/gla/gdn_chunk_kernels.cu``). Other inputs (CPU, fp32, a per-key-row beta) use the
    differentiable PyTorch forms of :mod:`triune_b200.ops.reference`."""
    from . import gla_cuda

    if gla_cuda.gdn_supported(q, k, v, g, beta):
        return gla_cuda.gdn_recurrent(q, k, v, g, beta, initial_state, scale, gate_logits)
    if gla_cuda.gdn_chunk_supported(q, k, v, g, beta) and q.shape[1] > 1:
        return gla_cuda.gdn_chunk(q, k, v, g, beta, initial_state, scale, gate_logits)
    gl = F.logsigmoid(g.float()) if gate_logits else g
    if q.shape[1] == 1 and initial_state is not None and not torch.is_grad_enabled():
        o, s = ref.gated_deltanet_decode_step(
            q[:, 0], k[:, 0], v[:, 0], gl[:, 0], initial_state, None if beta is None else beta[:, 0], scale
        )
        return o.unsqueeze(1), s
    return ref.gated_deltanet_chunk_parallel(q, k, v, gl, beta, initial_state, scale, chunk_size)


# ----------------------------------------------------------------------------
# Cross entropy
# ----------------------------------------------------------------------------
class _CrossEntropyFn(torch.autograd.Function):
    """Mean cross entropy over bf16 logits: one kernel computes the per-row loss and (softmax - onehot) / n_valid into a
    separate buffer (the logits stay intact); backward scales that buffer by the incoming scalar."""

    @staticmethod
    def forward(ctx, logits, targets, ignore_index, n_valid):
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V)
        if not _rows_ok(l2):
            l2 = l2.contiguous()
        t = targets.reshape(-1).contiguous()
        need = ctx.needs_input_grad[0]
        inv = 1.0 / float(n_valid)
        losses, grad = _ext.ext().ce_loss_grad(l2, t, ignore_index, inv if need else 0.0)
        _tick()
        if need:
            ctx.save_for_backward(grad)
        ctx.shape = logits.shape
        return losses.sum() * inv

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return (grad * g.to(grad.dtype)).view(ctx.shape), None, None, None


def cross_entropy(logits, targets, ignore_index: int = -100, n_valid: Optional[int] = None):
    """Mean CE over the non-ignored rows (``triune/kernels/fast_cross_entropy.py:20-108``). ``n_valid`` (their count)
    avoids a host synchronisation."""
    if _ext.use_kernels(logits) and logits.dtype == torch.bfloat16 and logits.shape[-1] % 8 == 0 and targets.is_cuda:
        if n_valid is None:
            n_valid = max(1, int((targets != ignore_index).sum().item()))
        return _CrossEntropyFn.apply(logits, targets.long(), ignore_index, n_valid)
    return ref.cross_entropy(logits, targets, ignore_index)


class _LinearCEFn(torch.autograd.Function):
    """Head GEMM + cross entropy in row chunks; the [N,V] logits never exist in full.

    For each chunk: logits = h W^T (+b) on tensor cores, one kernel turns them into the loss and, in
    place, into d(logits); two more GEMMs fold that into dh and dW. Gradients are therefore complete
    at the end of forward; backward only scales them by the incoming scalar.
    """

    @staticmethod
    def forward(ctx, h, w, bias, targets, ignore_index, n_valid, chunk_rows):
        d = h.shape[-1]
        h2 = h.reshape(-1, d)
        if not _tma_ok(h2):
            h2 = h2.contiguous()
        t = targets.reshape(-1).contiguous()
        N, V = h2.shape[0], w.shape[0]
        need_grad = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        inv = 1.0 / float(n_valid)
        losses = torch.empty(N, device=h.device, dtype=torch.float32)
        dh = torch.empty_like(h2) if need_grad else None
        dw = torch.empty(V, d, device=h.device, dtype=torch.float32) if need_grad else None
        db = torch.zeros(V, device=h.device, dtype=torch.float32) if (need_grad and bias is not None) else None
        e = _ext.ext()
        first = True
        for s in range(0, N, chunk_rows):
            hc = h2[s : s + chunk_rows]
            logits = gemm(hc, w, bias=bias)
            losses[s : s + chunk_rows] = e.ce_fwd_bwd(logits, t[s : s + chunk_rows], ignore_index,
                                                      inv if need_grad else 0.0)
            _tick()
            if need_grad:
                gemm(logits, w, dh[s : s + chunk_rows], b_mn=True)
                gemm(logits, hc, dw, a_mn=True, b_mn=True, accumulate=not first)
                if db is not None:
                    e.colsum(logits, db)  # column sums added into the fp32 bias gradient (two-phase kernel)
                    _tick(2)
                first = False
        loss = losses.sum() * inv
        if need_grad:
            ctx.save_for_backward(dh, dw, db if db is not None else torch.empty(0), w,
                                  bias if bias is not None else torch.empty(0))
        ctx.in_shape = h.shape
        ctx.has_bias = bias is not None
        return loss

    @staticmethod
    def backward(ctx, g):
        dh, dw, db, w, bias = ctx.saved_tensors
        dh_out = (dh * g.to(dh.dtype)).view(ctx.in_shape)
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            mg.add_(dw * g)
            dw_out = None
        else:
            dw_out = (dw * g).to(w.dtype)
        db_out = None
        if ctx.has_bias:
            bmg = getattr(bias, "main_grad", None)
            if bmg is not None:
                bmg.add_(db * g)
            else:
                db_out = (db * g).to(bias.dtype)
        return dh_out, dw_out, db_out, None, None, None, None


def linear_cross_entropy(h, w, targets, bias=None, ignore_index: int = -100, n_valid: Optional[int] = None,
                         chunk_rows: int = 8192):
    """Mean CE of (h @ w^T + bias) against targets. ``n_valid`` (non-ignored count) avoids a host sync."""
    if _ext.use_kernels(h, w) and h.dtype == torch.bfloat16 and w.shape[0] % 8 == 0:
        if n_valid is None:
            n_valid = max(1, int((targets != ignore_index).sum().item()))
        return _LinearCEFn.apply(h, w, bias, targets, ignore_index, n_valid, chunk_rows)
    loss, _ = ref.linear_cross_entropy(h, w, targets, bias, ignore_index)
    return loss


# ----------------------------------------------------------------------------
# Mixture of experts
# ----------------------------------------------------------------------------
def moe_route(logits, expert_bias, top_k, temperature=1.0):
    return ref.moe_route(logits, expert_bias, top_k, temperature)


class _RouteTopKFn(torch.autograd.Function):
    """Top-k routing in one kernel; differentiable in the mixing weights (probabilities recomputed in the backward)."""

    @staticmethod
    def forward(ctx, logits, bias, temperature, top_k):
        t_dev = temperature if torch.is_tensor(temperature) else None
        t_val = 1.0 if t_dev is not None else float(temperature)
        if t_dev is not None:
            t_dev = t_dev.detach().reshape(1).float().contiguous()
        idx, w, keys, counts = _ext.ext().moe_route_topk(logits, bias.float().contiguous(), t_dev, t_val, top_k)
        _tick(2)
        ctx.save_for_backward(logits, idx, w, t_dev if t_dev is not None else torch.empty(0))
        ctx.t_val, ctx.has_t = t_val, t_dev is not None
        ctx.mark_non_differentiable(idx, keys, counts)
        return idx, w, keys, counts

    @staticmethod
    def backward(ctx, _didx, dw, _dkeys, _dcounts):
        logits, idx, w, t_dev = ctx.saved_tensors
        dl = _ext.ext().moe_route_bwd(logits, t_dev if ctx.has_t else None, ctx.t_val, idx, w, dw.float().contiguous())
        _tick()
        return dl, None, None, None


def route_plan_supported(logits, top_k: int) -> bool:
    return (_ext.use_kernels(logits) and logits.dtype == torch.float32 and logits.dim() == 2 and logits.shape[1] <= 64
            and 1 <= top_k <= 4 and top_k <= logits.shape[1])


class RoutePlan(tuple):
    """The dispatch plan of :func:`moe_route_plan`: the 5-tuple of :func:`moe_plan` whose expert row ranges are padded
    to multiples of 256 (``row_pad``), i.e. to whole pairs of 128-row tiles."""

    row_pad = 256
    slot_counts = None  # [E, k] int32: assignments REQUESTED per (expert, k-slot), from the routing kernel


def moe_route_plan(logits, expert_bias, top_k: int, temperature=1.0, capacity: Optional[int] = None):
    """Routing + capacity admission + dispatch plan with ONE sort and three kernels, no host synchronisation.

    Returns ``(idx [N,k] int64, w [N,k] fp32 (differentiable), keep [N,k] bool, plan)`` where ``plan`` is the tuple
    :func:`moe_plan` returns. ``capacity`` (per (k-slot, expert), highest weight first, ties to the lower token index) may
    be ``None`` for no limit."""
    N, E = logits.shape
    idx, w, keys, counts = _RouteTopKFn.apply(logits.contiguous(), expert_bias, temperature, top_k)
    skeys, order = torch.sort(keys, stable=True)
    cap = int(capacity) if capacity is not None and capacity < N else N
    pos, keep, row_src, tile_group, offsets, accepted = _ext.ext().moe_plan_sorted(skeys, order, counts, N, top_k, cap)
    _tick(3)
    plan = RoutePlan((pos, row_src, tile_group, offsets, accepted))
    plan.slot_counts = counts
    return idx, w, keep, plan


def moe_plan(idx: torch.Tensor, keep: Optional[torch.Tensor], num_experts: int, tile: int = 128):
    """Device-side dispatch plan (no host sync).

    idx [N,k] expert ids, keep [N,k] accepted mask (or None). Expert row ranges are padded to multiples of
    ``tile`` inside a buffer of static size R = ceil_tile(N*k) + E*tile. Returns
      pos [N,k] int32          row of each assignment in the expert-major buffer (-1 = dropped)
      row_src [R] int32        source token of each buffer row (-1 = padding)
      tile_group [R/tile] int32 expert of each row tile (-1 = unused)
      group_offsets [E+1] int32 padded row offsets per expert
      counts [E] int64         accepted assignments per expert
    """
    N, k = idx.shape
    E = num_experts
    dev = idx.device
    flat_e = idx.reshape(-1)
    if keep is not None:
        flat_e = torch.where(keep.reshape(-1), flat_e, torch.full_like(flat_e, E))
    order = torch.argsort(flat_e, stable=True)
    counts_all = torch.zeros(E + 1, device=dev, dtype=torch.int64).scatter_add_(0, flat_e, torch.ones_like(flat_e))
    counts = counts_all[:E]
    padded = (counts + tile - 1) // tile * tile
    cum_p = torch.cumsum(padded, 0)
    starts_p = cum_p - padded
    starts = torch.cumsum(counts_all, 0) - counts_all
    e_sorted = flat_e[order]
    rank = torch.arange(N * k, device=dev) - starts[e_sorted]
    valid = e_sorted < E
    starts_p_ext = torch.cat((starts_p, starts_p.new_zeros(1)))
    pos_sorted = torch.where(valid, starts_p_ext[e_sorted] + rank, torch.full_like(rank, -1))
    pos = torch.empty(N * k, device=dev, dtype=torch.int64)
    pos[order] = pos_sorted
    R = ((N * k + tile - 1) // tile) * tile + E * tile
    row_src = torch.full((R + 1,), -1, device=dev, dtype=torch.int64)
    row_src[torch.where(valid, pos_sorted, torch.full_like(pos_sorted, R))] = order // k
    row_src = row_src[:R]
    tile_start = torch.arange(R // tile, device=dev) * tile
    tg = torch.searchsorted(cum_p, tile_start, right=True)
    tile_group = torch.where(tg < E, tg, torch.full_like(tg, -1))
    group_offsets = torch.cat((cum_p.new_zeros(1), cum_p))
    return (
        pos.view(N, k).to(torch.int32),
        row_src.to(torch.int32),
        tile_group.to(torch.int32),
        group_offsets.to(torch.int32),
        counts,
    )


class _GatherRowsFn(torch.autograd.Function):
    """xp[r] = x[row_src[r]] (zero rows for padding). Backward sums the k copies of each token."""

    @staticmethod
    def forward(ctx, x, row_src, pos):
        ctx.save_for_backward(pos)
        out = _ext.ext().gather_rows(x, row_src, None)
        _tick()
        return out

    @staticmethod
    def backward(ctx, dxp):
        (pos,) = ctx.saved_tensors
        dx = _ext.ext().combine_rows(dxp.contiguous(), pos, None, None, 0.0)
        _tick()
        return dx, None, None


class _CombineRowsFn(torch.autograd.Function):
    """out[t] = sum_j w[t,j] * yp[pos[t,j]] (+ add_scale * add[t])."""

    @staticmethod
    def forward(ctx, yp, pos, w, row_src, add, add_scale):
        ctx.save_for_backward(yp, pos, w, row_src)
        ctx.add_scale = add_scale
        ctx.has_add = add is not None
        out = _ext.ext().combine_rows(yp, pos, w, add, add_scale)
        _tick()
        return out

    @staticmethod
    def backward(ctx, dout):
        yp, pos, w, row_src = ctx.saved_tensors
        e = _ext.ext()
        dout = dout.contiguous()
        # per buffer row weight: w of the assignment that owns the row
        R = row_src.shape[0]
        row_w = torch.zeros(R + 1, device=dout.device, dtype=torch.float32)
        p64 = pos.reshape(-1).long()
        row_w[torch.where(p64 >= 0, p64, torch.full_like(p64, R))] = w.reshape(-1)
        dyp = e.gather_rows(dout, row_src, row_w[:R].contiguous())
        dw = e.row_dots(dout, yp, pos)
        _tick(2)
        dadd = dout * ctx.add_scale if ctx.has_add else None
        return dyp, None, dw, None, dadd, None


class _ExpertMLPFn(torch.autograd.Function):
    """Grouped expert FFN on the expert-major buffer: gelu(xp W1[e]^T + b1[e]) W2[e]^T + b2[e]."""

    @staticmethod
    def forward(ctx, xp, w1, b1, w2, b2, tile_group, group_offsets, paired=False):
        R = xp.shape[0]
        ctx.paired = bool(paired) and R % 256 == 0
        Hd = w1.shape[1]
        # Row tiles past the last expert are never written and never read: the combine / gather kernels
        # follow `pos`, and the grouped weight-gradient GEMMs stay inside group_offsets.
        dact = torch.empty(R, Hd, device=xp.device, dtype=xp.dtype)  # GELU' of the pre-activation
        h = torch.empty(R, Hd, device=xp.device, dtype=xp.dtype)
        yp = torch.empty(R, w2.shape[1], device=xp.device, dtype=xp.dtype)
        gemm(xp, w1, h, bias=b1, gelu=True, aux_out=dact, mode=GEMM_GROUPED_M, tile_group=tile_group)
        gemm(h, w2, yp, bias=b2, mode=GEMM_GROUPED_M, tile_group=tile_group, paired_groups=ctx.paired)
        ctx.save_for_backward(xp, w1, b1, w2, b2, dact, h, tile_group, group_offsets)
        return yp

    @staticmethod
    def backward(ctx, dyp):
        xp, w1, b1, w2, b2, dact, h, tile_group, group_offsets = ctx.saved_tensors
        dyp = dyp.contiguous()
        E = w1.shape[0]
        R = xp.shape[0]
        dpre = torch.empty(R, w1.shape[1], device=xp.device, dtype=xp.dtype)
        gemm(dyp, w2, dpre, b_mn=True, dgelu_aux=dact, mode=GEMM_GROUPED_M, tile_group=tile_group)
        dxp = torch.empty_like(xp)
        gemm(dpre, w1, dxp, b_mn=True, mode=GEMM_GROUPED_M, tile_group=tile_group, paired_groups=ctx.paired)
        ones = torch.ones(R, 8, device=xp.device, dtype=xp.dtype)

        def wgrad(w, a, b):
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                gemm(a, b, mg, a_mn=True, b_mn=True, accumulate=True, mode=GEMM_GROUPED_K,
                     group_offsets=group_offsets, num_groups=E)
                return None
            return gemm(a, b, a_mn=True, b_mn=True, mode=GEMM_GROUPED_K, group_offsets=group_offsets, num_groups=E)

        def bgrad(bp, a):
            s = gemm(ones, a, a_mn=True, b_mn=True, mode=GEMM_GROUPED_K, group_offsets=group_offsets, num_groups=E,
                     out_dtype=torch.float32)[:, 0, :]
            mg = getattr(bp, "main_grad", None)
            if mg is not None:
                mg.add_(s)
                return None
            return s.to(bp.dtype)

        dw2 = wgrad(w2, dyp, h)
        db2 = bgrad(b2, dyp)
        dw1 = wgrad(w1, dpre, xp)
        db1 = bgrad(b1, dpre)
        return dxp, dw1, db1, dw2, db2, None, None, None


def moe_experts(x2, idx, weights, keep, w1, b1, w2, b2, shared_out=None, shared_scale: float = 0.0, plan=None):
    """Sparse expert FFN. x2 [N,d]; idx/weights/keep [N,k]; stacked expert weights w1 [E,H,d], b1 [E,H],
    w2 [E,d,H], b2 [E,d]. Returns sum_j w_j * expert_{idx_j}(x) (+ shared_scale * shared_out)."""
    E = w1.shape[0]
    if _ext.use_kernels(x2, w1, w2) and x2.dtype == torch.bfloat16:
        pos, row_src, tile_group, group_offsets, _ = plan if plan is not None else moe_plan(idx, keep, E)
        xp = _GatherRowsFn.apply(x2.contiguous(), row_src, pos)
        paired = getattr(plan, "row_pad", 128) == 256
        if not _wants_grad(xp, w1, b1, w2, b2):
            R = xp.shape[0]
            h = torch.empty(R, w1.shape[1], device=xp.device, dtype=xp.dtype)
            yp = torch.empty(R, w2.shape[1], device=xp.device, dtype=xp.dtype)
            gemm(xp, w1, h, bias=b1, gelu=True, mode=GEMM_GROUPED_M, tile_group=tile_group)
            gemm(h, w2, yp, bias=b2, mode=GEMM_GROUPED_M, tile_group=tile_group, paired_groups=paired and R % 256 == 0)
        else:
            yp = _ExpertMLPFn.apply(xp, w1, b1, w2, b2, tile_group, group_offsets, paired)
        wk = weights.float().contiguous()
        return _CombineRowsFn.apply(yp, pos, wk, row_src, shared_out, float(shared_scale))
    # reference path: loop over experts
    N, d = x2.shape
    out = torch.zeros(N, d, dtype=torch.float32, device=x2.device)
    wz = weights.float() * (keep.float() if keep is not None else 1.0)
    for e in range(E):
        sel = idx == e
        tok = sel.any(-1).nonzero(as_tuple=True)[0]
        if tok.numel() == 0:
            continue
        we = (wz * sel)[tok].sum(-1, keepdim=True)
        y = F.linear(ref.gelu_tanh(F.linear(x2[tok], w1[e], b1[e])), w2[e], b2[e])
        out.index_add_(0, tok, y.float() * we)
    if shared_out is not None:
        out = out + shared_scale * shared_out.float()
    return out.to(x2.dtype)


# ----------------------------------------------------------------------------
# Optimizer / misc ops re-exported for the public facade
# ----------------------------------------------------------------------------
def muon_ns(G, steps: int = 3, coeffs=(1.875, -1.25, 0.375)):
    from . import optim_cuda

    if optim_cuda.ns_supported(G):
        return optim_cuda.newton_schulz(G, steps, coeffs)
    return ref.newton_schulz(G, steps, coeffs)


def triangular_steer_update(P, G, momentum: float, steer_scale: float):
    if _ext.use_kernels(P, G) and P.dtype == torch.float32 and P.is_contiguous() and G.is_contiguous():
        _ext.ext().steer_update(P, G, momentum, steer_scale)
        _tick()
        return P
    return ref.steer_update(P, G, momentum, steer_scale)


def route_tiers(logits, threshold: float = 0.5):
    if _ext.use_kernels(logits) and logits.dtype == torch.float32:
        tiers, _ = _ext.ext().route_tiers(logits.contiguous(), threshold)
        _tick()
        return tiers
    return ref.route_tiers(logits, threshold)


def neuron_heatmap(act, num_bins: int):
    if _ext.use_kernels(act):
        out = _ext.ext().neuron_heatmap(act.float().contiguous().flatten(), num_bins)
        _tick(2)
        return out.to(torch.int64) & 0xFFFFFFFF
    return ref.neuron_heatmap(act, num_bins)


def tier_colour_render(act, tiers):
    if _ext.use_kernels(act):
        out = _ext.ext().tier_render(act.float().contiguous(), tiers.to(torch.int32).contiguous())
        _tick()
        return out.view(torch.uint8).view(act.shape[0], act.shape[1], 4)
    return ref.tier_colour_render(act, tiers)


fwht16 = ref.fwht16
newton_schulz_reference = ref.newton_schulz


# ----------------------------------------------------------------------------
# Quantised linears (serving path)
# ----------------------------------------------------------------------------
def fp8_linear(x2, wq, ws, block: int = 128, out_dtype=torch.bfloat16):
    """y = x @ dequant(wq, ws)^T with activations quantised per 1x128 row segment (block-scaled E4M3)."""
    from . import quant_cuda

    if quant_cuda.fp8_supported(x2, wq):
        return quant_cuda.fp8_block_linear(x2, wq, ws, block, out_dtype)
    xq, xs = ref.fp8_block_quantize_act(x2, block)
    return ref.fp8_block_gemm(xq, xs, wq, ws, block, out_dtype)


def nvfp4_linear(x2, packed, scales, tscale, out_dtype=torch.bfloat16):
    """y = x @ dequant(packed, scales, tscale)^T (W4A16: weights decoded on the fly, bf16 tensor-core GEMM)."""
    from . import quant_cuda

    if quant_cuda.nvfp4_supported(x2, packed):
        return quant_cuda.nvfp4_linear(x2, packed, scales, tscale, out_dtype)
    w = ref.nvfp4_dequantize(packed, scales, tscale, torch.float32)
    return (x2.float() @ w.t()).to(out_dtype)


def nvfp4_quantize(w, scale_dtype=torch.float8_e4m3fn, hadamard: bool = False):
    """[N,K] -> (packed E2M1 [N,K/2], block scales [N,K/16], fp32 tensor scale); ``hadamard`` folds the 16-point
    Walsh-Hadamard rotation of each group of 16 inputs into the quantiser."""
    from . import quant_cuda

    if scale_dtype == torch.float8_e4m3fn and _ext.use_kernels(w) and w.dtype in (torch.bfloat16, torch.float32):
        return quant_cuda.nvfp4_quantize(w, hadamard)
    return ref.nvfp4_quantize(ref.fwht16(w.float()) if hadamard else w, scale_dtype)


def nvfp4_dequantize(packed, scales, tscale, dtype=torch.bfloat16):
    from . import quant_cuda

    if _ext.use_kernels(packed) and torch.is_tensor(tscale) and tscale.is_cuda:
        return quant_cuda.nvfp4_dequant(packed, scales, tscale).to(dtype)
    return ref.nvfp4_dequantize(packed, scales, tscale, dtype)


def fwht16(x):
    from . import quant_cuda

    if _ext.use_kernels(x) and x.dtype == torch.bfloat16 and x.numel() % 16 == 0:
        return quant_cuda.fwht16(x)
    return ref.fwht16(x)


# ----------------------------------------------------------------------------
# LoRA: frozen base GEMM with the rank-r update accumulated into its output
# ----------------------------------------------------------------------------
class _LoRALinearFn(torch.autograd.Function):
    """y = x W^T + b + s * (x A^T) B^T with W, b frozen. The low-rank product is added to the base GEMM's output tile
    by tile through the GEMM's reduce-add epilogue, so y is written once and updated in place (no separate add pass);
    the backward never forms B A."""

    @staticmethod
    def forward(ctx, x, w, bias, A, B, scaling):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if not _tma_ok(x2):
            x2 = x2.contiguous()
        y = gemm(x2, w, bias=bias)
        t = gemm(x2, A)                                  # [M, r]
        gemm(t, B, y, accumulate=True, alpha=float(scaling))
        ctx.save_for_backward(x2, w, A, B, t)
        ctx.scaling, ctx.in_shape = float(scaling), x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, A, B, t = ctx.saved_tensors
        s = ctx.scaling
        dy2 = dy.reshape(-1, w.shape[0])
        if not _tma_ok(dy2):
            dy2 = dy2.contiguous()
        u = gemm(dy2, B, b_mn=True, alpha=s)             # [M, r] = s * dy B
        dx = dA = dB = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True)
            gemm(u, A, dx, b_mn=True, accumulate=True)
            dx = dx.view(ctx.in_shape)
        if ctx.needs_input_grad[3]:
            dA = gemm(u, x2, a_mn=True, b_mn=True, out_dtype=torch.float32).to(A.dtype)      # [r, K]
        if ctx.needs_input_grad[4]:
            dB = gemm(dy2, t, a_mn=True, b_mn=True, alpha=s, out_dtype=torch.float32).to(B.dtype)  # [N, r]
        return dx, None, None, dA, dB, None


def lora_linear(x, w, bias, A, B, scaling: float):
    """LoRA linear over a frozen base weight. A: [r, in], B: [out, r]."""
    r = A.shape[0]
    if (_ext.use_kernels(x, w, A, B) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and A.dtype == torch.bfloat16
            and r % 8 == 0 and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0 and not w.requires_grad):
        return _LoRALinearFn.apply(x, w, bias, A, B, scaling)
    return F.linear(x, w, bias) + F.linear(F.linear(x, A), B) * scaling
