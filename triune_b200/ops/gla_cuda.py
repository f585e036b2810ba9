"""Dispatch to the sm_100a chunked GLA kernels (forward, backward, decode step).

Two entry points:
  * :func:`gla_chunk` for separate ``[B,T,H,64]`` tensors (the public ``ops.gla`` signature);
  * :func:`gla_attention_core` for the model: it consumes the fused projection output ``qkvg [B*T, 4*H*64]``
    directly (feature map + RoPE kernel, then the chunk kernels read v and the gate logits in place through
    strided TMA maps) and its backward writes all four gradients into one ``d qkvg`` buffer.

Reference: ``triune/kernels/fast_gla.py:692-778`` (``fast_chunk_gla``) and ``triune/model/attention.py:360-572``.
"""

from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _ext

_CHECK = os.environ.get("TRIUNE_CHECK_STATUS", "0") == "1"
GLA_MIN_LOG_DECAY = -5.0  # the kernels' lower clamp of the per-token log decay (csrc/gla/gla.cuh)
last_status = None  # device int32 status word of the most recent launch group (0 = ok)


def _note(status):
    global last_status
    last_status = status
    if _CHECK and int(status.item()) != 0:
        raise RuntimeError(f"GLA kernel reported status {int(status.item())} (bounded wait expired)")


def _tick(n):
    from . import _tick as t

    t(n)


def supported(q, k, v, g, initial_state) -> bool:
    """True when the CUDA kernels cover this call (bf16, head dims multiples of 64 up to 256, T >= 64 or T == 1)."""
    if not _ext.use_kernels(q, k, v, g):
        return False
    B, T, H, D = q.shape
    Dv = v.shape[-1]
    if q.dtype != torch.bfloat16 or D % 64 != 0 or Dv % 64 != 0 or D > 256 or Dv > 256:
        return False
    if T == 1:
        return initial_state is not None and not torch.is_grad_enabled()
    return T >= 64


def _as_matrix(x: torch.Tensor) -> torch.Tensor:
    """[B,T,H,64] -> a 2-D [B*T, ld] matrix view whose columns h*64.. hold head h (copying only if needed)."""
    B, T, H, D = x.shape
    if x.stride(3) == 1 and x.stride(2) == D and x.stride(0) == T * x.stride(1) and x.stride(1) % 8 == 0 \
            and x.data_ptr() % 16 == 0:
        return x.as_strided((B * T, H * D), (x.stride(1), 1))
    return x.contiguous().view(B * T, H * D)


class _GLAFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, init, gate_logits):
        B, T, H, D = q.shape
        e = _ext.ext()
        qm, km, vm, gm = (_as_matrix(t.to(torch.bfloat16)) for t in (q, k, v, g))
        out = torch.empty(B * T, H * D, device=q.device, dtype=torch.bfloat16)
        states, decay, fin, status = e.gla_fwd(qm, 0, km, 0, vm, 0, gm, 0, out, 0, init, B, T, H, gate_logits)
        _tick(3)
        _note(status)
        ctx.save_for_backward(qm, km, vm, gm, states, decay, fin)
        ctx.dims = (B, T, H, D, gate_logits, init is not None)
        ctx.set_materialize_grads(False)
        return out.view(B, T, H, D), fin.view(B, H, D, D)

    @staticmethod
    def backward(ctx, dout, dfin):
        # The final state is differentiable: its gradient seeds the reverse inter-chunk scan (it is the state
        # gradient after the last chunk), adds rowsum(dS_T * S_T) to every token's gate gradient, and the scan's
        # last value is the gradient of the initial state.
        qm, km, vm, gm, states, decay, fin = ctx.saved_tensors
        B, T, H, D, gate_logits, has_init = ctx.dims
        e = _ext.ext()
        if dout is None:
            dout = torch.zeros(B, T, H, D, device=qm.device, dtype=torch.bfloat16)
        dom = _as_matrix(dout.to(torch.bfloat16))
        dq, dk, dv, dg = (torch.empty(B * T, H * D, device=dom.device, dtype=torch.bfloat16) for _ in range(4))
        status, dinit = e.gla_bwd(qm, 0, km, 0, vm, 0, gm, 0, dom, 0, states, decay, dq, 0, dk, 0, dv, 0, dg, 0, B, T, H,
                                  gate_logits, dfin, fin if dfin is not None else None)
        _tick(4)
        _note(status)
        sh = (B, T, H, D)
        dinit = dinit.view(B, H, D, D) if (has_init and ctx.needs_input_grad[4]) else None
        return dq.view(sh), dk.view(sh), dv.view(sh), dg.view(sh), dinit, None


def gla_chunk(q, k, v, g, initial_state, scale, gate_logits):
    """Kernel path of ``ops.gla``. Ragged tails (T % 64) are finished by the reference op with state carry."""
    from . import reference as ref

    B, T, H, D = q.shape
    if D != 64 or v.shape[-1] != 64:
        return _gla_wide_heads(q, k, v, g, initial_state, scale, gate_logits)
    if T == 1:
        return decode_step(q, k, v, g, initial_state, gate_logits)
    Tm = (T // 64) * 64
    out, state = _GLAFn.apply(q[:, :Tm], k[:, :Tm], v[:, :Tm], g[:, :Tm], initial_state, gate_logits)
    if Tm < T:
        # ragged tail: the reference op continues from the kernels' final state (which carries its gradient back into
        # the first Tm tokens) with the kernels' clamp of the per-token log decay
        gl = torch.nn.functional.logsigmoid(g[:, Tm:].float()) if gate_logits else g[:, Tm:].float()
        gl = gl.clamp(min=GLA_MIN_LOG_DECAY, max=0.0)
        o2, state = ref.gla_chunk(q[:, Tm:], k[:, Tm:], v[:, Tm:], gl, state, 1.0)
        out = torch.cat((out, o2.to(out.dtype)), dim=1)
    if scale != 1.0:
        out = out * scale
    return out, state


def _gla_wide_heads(q, k, v, g, initial_state, scale, gate_logits):
    """Heads wider than 64 on the 64-wide kernels.

    The decay is diagonal over key dimensions, so the state rows of different key dimensions never mix:
    S[d, :] only sees q_d, k_d, g_d. A head with dk = 64 a, dv = 64 c is therefore exactly the sum over the ``a``
    key slices of ``a * c`` independent 64 x 64 heads (key slice i with value slice j), and the state is their block
    matrix. The slices are laid out as extra heads; autograd sums the gradients of the repeated slices.
    """
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    a, c = Dk // 64, Dv // 64

    def keys(x):  # [B,T,H,Dk] -> [B,T,H*a*c,64], key slice i repeated for every value slice
        return x.reshape(B, T, H, a, 1, 64).expand(B, T, H, a, c, 64).reshape(B, T, H * a * c, 64)

    v4 = v.reshape(B, T, H, 1, c, 64).expand(B, T, H, a, c, 64).reshape(B, T, H * a * c, 64)
    init4 = None
    if initial_state is not None:
        init4 = (initial_state.float().reshape(B, H, a, 64, c, 64).permute(0, 1, 2, 4, 3, 5)
                 .reshape(B, H * a * c, 64, 64).contiguous())
    o4, s4 = gla_chunk(keys(q), keys(k), v4, keys(g), init4, 1.0, gate_logits)
    out = o4.reshape(B, T, H, a, c, 64).float().sum(3).reshape(B, T, H, Dv)
    if scale != 1.0:
        out = out * scale
    state = s4.reshape(B, H, a, c, 64, 64).permute(0, 1, 2, 4, 3, 5).reshape(B, H, Dk, Dv)
    return out.to(q.dtype), state


@torch.no_grad()
def decode_step(q, k, v, g, state, gate_logits):
    """O(1) decode: q,k,v,g [B,1,H,64]; state [B,H,64,64] fp32 (updated in place when fp32-contiguous)."""
    B, T, H, D = q.shape
    e = _ext.ext()
    st = state if (state.dtype == torch.float32 and state.is_contiguous()) else state.float().contiguous()
    qm, km, vm, gm = (_as_matrix(t.to(torch.bfloat16)) for t in (q, k, v, g))
    out = torch.empty(B, H * D, device=q.device, dtype=torch.bfloat16)
    e.gla_decode(qm, 0, km, 0, vm, 0, gm, 0, st, out, 0, B, H, gate_logits)
    _tick(1)
    return out.view(B, 1, H, D), st


def gdn_supported(q, k, v, g, beta) -> bool:
    """True when the recurrent Gated DeltaNet kernel covers this call: bf16, head dim 64 or 128 (keys = values), no
    gradient wanted."""
    if not _ext.use_kernels(q, k, v, g) or q.dtype != torch.bfloat16:
        return False
    D = q.shape[-1]
    if D not in (64, 128) or v.shape[-1] != D:
        return False
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, g, beta)):
        return False
    return True


def gdn_chunk_supported(q, k, v, g, beta) -> bool:
    """True when the chunk-parallel training kernels cover this call: bf16, head dim 64 or 128 (keys = values), beta
    absent or one value per (token, head)."""
    if not _ext.use_kernels(q, k, v, g) or q.dtype != torch.bfloat16:
        return False
    D = q.shape[-1]
    if D not in (64, 128) or v.shape[-1] != D:
        return False
    return beta is None or beta.dim() == 3


class _GDNChunkFn(torch.autograd.Function):
    """Chunk-parallel Gated DeltaNet on the tcgen05 kernels (``csrc/gla/gdn_chunk_kernels.cu``): UT transform per
    chunk, sequential state pass, chunk outputs; the backward pass mirrors it stage by stage (see
    :mod:`triune_b200.ops.gdn_stages` for the algebra and the oracle of every stage)."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, init, scale, gate_logits):
        B, T, H, D = q.shape
        e = _ext.ext()
        pad = (-T) % 64
        if pad:
            # appended tokens with no key, no value and no decay leave the state and the real outputs untouched
            zeros = q.new_zeros(B, pad, H, D)
            q, k, v = (torch.cat((t, zeros), dim=1) for t in (q, k, v))
            g = torch.cat((g, g.new_full((B, pad, H, D), 30.0 if gate_logits else 0.0)), dim=1)
            if beta is not None:
                beta = torch.cat((beta, beta.new_zeros(B, pad, H)), dim=1)
        Tp = T + pad
        qm, km, vm, gm = (_as_matrix(t.to(torch.bfloat16)) for t in (q, k, v, g))
        out = torch.empty(B * Tp, H * D, device=q.device, dtype=torch.bfloat16)
        bt = beta.float().reshape(B * Tp, H).contiguous() if beta is not None else None
        ini = init.float().reshape(B * H, D, D).contiguous() if init is not None else None
        need = any(ctx.needs_input_grad[:6])
        res = e.gdn_chunk_fwd(qm, 0, km, 0, vm, 0, gm, 0, bt, ini, out, 0, B, Tp, H, D, bool(gate_logits), float(scale),
                              need and bt is not None)
        _tick(3)
        _note(res[9])
        if need:
            ctx.save_for_backward(qm, km, vm, gm, bt if bt is not None else torch.empty(0, device=q.device), *res[:9])
        ctx.dims = (B, T, Tp, H, D, float(scale), bool(gate_logits), beta is not None, init is not None,
                    None if beta is None else beta.dtype)
        ctx.set_materialize_grads(False)
        return out.view(B, Tp, H, D)[:, :T], res[8].view(B, H, D, D)

    @staticmethod
    def backward(ctx, dout, dfin):
        qm, km, vm, gm, bt, *saved = ctx.saved_tensors
        B, T, Tp, H, D, scale, gate_logits, has_beta, has_init, beta_dtype = ctx.dims
        e = _ext.ext()
        dom = torch.zeros(B, Tp, H, D, device=qm.device, dtype=torch.bfloat16)
        if dout is not None:
            dom[:, :T] = dout
        dom = dom.view(B * Tp, H * D)
        dq, dk, dv, dg = (torch.empty(B * Tp, H * D, device=qm.device, dtype=torch.bfloat16) for _ in range(4))
        dfl = dfin.float().reshape(B * H, D, D).contiguous() if dfin is not None else None
        dbeta, ds0, status = e.gdn_chunk_bwd(qm, 0, km, 0, vm, 0, gm, 0, dom, 0, bt if has_beta else None, dfl, list(saved),
                                             dq, 0, dk, 0, dv, 0, dg, 0, B, Tp, H, D, gate_logits, scale)[:3]
        _tick(6)
        _note(status)
        sh = (B, Tp, H, D)
        cut = lambda t: t.view(sh)[:, :T]
        db = dbeta.view(B, Tp, H)[:, :T].to(beta_dtype) if has_beta else None
        return cut(dq), cut(dk), cut(dv), cut(dg), db, ds0.view(B, H, D, D) if has_init else None, None, None


def gdn_chunk(q, k, v, g, beta, initial_state, scale, gate_logits):
    """Kernel path of ``ops.gated_deltanet`` under autograd; returns (out [B,T,H,D] bf16, final state fp32)."""
    return _GDNChunkFn.apply(q, k, v, g, beta, initial_state, float(scale), bool(gate_logits))


@torch.no_grad()
def gdn_recurrent(q, k, v, g, beta, initial_state, scale, gate_logits):
    """Exact Gated DeltaNet recurrence in one kernel per call (prefill of any length, or one decode step).

    q,k,v,g [B,T,H,D]; beta None, [B,T,H] or [B,T,H,D]; returns (out [B,T,H,D] bf16, state [B,H,D,D] fp32).
    Reference: the token loop of ``triune/kernels/fast_gla.py:781-836``.
    """
    B, T, H, D = q.shape
    e = _ext.ext()
    if initial_state is None:
        st = torch.zeros(B, H, D, D, device=q.device, dtype=torch.float32)
    else:
        st = initial_state.float().contiguous().clone()
    qm, km, vm, gm = (_as_matrix(t.to(torch.bfloat16)) for t in (q, k, v, g))
    out = torch.empty(B * T, H * D, device=q.device, dtype=torch.bfloat16)
    bt = None if beta is None else beta.float().contiguous()
    e.gdn_recurrent(qm, 0, km, 0, vm, 0, gm, 0, bt, st, out, 0, B, T, H, D, gate_logits, float(scale))
    _tick(1)
    return out.view(B, T, H, D), st


class _GLACoreFn(torch.autograd.Function):
    """qkvg [B*T, 4*H*64] -> attention output [B*T, H*64] (feature map, RoPE and the chunk scan fused)."""

    @staticmethod
    def forward(ctx, qkvg, cos_half, sin_half, init, B, T, H):
        D = 64
        HD = H * D
        e = _ext.ext()
        qk = e.qk_prep_fwd(qkvg, HD, cos_half, sin_half, T, H, D).view(B * T, 2 * HD)
        out = torch.empty(B * T, HD, device=qkvg.device, dtype=torch.bfloat16)
        states, decay, fin, status = e.gla_fwd(qk, 0, qk, HD, qkvg, 2 * HD, qkvg, 3 * HD, out, 0, init, B, T, H, True)
        _tick(4)
        _note(status)
        none = torch.empty(0, device=qkvg.device)
        ctx.save_for_backward(qkvg, qk, states, decay, cos_half if cos_half is not None else none,
                              sin_half if sin_half is not None else none)
        ctx.dims = (B, T, H, cos_half is not None)
        fin = fin.view(B, H, D, D)
        ctx.mark_non_differentiable(fin)
        return out, fin

    @staticmethod
    def backward(ctx, dout, dfin):
        qkvg, qk, states, decay, cs, sn = ctx.saved_tensors
        B, T, H, rope = ctx.dims
        D = 64
        HD = H * D
        e = _ext.ext()
        dout = dout.contiguous()
        dqk = torch.empty_like(qk)
        dqkvg = torch.empty_like(qkvg)
        status, _ = e.gla_bwd(qk, 0, qk, HD, qkvg, 2 * HD, qkvg, 3 * HD, dout, 0, states, decay, dqk, 0, dqk, HD, dqkvg,
                              2 * HD, dqkvg, 3 * HD, B, T, H, True, None, None)
        e.qk_prep_bwd(qkvg, HD, dqk.view(B * T, 2, H, D), dqkvg, cs if rope else None, sn if rope else None, T, H, D)
        _tick(5)
        _note(status)
        return dqkvg, None, None, None, None, None, None


def core_supported(qkvg: torch.Tensor, T: int, D: int) -> bool:
    return (
        _ext.use_kernels(qkvg)
        and qkvg.dtype == torch.bfloat16
        and D == 64
        and T % 64 == 0
        and T >= 64
        and qkvg.is_contiguous()
    )


def gla_attention_core(qkvg, cos, sin, init, B, T, H):
    ch = cos[:, :32].float().contiguous() if cos is not None else None
    sh = sin[:, :32].float().contiguous() if sin is not None else None
    return _GLACoreFn.apply(qkvg, ch, sh, init, B, T, H)
