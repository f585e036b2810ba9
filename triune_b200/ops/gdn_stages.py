"""Gated DeltaNet, chunk-parallel, as the explicit stages the sm_100a kernels implement (forward and backward).

Recurrence (``triune/kernels/fast_gla.py:781-836`` of the reference): with a per-key-dimension log decay ``g <= 0``,

    u_t = beta_t (v_t - S_{t-1}^T k_t),    S_t = diag(e^{g_t}) S_{t-1} + k_t u_t^T,    o_t = S_t^T q_t.

Inside a chunk of C tokens, with ``b = cumsum(g)`` (inclusive), ``bp = b - g`` (exclusive) and ``b_C`` the last row:

    Kbar_t = k_t e^{bp_t}        Qbar_t = q_t e^{b_t}        Kend_t = k_t e^{b_C - b_t}
    Lraw[t,s] = sum_d k_td k_sd e^{bp_td - b_sd}  (s <  t)      L = diag(beta) Lraw      T = (I + L)^{-1}
    A[t,s]    = sum_d q_td k_sd e^{b_td  - b_sd}  (s <= t)
    U0 = T (beta V)      W = T (beta Kbar)                                   (stage F1, per chunk)
    U  = U0 - W S        S' = diag(e^{b_C}) S + Kend^T U                     (stage F2, sequential over chunks)
    O  = A U + Qbar S                                                        (stage F3, per chunk)

Backward, given dO and dS' flowing in from the next chunk:

    G1 = A^T dO          H1 = Qbar^T dO                                      (stage B1, per chunk)
    dU = G1 + Kend dS'   dS = H1 + diag(e^{b_C}) dS' - W^T dU                (stage B2, reverse sequential)
    dQbar = dO S^T       dKend = U dS'^T        dW = -dU S^T                 (stage B3a, per chunk)
    dVb = T^T dU         dKb = T^T dW           dL = -strict(dVb U0^T + dKb W^T)
    dv = beta dVb        dbeta = <dVb, V> + <dKb, Kbar> + <dL, Lraw>         (stage B3b, per chunk)
    dA = mask(dO U^T)    dLraw = diag(beta) dL
    dq   = e^{b} dQbar + sum_s dA[t,s] k_s e^{b_t - b_s}
    dk_w = e^{b_C - b} dKend + sum_t dA[t,s] q_t e^{b_t - b_s} + sum_t dLraw[t,s] k_t e^{bp_t - b_s}
    dk_r = e^{bp} beta dKb   + sum_s dLraw[t,s] k_s e^{bp_t - b_s}          (stage B3c, per chunk)
    dk = dk_w + dk_r

The decay gradient follows from a global identity: everything depends on g only through ``q e^{B}``, the write key
``k e^{-B}`` and the read key ``k e^{B_{t-1}}`` (B the cumulative log decay over the whole sequence), hence

    dL/dB_t = q_t dq_t - k_t dk_w,t + k_{t+1} dk_r,t+1      and      dg_tau = sum_{t >= tau} dL/dB_t.

All functions here work on ``[B, H, NT, C, D]`` tensors in the dtype they are given (fp64 in the tests) and are the
oracle for every kernel stage; :func:`gated_deltanet_chunked` strings them together with a hand-written backward and
is the CPU executor of ``ops.gated_deltanet`` under autograd.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

MIN_LOG_DECAY = -5.0  # the kernels' lower clamp of the per-token log decay


def _pair_scores(x, y, bx, by, strict: bool):
    """S[t,s] = sum_d x[t,d] y[s,d] exp(bx[t,d] - by[s,d]) masked to s <= t (s < t when strict). Pairwise form:
    exact for any decay, O(C^2 D) memory, for tests and the CPU path only."""
    C = x.shape[-2]
    e = torch.exp(torch.clamp(bx.unsqueeze(-2) - by.unsqueeze(-3), max=0.0))  # [.., t, s, d]
    s = (x.unsqueeze(-2) * y.unsqueeze(-3) * e).sum(-1)
    mask = torch.ones(C, C, dtype=torch.bool, device=x.device).tril(-1 if strict else 0)
    return s * mask


def chunk_layout(x: torch.Tensor, C: int, fill: float = 0.0):
    """[B, T, H, D] -> [B, H, NT, C, D] with zero rows appended (no key, no value, no decay: a no-op for the state)."""
    B, T, H, D = x.shape
    pad = (-T) % C
    x = x.permute(0, 2, 1, 3)
    if pad:
        x = torch.cat((x, x.new_full((B, H, pad, D), fill)), dim=2)
    return x.reshape(B, H, (T + pad) // C, C, D)


def stage_f1(k, v, gl, beta):
    """Per chunk: (U0, W, T, Lraw). k, v, gl: [.., C, D]; beta [.., C, 1] or None."""
    b = torch.cumsum(gl, dim=-2)
    bp = b - gl
    Lraw = _pair_scores(k, k, bp, b, strict=True)
    kbar = k * torch.exp(bp)
    rv, rk = (v, kbar) if beta is None else (v * beta, kbar * beta)
    L = Lraw if beta is None else Lraw * beta
    C = k.shape[-2]
    eye = torch.eye(C, dtype=k.dtype, device=k.device)
    T = torch.linalg.solve_triangular(eye + L, eye.expand_as(L).contiguous(), upper=False, unitriangular=True)
    return T @ rv, T @ rk, T, Lraw


def stage_f2(U0, W, k, gl, S0):
    """Sequential over chunks: returns (U [.., NT, C, Dv], S_chunk_start [.., NT, Dk, Dv], S_final)."""
    b = torch.cumsum(gl, dim=-2)
    b_last = b[..., -1:, :]
    kend = k * torch.exp(b_last - b)
    decay = torch.exp(b_last).transpose(-1, -2)  # [.., NT, Dk, 1]
    S = S0
    us, states = [], []
    for c in range(U0.shape[2]):
        states.append(S)
        Uc = U0[:, :, c] - W[:, :, c] @ S
        us.append(Uc)
        S = S * decay[:, :, c] + kend[:, :, c].transpose(-1, -2) @ Uc
    return torch.stack(us, dim=2), torch.stack(states, dim=2), S


def stage_f3(q, k, gl, U, S_start):
    b = torch.cumsum(gl, dim=-2)
    A = _pair_scores(q, k, b, b, strict=False)
    return A @ U + (q * torch.exp(b)) @ S_start


def stage_b1(q, k, gl, dO):
    b = torch.cumsum(gl, dim=-2)
    A = _pair_scores(q, k, b, b, strict=False)
    return A.transpose(-1, -2) @ dO, (q * torch.exp(b)).transpose(-1, -2) @ dO


def stage_b2(G1, H1, W, k, gl, dS_final):
    """Reverse sequential: returns (dU [.., NT, C, Dv], dS_end [.., NT, Dk, Dv] = gradient of the state at each chunk's
    end, dS0)."""
    b = torch.cumsum(gl, dim=-2)
    b_last = b[..., -1:, :]
    kend = k * torch.exp(b_last - b)
    decay = torch.exp(b_last).transpose(-1, -2)
    NT = G1.shape[2]
    dS = dS_final
    dus, dends = [None] * NT, [None] * NT
    for c in range(NT - 1, -1, -1):
        dends[c] = dS
        dUc = G1[:, :, c] + kend[:, :, c] @ dS
        dus[c] = dUc
        dS = H1[:, :, c] + decay[:, :, c] * dS - W[:, :, c].transpose(-1, -2) @ dUc
    return torch.stack(dus, dim=2), torch.stack(dends, dim=2), dS


def stage_b3a(dO, U, dU, S_start, dS_end):
    St = S_start.transpose(-1, -2)
    return dO @ St, U @ dS_end.transpose(-1, -2), -(dU @ St)  # dQbar, dKend, dW


def stage_b3b(T, dU, dW, U0, W, k, v, gl, beta, Lraw):
    """Returns (dv, dk_r1 = e^{bp} beta dKb, dbeta [.., C] or None, dLraw)."""
    b = torch.cumsum(gl, dim=-2)
    bp = b - gl
    Tt = T.transpose(-1, -2)
    dVb, dKb = Tt @ dU, Tt @ dW
    C = T.shape[-1]
    strict = torch.ones(C, C, dtype=torch.bool, device=T.device).tril(-1)
    dL = -(dVb @ U0.transpose(-1, -2) + dKb @ W.transpose(-1, -2)) * strict
    kbar = k * torch.exp(bp)
    if beta is None:
        return dVb, dKb * torch.exp(bp), None, dL
    dbeta = (dVb * v).sum(-1) + (dKb * kbar).sum(-1) + (dL * Lraw).sum(-1)
    return dVb * beta, dKb * beta * torch.exp(bp), dbeta, dL * beta


def stage_b3c(q, k, gl, dO, U, dLraw, dQbar, dKend, dk_r1):
    """Returns (dq, dk, E1 = q dq - k dk_w, E2 = k dk_r) per token."""
    b = torch.cumsum(gl, dim=-2)
    bp = b - gl
    b_last = b[..., -1:, :]
    C = q.shape[-2]
    incl = torch.ones(C, C, dtype=torch.bool, device=q.device).tril(0)
    dA = (dO @ U.transpose(-1, -2)) * incl
    # pairwise decay weights (exact): w_b[t,s,d] = e^{b_t - b_s}, w_p[t,s,d] = e^{bp_t - b_s}
    w_b = torch.exp(torch.clamp(b.unsqueeze(-2) - b.unsqueeze(-3), max=0.0))
    w_p = torch.exp(torch.clamp(bp.unsqueeze(-2) - b.unsqueeze(-3), max=0.0))
    dq = dQbar * torch.exp(b) + torch.einsum("...ts,...tsd,...sd->...td", dA, w_b, k)
    dk_w = (dKend * torch.exp(b_last - b) + torch.einsum("...ts,...tsd,...td->...sd", dA, w_b, q)
            + torch.einsum("...ts,...tsd,...td->...sd", dLraw, w_p, k))
    dk_r = dk_r1 + torch.einsum("...ts,...tsd,...sd->...td", dLraw, w_p, k)
    return dq, dk_w + dk_r, q * dq - k * dk_w, k * dk_r


def decay_gradient(E1, E2):
    """dg over the flattened time axis [.., T, D]: inclusive suffix sum of E1 plus exclusive suffix sum of E2."""
    s1 = torch.flip(torch.cumsum(torch.flip(E1, dims=(-2,)), dim=-2), dims=(-2,))
    s2 = torch.flip(torch.cumsum(torch.flip(E2, dims=(-2,)), dim=-2), dims=(-2,)) - E2
    return s1 + s2


def forward_stages(q, k, v, gl, beta, S0):
    """All tensors in chunk layout. Returns (O, S_final, saved tensors for the backward stages)."""
    U0, W, T, Lraw = stage_f1(k, v, gl, beta)
    U, S_start, S_fin = stage_f2(U0, W, k, gl, S0)
    O = stage_f3(q, k, gl, U, S_start)
    return O, S_fin, (U0, W, T, Lraw, U, S_start)


def backward_stages(q, k, v, gl, beta, saved, dO, dS_final):
    U0, W, T, Lraw, U, S_start = saved
    G1, H1 = stage_b1(q, k, gl, dO)
    dU, dS_end, dS0 = stage_b2(G1, H1, W, k, gl, dS_final)
    dQbar, dKend, dW = stage_b3a(dO, U, dU, S_start, dS_end)
    dv, dk_r1, dbeta, dLraw = stage_b3b(T, dU, dW, U0, W, k, v, gl, beta, Lraw)
    dq, dk, E1, E2 = stage_b3c(q, k, gl, dO, U, dLraw, dQbar, dKend, dk_r1)
    shp = E1.shape
    flat = (shp[0], shp[1], shp[2] * shp[3], shp[4])
    dgl = decay_gradient(E1.reshape(flat), E2.reshape(flat)).reshape(shp)
    # A differentiated final state adds rowsum(dS_T * S_T) to every token's decay gradient (S_T = e^{B_T} times the
    # decay-free state); the caller holds S_T and adds that term.
    return dq, dk, dv, dgl, dbeta, dS0


class _ChunkedFn(torch.autograd.Function):
    """Chunk-parallel Gated DeltaNet with the stage-wise backward (any device, any float dtype)."""

    @staticmethod
    def forward(ctx, q, k, v, gl, beta, S0, scale, C):
        B, T, H, D = q.shape
        dt = torch.float64 if q.dtype == torch.float64 else torch.float32
        qc, kc, vc = (chunk_layout(x.to(dt), C) for x in (q, k, v))
        gc = chunk_layout(torch.clamp(gl.to(dt), min=MIN_LOG_DECAY, max=0.0), C)
        bc = None
        if beta is not None:
            bc = chunk_layout(beta.to(dt).unsqueeze(-1), C)
        S = S0.to(dt) if S0 is not None else qc.new_zeros(B, H, D, v.shape[-1])
        O, S_fin, saved = forward_stages(qc, kc, vc, gc, bc, S)
        ctx.save_for_backward(qc, kc, vc, gc, bc if bc is not None else qc.new_zeros(0), S_fin, *saved)
        ctx.meta = (B, T, H, D, v.shape[-1], float(scale), beta is not None, S0 is not None, q.dtype, gl.dtype,
                    None if beta is None else beta.dtype)
        out = (O * scale).reshape(B, H, -1, v.shape[-1])[:, :, :T].permute(0, 2, 1, 3)
        return out.to(q.dtype), S_fin

    @staticmethod
    def backward(ctx, dout, dS_fin):
        qc, kc, vc, gc, bc, S_fin, *saved = ctx.saved_tensors
        B, T, H, D, Dv, scale, has_beta, has_s0, qdt, gdt, bdt = ctx.meta
        C = qc.shape[3]
        dt = qc.dtype
        if dout is None:
            dO = qc.new_zeros(B, H, qc.shape[2], C, Dv)
        else:
            dO = chunk_layout(dout.to(dt) * scale, C)
        dSf = dS_fin.to(dt) if dS_fin is not None else torch.zeros_like(S_fin)
        dq, dk, dv, dgl, dbeta, dS0 = backward_stages(qc, kc, vc, gc, bc if has_beta else None, tuple(saved), dO, dSf)
        if dS_fin is not None:
            dgl = dgl + (dSf * S_fin).sum(-1)[:, :, None, None, :]

        def unchunk(x):
            return x.reshape(B, H, -1, x.shape[-1])[:, :, :T].permute(0, 2, 1, 3)

        inside = (gc > MIN_LOG_DECAY) & (gc < 0.0) | (gc == 0.0)  # the clamp passes no gradient outside [-5, 0]
        dgl = dgl * inside
        return (unchunk(dq).to(qdt), unchunk(dk).to(qdt), unchunk(dv).to(qdt), unchunk(dgl).to(gdt),
                unchunk(dbeta.unsqueeze(-1)).squeeze(-1).to(bdt) if has_beta else None,
                dS0.to(torch.float32 if dt == torch.float32 else dt) if has_s0 else None, None, None)


def gated_deltanet_chunked(q, k, v, log_decay, beta: Optional[torch.Tensor] = None,
                           initial_state: Optional[torch.Tensor] = None, scale: float = 1.0,
                           chunk_size: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Differentiable chunk-parallel Gated DeltaNet. q, k, v, log_decay: [B, T, H, D]; beta None or [B, T, H];
    returns (out [B, T, H, Dv], final_state [B, H, Dk, Dv])."""
    return _ChunkedFn.apply(q, k, v, log_decay, beta, initial_state, scale, chunk_size)
