"""Plain-PyTorch statements of every operator in the framework.

These are (a) the CPU path, (b) the numerical oracles the CUDA kernels are tested
against, and (c) differentiable fall-backs for shapes a kernel does not cover.
Nothing here is on a GPU hot path: the dispatchers in ``triune_b200.ops`` route CUDA
tensors to the sm_100a kernels.

Semantics follow the reference project (paths relative to its root):
  * RMSNorm / fused add-RMSNorm        triune/kernels/fast_rmsnorm.py:181-335
  * half-split rotary                  triune/kernels/fast_rope.py:16-154
  * GLA feature map                    triune/model/attention.py:509-531
  * GLA recurrence / chunked form      triune/kernels/fast_gla.py:569-778
  * Gated DeltaNet recurrence          triune/kernels/fast_gla.py:781-836
  * cross-entropy (ignore_index)       triune/kernels/fast_cross_entropy.py:110-170
  * Newton-Schulz polar iteration      triune/kernels/fast_muon.py:15-161
  * triangular AdamW core              triune/kernels/fast_triangular.py:91-173
  * NVFP4 / E2M1 codec, FWHT-16        triune/kernels/fast_nvfp4.py:17-143
  * tier router, heatmap, steer update csrc/engine/engine.cpp:314-475
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

# A per-token log-decay below this value is clamped inside the chunked kernels. It bounds the
# decay span of one 16-token sub-chunk to 80 nats so the factored sub-chunk products stay inside the
# fp32/bf16 exponent range; exp(-5) per token already erases a state dimension within three tokens.
GLA_MIN_LOG_DECAY = -5.0


# ----------------------------------------------------------------------------
# Normalisation / activations / rotary
# ----------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * inv * weight.float()).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """Returns (rmsnorm(x + residual), x + residual)."""
    s = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(s, weight, eps), s


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(x, approximate="tanh")


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate) * up


def rope_tables(seq_len: int, head_dim: int, base: float = 10000.0, offset: int = 0, device=None):
    """cos/sin tables [seq_len, head_dim] in the half-split convention (fp32)."""
    half = head_dim // 2
    inv_freq = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float32, device=device) / half))
    pos = torch.arange(offset, offset + seq_len, dtype=torch.float32, device=device)
    ang = torch.outer(pos, inv_freq)
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, T, H, D]; cos/sin: [T, D]. Half-split rotation: (x1, x2) -> (x1 c - x2 s, x2 c + x1 s)."""
    x1, x2 = x.chunk(2, dim=-1)
    rot = torch.cat((-x2, x1), dim=-1)
    c = cos.to(x.dtype)[None, :, None, :]
    s = sin.to(x.dtype)[None, :, None, :]
    return x * c + rot * s


def qkvg_prep(q, k, g, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor]):
    """GLA feature map: q,k -> normalize(elu+1) then RoPE; g -> logsigmoid. Inputs [B,T,H,D]."""
    out_dtype = q.dtype
    qf = F.normalize(F.elu(q.float()) + 1.0, p=2.0, dim=-1, eps=1e-6)
    kf = F.normalize(F.elu(k.float()) + 1.0, p=2.0, dim=-1, eps=1e-6)
    if cos is not None:
        qf = apply_rope(qf, cos.float(), sin.float())
        kf = apply_rope(kf, cos.float(), sin.float())
    gl = F.logsigmoid(g.float())
    return qf.to(out_dtype), kf.to(out_dtype), gl.to(out_dtype)


# ----------------------------------------------------------------------------
# Gated linear attention
# ----------------------------------------------------------------------------
def gla_recurrent(q, k, v, g, initial_state=None, scale: float = 1.0):
    """Token-by-token oracle. q,k,g: [B,T,H,dk], v: [B,T,H,dv]; state [B,H,dk,dv].

    S_t = diag(exp(min(g_t,0))) S_{t-1} + k_t v_t^T ;  o_t = scale * q_t^T S_t
    """
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    dt = torch.float64 if q.dtype == torch.float64 else torch.float32
    S = (
        initial_state.to(dt).clone()
        if initial_state is not None
        else torch.zeros(B, H, dk, dv, dtype=dt, device=q.device)
    )
    qf, kf, vf = q.to(dt), k.to(dt), v.to(dt)
    decay = torch.exp(torch.clamp(g.to(dt), max=0.0))
    outs = []
    for t in range(T):
        S = S * decay[:, t].unsqueeze(-1) + kf[:, t].unsqueeze(-1) * vf[:, t].unsqueeze(-2)
        outs.append(torch.einsum("bhk,bhkv->bhv", qf[:, t], S) * scale)
    return torch.stack(outs, dim=1).to(q.dtype), S


def gla_decode_step(q, k, v, g, state, scale: float = 1.0):
    """One O(1) decode step. q,k,g: [B,H,dk], v: [B,H,dv], state [B,H,dk,dv] (fp32). Returns (o, new_state)."""
    sf = state.float()
    new_state = sf * torch.exp(torch.clamp(g.float(), max=0.0)).unsqueeze(-1) + k.float().unsqueeze(
        -1
    ) * v.float().unsqueeze(-2)
    o = torch.einsum("bhk,bhkv->bhv", q.float(), new_state) * scale
    return o.to(q.dtype), new_state


def _chunk_scores(qc, kc, bq, bk, strict: bool):
    """Exact decayed scores A[t,s] = sum_d q[t,d] k[s,d] exp(bq[t,d]-bk[s,d]) for s<=t (s<t if strict).

    qc,kc,bq,bk: [..., C, d] (fp32/fp64). Uses 16-token sub-chunks: off-diagonal sub-blocks are
    factored around the first row of the query sub-chunk (all exponents <= 0), the diagonal sub-blocks
    are evaluated pairwise, which is exact for any decay.
    """
    C = qc.shape[-2]
    SC = 16
    n_sub = (C + SC - 1) // SC
    A = qc.new_zeros(*qc.shape[:-2], C, C)
    for i in range(n_sub):
        t0, t1 = i * SC, min(C, (i + 1) * SC)
        qi, bqi = qc[..., t0:t1, :], bq[..., t0:t1, :]
        if i > 0:
            ref = bq[..., t0 : t0 + 1, :]
            # bq (query side) may be an offset cumsum (strict form) whose first row is larger than bk of
            # earlier rows only by the row's own decay, so min(.,0) keeps every exponent non-positive.
            qs = qi * torch.exp(torch.clamp(bqi - ref, max=0.0))
            ks = kc[..., :t0, :] * torch.exp(torch.clamp(ref - bk[..., :t0, :], max=0.0))
            A[..., t0:t1, :t0] = qs @ ks.transpose(-1, -2)
        # diagonal block, pairwise
        d = bqi.unsqueeze(-2) - bk[..., t0:t1, :].unsqueeze(-3)  # [.., t, s, d]
        w = torch.exp(torch.clamp(d, max=0.0))
        blk = (qi.unsqueeze(-2) * kc[..., t0:t1, :].unsqueeze(-3) * w).sum(-1)
        n = t1 - t0
        mask = torch.ones(n, n, dtype=torch.bool, device=qc.device).tril(-1 if strict else 0)
        A[..., t0:t1, t0:t1] = blk * mask
    return A


def gla_chunk(q, k, v, g, initial_state=None, scale: float = 1.0, chunk_size: int = 64):
    """Chunk-parallel GLA, differentiable, any T (ragged tail handled as a short chunk).

    Same recurrence as :func:`gla_recurrent`. Three phases, which is also how the CUDA kernels are
    organised: per-chunk local state, sequential inter-chunk scan, per-chunk outputs.
    """
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    dt = torch.float64 if q.dtype == torch.float64 else torch.float32
    S = (
        initial_state.to(dt)
        if initial_state is not None
        else torch.zeros(B, H, dk, dv, dtype=dt, device=q.device)
    )
    qf = q.to(dt).permute(0, 2, 1, 3)
    kf = k.to(dt).permute(0, 2, 1, 3)
    vf = v.to(dt).permute(0, 2, 1, 3)
    gf = torch.clamp(g.to(dt), max=0.0).permute(0, 2, 1, 3)
    outs = []
    for c0 in range(0, T, chunk_size):
        c1 = min(T, c0 + chunk_size)
        qc, kc, vc, gc = qf[:, :, c0:c1], kf[:, :, c0:c1], vf[:, :, c0:c1], gf[:, :, c0:c1]
        b = torch.cumsum(gc, dim=-2)
        A = _chunk_scores(qc, kc, b, b, strict=False)
        o = A @ vc + (qc * torch.exp(b)) @ S
        outs.append(o * scale)
        b_last = b[:, :, -1:, :]
        k_end = kc * torch.exp(b_last - b)
        S = S * torch.exp(b_last).transpose(-1, -2) + k_end.transpose(-1, -2) @ vc
    out = torch.cat(outs, dim=2).permute(0, 2, 1, 3)
    return out.to(q.dtype), S


# ----------------------------------------------------------------------------
# Gated DeltaNet
# ----------------------------------------------------------------------------
def _beta_view(beta, t_slice=None):
    return beta


def gated_deltanet_recurrent(q, k, v, g, beta=None, initial_state=None, scale: float = 1.0):
    """Token-by-token oracle of the reference's delta rule.

    v_pred = k_t^T S_{t-1}; u_t = v_t - v_pred; S_t = diag(exp(min(g_t,0))) S_{t-1} + k_t (beta_t * u_t)^T;
    o_t = q_t^T S_t.  beta: None (=1), [B,T,H] or [B,T,H,dk] (per key-row write strength).
    """
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    dt = torch.float64 if q.dtype == torch.float64 else torch.float32
    S = (
        initial_state.to(dt).clone()
        if initial_state is not None
        else torch.zeros(B, H, dk, dv, dtype=dt, device=q.device)
    )
    qf, kf, vf = q.to(dt), k.to(dt), v.to(dt)
    decay = torch.exp(torch.clamp(g.to(dt), max=0.0))
    outs = []
    for t in range(T):
        v_pred = torch.einsum("bhk,bhkv->bhv", kf[:, t], S)
        u = vf[:, t] - v_pred
        write = kf[:, t].unsqueeze(-1) * u.unsqueeze(-2)
        if beta is not None:
            bt = beta[:, t].to(dt)
            write = write * (bt.unsqueeze(-1) if bt.ndim == 3 else bt[..., None, None])
        S = S * decay[:, t].unsqueeze(-1) + write
        outs.append(torch.einsum("bhk,bhkv->bhv", qf[:, t], S) * scale)
    return torch.stack(outs, dim=1).to(q.dtype), S


def gated_deltanet_chunk(q, k, v, g, beta=None, initial_state=None, scale: float = 1.0, chunk_size: int = 64):
    """Chunk-parallel Gated DeltaNet (UT/WY transform with per-dimension decay), differentiable.

    With u_t = beta_t (v_t - S_{t-1}^T k_t) the state follows the GLA recurrence with values u, and the
    u of one chunk solve a unit-lower-triangular system
        (I + L) U = beta (V - Kbar S_0),   L[t,s] = beta_t sum_d k_t k_s exp(b_{t-1}-b_s) (s<t),
        Kbar_t = k_t * exp(b_{t-1}),
    so each chunk costs one triangular solve plus GLA-shaped products. Only scalar-per-head or absent
    beta is supported here; a per-row [B,T,H,dk] beta falls back to the recurrence.
    """
    if beta is not None and beta.ndim == 4:
        return gated_deltanet_recurrent(q, k, v, g, beta, initial_state, scale)
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    dt = torch.float64 if q.dtype == torch.float64 else torch.float32
    S = (
        initial_state.to(dt)
        if initial_state is not None
        else torch.zeros(B, H, dk, dv, dtype=dt, device=q.device)
    )
    qf = q.to(dt).permute(0, 2, 1, 3)
    kf = k.to(dt).permute(0, 2, 1, 3)
    vf = v.to(dt).permute(0, 2, 1, 3)
    gf = torch.clamp(g.to(dt), max=0.0).permute(0, 2, 1, 3)
    bf = None if beta is None else beta.to(dt).permute(0, 2, 1).unsqueeze(-1)  # [B,H,T,1]
    outs = []
    for c0 in range(0, T, chunk_size):
        c1 = min(T, c0 + chunk_size)
        qc, kc, vc, gc = qf[:, :, c0:c1], kf[:, :, c0:c1], vf[:, :, c0:c1], gf[:, :, c0:c1]
        C = c1 - c0
        b = torch.cumsum(gc, dim=-2)
        b_prev = b - gc  # cumulative decay up to and excluding token t
        L = _chunk_scores(kc, kc, b_prev, b, strict=True)
        rhs = vc - (kc * torch.exp(b_prev)) @ S
        if bf is not None:
            bc = bf[:, :, c0:c1]
            L = L * bc
            rhs = rhs * bc
        eye = torch.eye(C, dtype=dt, device=q.device)
        U = torch.linalg.solve_triangular(eye + L, rhs, upper=False, unitriangular=True)
        A = _chunk_scores(qc, kc, b, b, strict=False)
        o = A @ U + (qc * torch.exp(b)) @ S
        outs.append(o * scale)
        b_last = b[:, :, -1:, :]
        S = S * torch.exp(b_last).transpose(-1, -2) + (kc * torch.exp(b_last - b)).transpose(-1, -2) @ U
    out = torch.cat(outs, dim=2).permute(0, 2, 1, 3)
    return out.to(q.dtype), S


def _chunk_scores_factored(qc, kc, bq, bk, strict: bool):
    """The decayed scores of :func:`_chunk_scores` with every 16 x 16 block written as a matrix product around the
    block's first query row (the layout of the tcgen05 kernels): off-diagonal blocks as there, diagonal blocks as
    (q e^{bq - ref}) (k e^{ref - bk})^T with exponents up to +80 on the key side. Exact while the decay inside a
    16-token sub-chunk stays above e^-80 (log-sigmoid gates reach that only with logits below -5 on every step); no
    [.., 16, 16, d] intermediates are built, so memory and time drop by the head dimension."""
    C = qc.shape[-2]
    SC = 16
    n_sub = (C + SC - 1) // SC
    rows = []
    for i in range(n_sub):
        t0, t1 = i * SC, min(C, (i + 1) * SC)
        ref = bq[..., t0 : t0 + 1, :]
        qs = qc[..., t0:t1, :] * torch.exp(torch.clamp(bq[..., t0:t1, :] - ref, max=0.0))
        ks = kc[..., :t1, :] * torch.exp(torch.clamp(ref - bk[..., :t1, :], max=80.0))
        blk = qs @ ks.transpose(-1, -2)                                    # [.., t1-t0, t1]
        n = t1 - t0
        mask = torch.ones(n, n, dtype=torch.bool, device=qc.device).tril(-1 if strict else 0)
        diag = blk[..., t0:t1] * mask
        pad = blk.new_zeros(*blk.shape[:-1], C - t1)
        rows.append(torch.cat((blk[..., :t0], diag, pad), dim=-1))
    return torch.cat(rows, dim=-2)


def gated_deltanet_chunk_parallel(q, k, v, g, beta=None, initial_state=None, scale: float = 1.0, chunk_size: int = 64):
    """Chunk-parallel Gated DeltaNet in the WY form, differentiable; the training path of ``ops.gated_deltanet``.

    Same algebra as :func:`gated_deltanet_chunk`, arranged so that everything except the state recurrence is ONE batched
    operation over all chunks: with T = (I + L)^{-1} per chunk, U0 = T (beta V) and W = T (beta Kbar) the effective
    values of chunk c are U_c = U0_c - W_c S_c, so the only sequential part is two small matrix products per chunk
    (W_c S_c and K_end_c^T U_c); scores, the triangular solves and the outputs run batched. Exact while no 16-token
    sub-chunk decays by more than e^-80 in total (see :func:`_chunk_scores_factored`). A per-row [B,T,H,dk] beta falls
    back to the token recurrence.
    """
    if beta is not None and beta.ndim == 4:
        return gated_deltanet_recurrent(q, k, v, g, beta, initial_state, scale)
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    C = chunk_size
    dt = torch.float64 if q.dtype == torch.float64 else torch.float32
    pad = (-T) % C
    NT = (T + pad) // C

    def prep(x, fill=0.0):  # [B,T,H,d] -> [B,H,NT,C,d], zero rows appended (no key, no value, no decay: a no-op)
        x = x.to(dt).permute(0, 2, 1, 3)
        if pad:
            x = torch.cat((x, x.new_full((B, H, pad, x.shape[-1]), fill)), dim=2)
        return x.reshape(B, H, NT, C, x.shape[-1])

    qf, kf, vf = prep(q), prep(k), prep(v)
    gf = torch.clamp(prep(g), max=0.0)
    b = torch.cumsum(gf, dim=-2)
    b_prev = b - gf
    b_last = b[..., -1:, :]                                                 # [B,H,NT,1,dk]
    L = _chunk_scores_factored(kf, kf, b_prev, b, strict=True)             # [B,H,NT,C,C]
    kbar = kf * torch.exp(b_prev)
    rhs_v, rhs_k = vf, kbar
    if beta is not None:
        bf = beta.to(dt).permute(0, 2, 1)
        if pad:
            bf = torch.cat((bf, bf.new_zeros(B, H, pad)), dim=2)
        bf = bf.reshape(B, H, NT, C, 1)
        L, rhs_v, rhs_k = L * bf, vf * bf, kbar * bf
    eye = torch.eye(C, dtype=dt, device=q.device)
    sol = torch.linalg.solve_triangular(eye + L, torch.cat((rhs_v, rhs_k), dim=-1), upper=False, unitriangular=True)
    U0, W = sol[..., :dv], sol[..., dv:]                                    # [B,H,NT,C,dv], [B,H,NT,C,dk]
    kend_t = (kf * torch.exp(b_last - b)).transpose(-1, -2)                 # [B,H,NT,dk,C]
    decay = torch.exp(b_last).transpose(-1, -2)                             # [B,H,NT,dk,1]
    S = initial_state.to(dt) if initial_state is not None else q.new_zeros(B, H, dk, dv, dtype=dt)
    states, us = [], []
    for c in range(NT):                                                     # the sequential part
        states.append(S)
        Uc = U0[:, :, c] - W[:, :, c] @ S
        us.append(Uc)
        S = S * decay[:, :, c] + kend_t[:, :, c] @ Uc
    S_all = torch.stack(states, dim=2)                                      # state before each chunk
    U = torch.stack(us, dim=2)
    A = _chunk_scores_factored(qf, kf, b, b, strict=False)
    o = (A @ U + (qf * torch.exp(b)) @ S_all) * scale
    out = o.reshape(B, H, NT * C, dv)[:, :, :T].permute(0, 2, 1, 3)
    return out.to(q.dtype), S


def gated_deltanet_decode_step(q, k, v, g, state, beta=None, scale: float = 1.0):
    sf = state.float()
    kf = k.float()
    u = v.float() - torch.einsum("bhk,bhkv->bhv", kf, sf)
    write = kf.unsqueeze(-1) * u.unsqueeze(-2)
    if beta is not None:
        bt = beta.float()
        write = write * (bt.unsqueeze(-1) if bt.ndim == 3 else bt[..., None, None])
    new_state = sf * torch.exp(torch.clamp(g.float(), max=0.0)).unsqueeze(-1) + write
    o = torch.einsum("bhk,bhkv->bhv", q.float(), new_state) * scale
    return o.to(q.dtype), new_state


# ----------------------------------------------------------------------------
# Losses
# ----------------------------------------------------------------------------
def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    t = targets.reshape(-1)
    total = F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), t, ignore_index=ignore_index, reduction="sum")
    return total / (t != ignore_index).sum().clamp_min(1)  # a batch with every target ignored has loss 0, not 0 / 0


def linear_cross_entropy(
    h: torch.Tensor,
    weight: torch.Tensor,
    targets: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    ignore_index: int = -100,
    chunk: int = 4096,
):
    """Head GEMM + CE without keeping the [N,V] logits: returns (mean loss, valid count).

    Differentiable by recomputation per chunk through autograd checkpointing of each chunk.
    """
    h2 = h.reshape(-1, h.shape[-1])
    t = targets.reshape(-1)
    n_valid = (t != ignore_index).sum().clamp_min(1)
    total = h2.new_zeros((), dtype=torch.float32)

    def _piece(hc, tc):
        lg = F.linear(hc, weight, bias).float()
        return F.cross_entropy(lg, tc, ignore_index=ignore_index, reduction="sum")

    for s in range(0, h2.shape[0], chunk):
        hc, tc = h2[s : s + chunk], t[s : s + chunk]
        if torch.is_grad_enabled() and (hc.requires_grad or weight.requires_grad):
            total = total + torch.utils.checkpoint.checkpoint(_piece, hc, tc, use_reentrant=False)
        else:
            total = total + _piece(hc, tc)
    return total / n_valid, n_valid


# ----------------------------------------------------------------------------
# Optimizer math
# ----------------------------------------------------------------------------
def newton_schulz(G: torch.Tensor, steps: int = 3, coeffs=(1.875, -1.25, 0.375), eps: float = 1e-7) -> torch.Tensor:
    """Quintic Newton-Schulz polar iteration on the last two dims (batched).

    X <- a X + (b A + c A^2) X with A = X X^T, after scaling X so its spectral norm is safely <= 1.
    The scale is max(1.15 * sigma_hat, ||X||_F / sqrt(min(m,n)), 0.7 ||X||_F) with sigma_hat from a few
    power-iteration steps, matching the reference's fast_muon safeguards.
    """
    a, b, c = coeffs
    X = G.float()
    transposed = X.shape[-2] > X.shape[-1]
    if transposed:
        X = X.transpose(-1, -2)
    m = X.shape[-2]
    fro = X.flatten(-2).norm(dim=-1).clamp_min(eps)
    # power iteration for sigma_max (deterministic start vector)
    vec = torch.ones(*X.shape[:-2], X.shape[-1], 1, dtype=X.dtype, device=X.device) / math.sqrt(X.shape[-1])
    for _ in range(4):
        w = X @ vec
        vec = X.transpose(-1, -2) @ w
        vec = vec / vec.norm(dim=-2, keepdim=True).clamp_min(eps)
    sigma = (X @ vec).norm(dim=-2).squeeze(-1)
    safe = torch.maximum(torch.maximum(1.15 * sigma, fro / math.sqrt(m)), 0.7 * fro)
    X = X / safe[..., None, None]
    for _ in range(steps):
        A = X @ X.transpose(-1, -2)
        Bm = b * A + c * (A @ A)
        X = a * X + Bm @ X
    if transposed:
        X = X.transpose(-1, -2)
    return X.to(G.dtype)


def triangular_adamw_core(S, m, v, step: int, lr: float, beta1: float, beta2: float, eps: float, triu: bool):
    """AdamW direction on a batch of (r+1)x(r+1) cores; in place on m, v. Returns delta (same shape)."""
    if triu:
        mask = torch.ones_like(S[0], dtype=torch.bool).triu()
        S = S * mask
    m.mul_(beta1).add_(S, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(S, S, value=1 - beta2)
    mh = m / (1 - beta1**step)
    vh = v / (1 - beta2**step)
    delta = mh / (vh.sqrt() + eps)
    if triu:
        delta = delta * mask
    return delta


def steer_update(P: torch.Tensor, G: torch.Tensor, momentum: float, steer_scale: float) -> torch.Tensor:
    """In place P = momentum * P + steer_scale * (G - P)."""
    return P.copy_(momentum * P + steer_scale * (G - P))


# ----------------------------------------------------------------------------
# Routing tiers / visualisation
# ----------------------------------------------------------------------------
def route_tiers(logits: torch.Tensor, threshold: float = 0.5) -> torch.Tensor:
    """3-way softmax per row then tier pick: p0>=thr -> 0; else p1>=p2 -> 1; else 2."""
    p = torch.softmax(logits.float(), dim=-1)
    tier = torch.where(p[:, 0] >= threshold, 0, torch.where(p[:, 1] >= p[:, 2], 1, 2))
    return tier.to(torch.int32)


def neuron_heatmap(act: torch.Tensor, num_bins: int) -> torch.Tensor:
    """Bin |activation| (flat) into num_bins mean-abs buckets, max-normalise, map to packed ABGR u32."""
    a = act.float().abs().flatten()
    n = a.numel()
    out = torch.zeros(num_bins, dtype=torch.float32)
    if n == 0 or num_bins == 0:
        return torch.zeros(num_bins, dtype=torch.int64)
    per = max(1, n // num_bins)
    for i in range(num_bins):
        s = i * per
        e = n if i == num_bins - 1 else min(n, s + per)
        out[i] = a[s:e].mean() if e > s else 0.0
    mx = out.max().clamp_min(1e-12)
    vn = out / mx
    r = (torch.clamp(1.4 * vn, max=1.0) * 249.0).to(torch.int64)
    gch = (vn * vn * 115.0).to(torch.int64)
    bch = ((1.0 - 0.7 * vn) * 60.0).to(torch.int64)
    return (255 << 24) | (bch << 16) | (gch << 8) | r


TIER_COLOURS = ((0x10, 0xB9, 0x81), (0xF5, 0x9E, 0x0B), (0x8B, 0x5C, 0xF6))  # Reflex, Limbic, Cortex


def tier_colour_render(act: torch.Tensor, tiers: torch.Tensor) -> torch.Tensor:
    """act [rows, width] -> RGBA uint8 [rows, width, 4]; pixel = tier colour * clamp(|act|,0,1)."""
    inten = act.float().abs().clamp(0, 1)
    cols = torch.tensor(TIER_COLOURS, dtype=torch.float32, device=act.device)[tiers.long()]  # [rows,3]
    rgb = (cols[:, None, :] * inten[..., None]).to(torch.uint8)
    alpha = torch.full_like(rgb[..., :1], 255)
    return torch.cat((rgb, alpha), dim=-1)


# ----------------------------------------------------------------------------
# Quantisation codecs
# ----------------------------------------------------------------------------
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def fwht16(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal 16-point Walsh-Hadamard transform over consecutive groups of 16 (an involution)."""
    shape = x.shape
    y = x.float().reshape(-1, 16)
    h = 1
    while h < 16:
        y = y.reshape(-1, 16 // (2 * h), 2, h)
        a, b = y[:, :, 0], y[:, :, 1]
        y = torch.stack((a + b, a - b), dim=2).reshape(-1, 16)
        h *= 2
    return (y * 0.25).reshape(shape).to(x.dtype)


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest E2M1 code (4 bits: sign | 3-bit magnitude index), x already divided by its scale."""
    ax = x.abs()
    thr = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device, dtype=ax.dtype)
    idx = (ax.unsqueeze(-1) > thr).sum(-1).to(torch.uint8)
    return idx | ((x < 0).to(torch.uint8) << 3)


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=code.device)
    mag = lut[(code & 7).long()]
    return torch.where((code & 8) != 0, -mag, mag)


def nvfp4_quantize(w: torch.Tensor, scale_dtype=torch.float8_e4m3fn):
    """[N,K] -> (packed uint8 [N,K/2], block scales [N,K/16] in scale_dtype, fp32 tensor scale).

    True NVFP4: E2M1 values, one E4M3 scale per 16 elements, one fp32 per-tensor scale chosen so the
    largest block scale maps to the E4M3 maximum (448). ``scale_dtype=torch.bfloat16`` gives the
    reference's legacy layout (bf16 block scales, tensor scale 1).
    """
    N, K = w.shape
    assert K % 16 == 0
    wf = w.float().reshape(N, K // 16, 16)
    amax = wf.abs().amax(-1)
    if scale_dtype == torch.bfloat16:
        tscale = torch.ones((), dtype=torch.float32, device=w.device)
        sc = (amax / 6.0).clamp_min(1e-12).to(torch.bfloat16)
    else:
        tscale = (amax.max() / (6.0 * 448.0)).clamp_min(1e-12).float()
        sc = (amax / 6.0 / tscale).clamp(min=2.0**-9, max=448.0).to(scale_dtype)
    eff = sc.float() * tscale
    codes = e2m1_encode(wf / eff.unsqueeze(-1)).reshape(N, K)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return packed.contiguous(), sc.contiguous(), tscale


def nvfp4_dequantize(packed: torch.Tensor, scales: torch.Tensor, tscale, dtype=torch.bfloat16) -> torch.Tensor:
    N, K2 = packed.shape
    lo = e2m1_decode(packed & 0xF)
    hi = e2m1_decode(packed >> 4)
    vals = torch.stack((lo, hi), dim=-1).reshape(N, K2 * 2)
    eff = (scales.float() * float(tscale)).repeat_interleave(16, dim=1)
    return (vals * eff).to(dtype)


def nvfp4_quantize_act(x: torch.Tensor, hadamard: bool = False):
    """Activation side of the W4A4 GEMM: [M,K] -> (packed uint8 [M,K/2], E4M3 scales [M,K/16]) with the block scale
    amax/6 rounded to E4M3 and no tensor scale (activations are O(1) after a normalisation layer)."""
    M, K = x.shape
    xf = (fwht16(x.float()) if hadamard else x.float()).reshape(M, K // 16, 16)
    sc = (xf.abs().amax(-1) / 6.0).clamp(min=2.0**-9, max=448.0).to(torch.float8_e4m3fn)
    codes = e2m1_encode(xf / sc.float().unsqueeze(-1)).reshape(M, K)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous(), sc.contiguous()


def nvfp4_sf_kblocks(K: int) -> int:
    return -(-K // 256) * 4


def mxfp8_sf_kblocks(K: int) -> int:
    return -(-K // 128)


def _block_scale_bytes(scales_u8: torch.Tensor, kblocks: int) -> torch.Tensor:
    """Row-major one-byte scales [R, G] -> the tensor core's blocked layout [ceil(R/128), kblocks, 512] (uint8): per 128
    rows x 4 scale groups, byte (row % 32) * 16 + (row // 32) * 4 + group % 4; missing rows / groups are 0."""
    R, G = scales_u8.shape
    out = torch.zeros((-(-R // 128), kblocks, 512), dtype=torch.uint8, device=scales_u8.device)
    r = torch.arange(R, device=scales_u8.device).unsqueeze(1).expand(R, G)
    b = torch.arange(G, device=scales_u8.device).unsqueeze(0).expand(R, G)
    out[r // 128, b // 4, (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4] = scales_u8
    return out


def _unblock_scale_bytes(blocked: torch.Tensor, R: int, G: int, kblocks: int) -> torch.Tensor:
    r = torch.arange(R, device=blocked.device).unsqueeze(1).expand(R, G)
    b = torch.arange(G, device=blocked.device).unsqueeze(0).expand(R, G)
    flat = blocked.reshape(-(-R // 128), kblocks, 512)
    return flat[r // 128, b // 4, (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4].contiguous()


def nvfp4_block_scales(scales: torch.Tensor, K: int) -> torch.Tensor:
    """Row-major E4M3 scales [R, K/16] -> the blocked layout of the NVFP4 GEMM (blocks of 128 rows x 64 elements)."""
    assert scales.shape[1] == K // 16
    return _block_scale_bytes(scales.view(torch.uint8), nvfp4_sf_kblocks(K))


def nvfp4_unblock_scales(blocked: torch.Tensor, R: int, K: int) -> torch.Tensor:
    """Inverse of :func:`nvfp4_block_scales`: -> E4M3 [R, K/16]."""
    return _unblock_scale_bytes(blocked, R, K // 16, nvfp4_sf_kblocks(K)).view(torch.float8_e4m3fn)


def mxfp8_quantize(x: torch.Tensor):
    """[R,K] -> (E4M3 [R,K], exponent bytes [R,K/32]): one power-of-two scale 2^(byte-127) per 32 elements, the smallest
    that brings the block's largest magnitude under 448 (OCP microscaling MXFP8 with E4M3 elements)."""
    R, K = x.shape
    assert K % 32 == 0
    xf = x.float().reshape(R, K // 32, 32)
    amax = xf.abs().amax(-1)
    # e = ceil(log2(amax / 448)) without a logarithm: amax = m * 2^ex with m in [0.5, 1), 448 = 0.875 * 2^9
    m, ex = torch.frexp(amax.float())
    e = torch.where(amax > 0, (ex - 9 + (m > 0.875).to(ex.dtype)).double(), torch.full_like(amax, -127.0, dtype=torch.float64))
    e = e.clamp(-127, 127)
    q = (xf.double() * torch.exp2(-e).unsqueeze(-1)).float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).reshape(R, K)
    return q.contiguous(), (e + 127).to(torch.uint8).contiguous()


def mxfp8_dequantize(q: torch.Tensor, exps: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    scale = torch.exp2(exps.double() - 127.0).repeat_interleave(32, dim=1)
    return (q.double() * scale).to(dtype)


def mxfp8_block_scales(exps: torch.Tensor, K: int) -> torch.Tensor:
    assert exps.shape[1] == K // 32
    return _block_scale_bytes(exps, mxfp8_sf_kblocks(K))


def mxfp8_unblock_scales(blocked: torch.Tensor, R: int, K: int) -> torch.Tensor:
    return _unblock_scale_bytes(blocked, R, K // 32, mxfp8_sf_kblocks(K))


def mxfp8_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """fp32 oracle of the MXFP8 linear: both operands quantised per 1x32 block, product of the decoded values."""
    xq, xe = mxfp8_quantize(x)
    wq, we = mxfp8_quantize(w)
    return mxfp8_dequantize(xq, xe) @ mxfp8_dequantize(wq, we).t()


def nvfp4_w4a4_linear(x: torch.Tensor, packed, scales, tscale, hadamard: bool = False) -> torch.Tensor:
    """fp32 oracle of the W4A4 linear: both operands decoded from their codes and scales, product in fp32."""
    a_p, a_s = nvfp4_quantize_act(x, hadamard)
    a = nvfp4_dequantize(a_p, a_s, 1.0, torch.float32)
    return a @ nvfp4_dequantize(packed, scales, tscale, torch.float32).t()


def fp8_block_quantize_weight(w: torch.Tensor, block: int = 128):
    """[N,K] -> (E4M3 [N,K], fp32 scales [ceil(N/128), ceil(K/128)]): one scale per 128x128 block."""
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wp = F.pad(w.float(), (0, kb * block - K, 0, nb * block - N)).reshape(nb, block, kb, block)
    amax = wp.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / 448.0
    q = (wp / scale[:, None, :, None]).reshape(nb * block, kb * block)[:N, :K].to(torch.float8_e4m3fn)
    return q.contiguous(), scale.contiguous()


def fp8_block_quantize_act(x: torch.Tensor, block: int = 128):
    """[M,K] -> (E4M3 [M,K], fp32 scales [M, ceil(K/128)]): one scale per 1x128 row segment."""
    M, K = x.shape
    kb = (K + block - 1) // block
    xp = F.pad(x.float(), (0, kb * block - K)).reshape(M, kb, block)
    amax = xp.abs().amax(-1).clamp_min(1e-12)
    scale = amax / 448.0
    q = (xp / scale.unsqueeze(-1)).reshape(M, kb * block)[:, :K].to(torch.float8_e4m3fn)
    return q.contiguous(), scale.contiguous()


def fp8_block_gemm(xq, xs, wq, ws, block: int = 128, out_dtype=torch.bfloat16):
    """Dequantise-and-multiply oracle for the block-scaled FP8 GEMM: y = x @ w^T."""
    x = xq.float() * xs.repeat_interleave(block, dim=1)[:, : xq.shape[1]]
    w = wq.float() * ws.repeat_interleave(block, 0).repeat_interleave(block, 1)[: wq.shape[0], : wq.shape[1]]
    return (x @ w.t()).to(out_dtype)


# ----------------------------------------------------------------------------
# Mixture-of-experts routing
# ----------------------------------------------------------------------------
def moe_route(logits: torch.Tensor, expert_bias: torch.Tensor, top_k: int, temperature=1.0):
    """Top-k on biased logits; mixing weights from the unbiased (temperature) softmax, renormalised.

    Returns (idx [N,k] int64, weights [N,k] fp32, probs [N,E] fp32).
    """
    lf = logits.float()
    probs = torch.softmax(lf / temperature, dim=-1)
    _, idx = torch.topk(lf + expert_bias.float(), top_k, dim=-1)
    w = torch.gather(probs, -1, idx)
    if top_k > 1:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx, w, probs


def moe_capacity_mask(idx: torch.Tensor, w: torch.Tensor, num_experts: int, capacity: int) -> torch.Tensor:
    """Per (k-slot, expert) keep at most ``capacity`` tokens, highest weight first, ties to lower index.

    Returns a bool mask [N,k] of accepted assignments (reference: triune/model/moe.py:385-410).
    """
    N, k = idx.shape
    keep = torch.ones(N, k, dtype=torch.bool, device=idx.device)
    if capacity >= N:
        return keep
    for j in range(k):
        order = torch.argsort(-w[:, j].float(), stable=True)  # by weight, ties by index
        e_sorted = idx[order, j]
        order2 = torch.argsort(e_sorted, stable=True)
        e2 = e_sorted[order2]
        counts = torch.zeros(num_experts, device=idx.device, dtype=torch.int64).scatter_add_(0, e2, torch.ones_like(e2))
        starts = torch.cumsum(counts, 0) - counts
        rank = torch.arange(N, device=idx.device) - starts[e2]
        tok = order[order2]
        keep[tok, j] = rank < capacity
    return keep
