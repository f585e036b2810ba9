"""CPU oracles: chunked forms vs token recurrences, codecs, optimizer math."""

import math

import pytest
import torch
import torch.nn.functional as F

from triune_b200.ops import reference as ref


@pytest.mark.parametrize("T", [1, 17, 32, 70, 128])
@pytest.mark.parametrize("with_state", [False, True])
def test_gla_chunk_matches_recurrence(T, with_state):
    torch.manual_seed(T)
    B, H, D = 2, 2, 16
    q, k, v = (torch.randn(B, T, H, D, dtype=torch.float64) for _ in range(3))
    g = F.logsigmoid(torch.randn(B, T, H, D, dtype=torch.float64) * 2)
    s0 = torch.randn(B, H, D, D, dtype=torch.float64) if with_state else None
    o1, s1 = ref.gla_recurrent(q, k, v, g, s0)
    o2, s2 = ref.gla_chunk(q, k, v, g, s0, chunk_size=32)
    assert (o1 - o2).abs().max() < 1e-9 and (s1 - s2).abs().max() < 1e-9


def test_gla_extreme_decay_is_finite_and_exact():
    torch.manual_seed(0)
    B, T, H, D = 1, 96, 1, 8
    q, k, v = (torch.randn(B, T, H, D, dtype=torch.float64) for _ in range(3))
    g = torch.full((B, T, H, D), -20.0, dtype=torch.float64)
    o1, _ = ref.gla_recurrent(q, k, v, g)
    o2, _ = ref.gla_chunk(q, k, v, g)
    assert torch.isfinite(o2).all() and (o1 - o2).abs().max() < 1e-9


def test_gla_grads_flow():
    torch.manual_seed(1)
    B, T, H, D = 1, 40, 1, 8
    q, k, v = (torch.randn(B, T, H, D, dtype=torch.float64, requires_grad=True) for _ in range(3))
    g = (-torch.rand(B, T, H, D, dtype=torch.float64)).requires_grad_(True)
    o, s = ref.gla_chunk(q, k, v, g, chunk_size=16)
    (o.sum() + s.sum()).backward()
    o2, s2 = ref.gla_recurrent(q.detach().requires_grad_(True), k, v, g)
    assert all(t.grad is not None and torch.isfinite(t.grad).all() for t in (q, k, v, g))


@pytest.mark.parametrize("beta_kind", [None, "head"])
def test_gated_deltanet_chunk_matches_recurrence(beta_kind):
    torch.manual_seed(2)
    B, T, H, D = 2, 75, 2, 16
    q, v = (torch.randn(B, T, H, D, dtype=torch.float64) for _ in range(2))
    k = F.normalize(torch.randn(B, T, H, D, dtype=torch.float64), dim=-1)
    g = F.logsigmoid(torch.randn(B, T, H, D, dtype=torch.float64) * 2)
    beta = torch.rand(B, T, H, dtype=torch.float64) if beta_kind else None
    s0 = torch.randn(B, H, D, D, dtype=torch.float64)
    o1, s1 = ref.gated_deltanet_recurrent(q, k, v, g, beta, s0)
    o2, s2 = ref.gated_deltanet_chunk(q, k, v, g, beta, s0, chunk_size=32)
    assert (o1 - o2).abs().max() < 1e-8 and (s1 - s2).abs().max() < 1e-8


@pytest.mark.parametrize("beta_kind,T", [(None, 128), ("head", 75), ("head", 200)])
def test_gated_deltanet_parallel_form_matches_recurrence_with_gradients(beta_kind, T):
    """The chunk-parallel WY form (the training path) against the token recurrence: outputs, final state and the
    gradients of q, k, v, g, for whole and ragged numbers of chunks."""
    torch.manual_seed(4)
    B, H, D, Dv = 2, 2, 16, 24
    q = torch.randn(B, T, H, D, dtype=torch.float64) * 0.5
    k = F.normalize(torch.randn(B, T, H, D, dtype=torch.float64), dim=-1)
    v = torch.randn(B, T, H, Dv, dtype=torch.float64)
    g = F.logsigmoid(torch.randn(B, T, H, D, dtype=torch.float64) * 2)
    beta = torch.rand(B, T, H, dtype=torch.float64) if beta_kind else None
    s0 = torch.randn(B, H, D, Dv, dtype=torch.float64) * 0.1
    a = [t.clone().requires_grad_(True) for t in (q, k, v, g)]
    b = [t.clone().requires_grad_(True) for t in (q, k, v, g)]
    o1, s1 = ref.gated_deltanet_recurrent(*a, beta, s0, 0.7)
    o2, s2 = ref.gated_deltanet_chunk_parallel(*b, beta, s0, 0.7, chunk_size=64)
    do, ds = torch.randn_like(o1), torch.randn_like(s1)
    ((o1 * do).sum() + (s1 * ds).sum()).backward()
    ((o2 * do).sum() + (s2 * ds).sum()).backward()
    assert (o1 - o2).abs().max() < 1e-9 and (s1 - s2).abs().max() < 1e-9
    for x, y in zip(a, b):
        assert (x.grad - y.grad).abs().max() < 1e-8


def test_decode_step_matches_recurrence():
    torch.manual_seed(3)
    B, T, H, D = 2, 5, 2, 8
    q, k, v = (torch.randn(B, T, H, D) for _ in range(3))
    g = F.logsigmoid(torch.randn(B, T, H, D))
    o, s = ref.gla_recurrent(q, k, v, g)
    st = torch.zeros(B, H, D, D)
    for t in range(T):
        ot, st = ref.gla_decode_step(q[:, t], k[:, t], v[:, t], g[:, t], st)
        assert (ot - o[:, t]).abs().max() < 1e-5
    assert (st - s).abs().max() < 1e-5


def test_linear_cross_entropy_matches_dense():
    torch.manual_seed(4)
    h = torch.randn(50, 16, dtype=torch.float64, requires_grad=True)
    w = torch.randn(37, 16, dtype=torch.float64, requires_grad=True)
    t = torch.randint(0, 37, (50,))
    t[::5] = -100
    loss, nv = ref.linear_cross_entropy(h, w, t, chunk=16)
    loss.backward()
    h2, w2 = h.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    F.cross_entropy(F.linear(h2, w2), t, ignore_index=-100).backward()
    assert (h.grad - h2.grad).abs().max() < 1e-6 and (w.grad - w2.grad).abs().max() < 1e-6


def test_newton_schulz_semiorthogonal_and_input_untouched():
    torch.manual_seed(5)
    G = torch.randn(3, 24, 60)
    G0 = G.clone()
    X = ref.newton_schulz(G, steps=10)
    assert torch.equal(G, G0)
    assert (X @ X.transpose(1, 2) - torch.eye(24)).abs().max() < 1e-3
    Xt = ref.newton_schulz(G.transpose(1, 2).contiguous(), steps=10)
    assert (Xt.transpose(1, 2) - X).abs().max() < 1e-3


def test_triangular_adamw_equals_dense_on_triangular_core():
    torch.manual_seed(6)
    S = torch.randn(2, 9, 9).triu()
    m1, v1, m2, v2 = (torch.zeros_like(S) for _ in range(4))
    d1 = ref.triangular_adamw_core(S, m1, v1, 1, 1.0, 0.9, 0.999, 1e-8, True)
    d2 = ref.triangular_adamw_core(S, m2, v2, 1, 1.0, 0.9, 0.999, 1e-8, False)
    assert (d1 - d2.triu()).abs().max() < 1e-6
    assert d1.tril(-1).abs().max() == 0
    noisy = S + 1e-4 * torch.randn(2, 9, 9).tril(-1)
    d3 = ref.triangular_adamw_core(noisy, torch.zeros_like(S), torch.zeros_like(S), 1, 1.0, 0.9, 0.999, 1e-8, False)
    assert d3.tril(-1).abs().max() > 0.5  # unconstrained Adam amplifies sub-diagonal noise to O(1) steps


def test_nvfp4_codec_and_fwht():
    torch.manual_seed(7)
    x = torch.randn(8, 64)
    assert (ref.fwht16(ref.fwht16(x)) - x).abs().max() < 1e-5
    codes = torch.arange(16, dtype=torch.uint8)
    vals = ref.e2m1_decode(codes)
    assert torch.equal(ref.e2m1_encode(vals) & 7, codes & 7)
    w = torch.randn(64, 128)
    for sd in (torch.float8_e4m3fn, torch.bfloat16):
        p, s, t = ref.nvfp4_quantize(w, sd)
        assert p.shape == (64, 64) and s.shape == (64, 8)
        wd = ref.nvfp4_dequantize(p, s, t, torch.float32)
        assert F.cosine_similarity(w.flatten(), wd.flatten(), dim=0) > 0.95


def test_nvfp4_w4a4_oracle_and_blocked_scale_layout():
    torch.manual_seed(9)
    x, w = torch.randn(200, 384), torch.randn(136, 384) * 0.05
    p, s, t = ref.nvfp4_quantize(w)
    for hadamard in (False, True):
        pw, sw, tw = ref.nvfp4_quantize(ref.fwht16(w) if hadamard else w)
        y = ref.nvfp4_w4a4_linear(x, pw, sw, tw, hadamard)
        assert F.cosine_similarity(y.flatten(), (x @ w.t()).flatten(), dim=0) > 0.97
    blocked = ref.nvfp4_block_scales(s, 384)
    assert blocked.shape == (2, 8, 512)  # 136 rows -> 2 row blocks; K = 384 -> 2 stages of 256 -> 8 blocks of 64
    assert torch.equal(ref.nvfp4_unblock_scales(blocked, 136, 384).view(torch.uint8), s.view(torch.uint8))
    # row 101 (row block 0), k block 5 (k = 80..95): block 5 // 4 = 1, byte (101 % 32) * 16 + (101 // 32) * 4 + 5 % 4
    assert blocked[0, 1, 5 * 16 + 3 * 4 + 1] == s.view(torch.uint8)[101, 5]
    assert int(blocked[1, :, :].view(-1).count_nonzero()) <= 8 * 24  # rows 136.. and k blocks 6, 7 stay zero


def test_mxfp8_codec_and_oracle():
    torch.manual_seed(10)
    x = torch.randn(70, 96) * torch.logspace(-3, 3, 96)
    x[3] = 0
    q, e = ref.mxfp8_quantize(x)
    assert q.dtype == torch.float8_e4m3fn and e.shape == (70, 3) and e.dtype == torch.uint8
    assert float(q.float().abs().max()) <= 448.0
    # the scale is the SMALLEST power of two that fits: the block maximum lands in (224, 448]
    top = q.float().abs().reshape(70, 3, 32).amax(-1)
    assert bool(((top > 224 - 16) | (top == 0)).all())
    deq = ref.mxfp8_dequantize(q, e)
    assert (deq - x).abs().max() <= 0.0625 * x.abs().max()
    assert torch.equal(deq[3], torch.zeros(96))
    blocked = ref.mxfp8_block_scales(e, 96)
    assert blocked.shape == (1, 1, 512) and torch.equal(ref.mxfp8_unblock_scales(blocked, 70, 96), e)
    w = torch.randn(40, 96) * 0.05
    y = ref.mxfp8_linear(x, w)
    assert F.cosine_similarity(y.flatten(), (x @ w.t()).flatten(), dim=0) > 0.998


def test_fp8_block_quant_roundtrip():
    torch.manual_seed(8)
    x, w = torch.randn(50, 300), torch.randn(130, 300)
    xq, xs = ref.fp8_block_quantize_act(x)
    wq, ws = ref.fp8_block_quantize_weight(w)
    y = ref.fp8_block_gemm(xq, xs, wq, ws, out_dtype=torch.float32)
    assert F.cosine_similarity(y.flatten(), (x @ w.t()).flatten(), dim=0) > 0.995


def test_route_tiers_and_heatmap():
    lg = torch.tensor([[5.0, 0.0, 0.0], [0.0, 2.0, 1.0], [0.0, 1.0, 2.0]])
    assert ref.route_tiers(lg, 0.5).tolist() == [0, 1, 2]
    hm = ref.neuron_heatmap(torch.linspace(0, 1, 640), 64)
    assert hm.shape == (64,) and int(hm[-1]) >> 24 == 255


def test_moe_capacity_mask_priority():
    idx = torch.tensor([[0], [0], [0], [1]])
    w = torch.tensor([[0.2], [0.9], [0.5], [0.1]])
    keep = ref.moe_capacity_mask(idx, w, 2, 2)
    assert keep[:, 0].tolist() == [False, True, True, True]


def test_gla_final_state_gradient_matches_autograd():
    """The analytic gradient of the final state (for kernels that return it without one) equals autograd through the
    token recurrence, for keys, values, log decays and the initial state."""
    from triune_b200 import ops

    torch.manual_seed(0)
    B, T, H, D = 2, 37, 2, 8
    q, k, v = (torch.randn(B, T, H, D, dtype=torch.float64) for _ in range(3))
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, D, dtype=torch.float64))
    s0 = torch.randn(B, H, D, D, dtype=torch.float64)
    for use_s0 in (True, False):
        a = [t.clone().requires_grad_(True) for t in (k, v, g, s0)]
        _, sf = ref.gla_recurrent(q, a[0], a[1], a[2], a[3] if use_s0 else None, 1.0)
        G = torch.randn_like(sf)
        want = torch.autograd.grad((sf * G).sum(), a[:3] + ([a[3]] if use_s0 else []))
        b = [t.clone().requires_grad_(True) for t in (k, v, g, s0)]
        sf2 = ops.gla_final_state_with_grad(b[0], b[1], b[2], b[3] if use_s0 else None, sf.detach())
        assert torch.equal(sf2, sf.detach())
        got = torch.autograd.grad((sf2 * G).sum(), b[:3] + ([b[3]] if use_s0 else []))
        for x, y in zip(want, got):
            assert (x - y).abs().max() < 1e-10


@pytest.mark.parametrize("B,T,H,D,with_beta,with_s0,state_loss", [(2, 100, 2, 16, True, True, True),
                                                                   (1, 64, 1, 8, False, False, False),
                                                                   (1, 130, 2, 16, True, False, True)])
def test_gated_deltanet_stage_algebra_matches_autograd_of_the_recurrence(B, T, H, D, with_beta, with_s0, state_loss):
    """The stage-wise forward / backward that the CUDA kernels implement (UT transform, state pass, outputs and the
    hand-derived backward with the global decay-gradient identity) equals autograd through the token recurrence."""
    from triune_b200.ops import reference as ref
    from triune_b200.ops.gdn_stages import gated_deltanet_chunked

    torch.manual_seed(0)
    dt = torch.float64
    q = torch.randn(B, T, H, D, dtype=dt).requires_grad_(True)
    k = (torch.randn(B, T, H, D, dtype=dt) * 0.4).requires_grad_(True)
    v = torch.randn(B, T, H, D, dtype=dt).requires_grad_(True)
    g = (-torch.rand(B, T, H, D, dtype=dt) * 1.5).requires_grad_(True)
    beta = torch.rand(B, T, H, dtype=dt).requires_grad_(True) if with_beta else None
    s0 = (torch.randn(B, H, D, D, dtype=dt) * 0.3).requires_grad_(True) if with_s0 else None
    w, ws = torch.randn(B, T, H, D, dtype=dt), torch.randn(B, H, D, D, dtype=dt)
    ins = [t for t in (q, k, v, g, beta, s0) if t is not None]
    o1, f1 = ref.gated_deltanet_recurrent(q, k, v, g, beta, s0, 0.7)
    g1 = torch.autograd.grad((o1 * w).sum() + ((f1 * ws).sum() if state_loss else 0.0), ins)
    o2, f2 = gated_deltanet_chunked(q, k, v, g, beta, s0, 0.7, 32)
    g2 = torch.autograd.grad((o2 * w).sum() + ((f2 * ws).sum() if state_loss else 0.0), ins)
    assert (o1 - o2).abs().max() < 1e-10 and (f1 - f2).abs().max() < 1e-10
    for a, b in zip(g1, g2):
        assert (a - b).abs().max() < 1e-9
