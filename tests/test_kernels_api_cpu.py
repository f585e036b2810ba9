"""The reference's kernel-level API names on this framework's operators (CPU: the PyTorch paths), against plain PyTorch."""

import math

import pytest
import torch
import torch.nn.functional as F

from triune_b200 import kernels as K


def test_every_name_of_the_reference_kernel_package_exists():
    names = """is_triton_available get_kernel_backend get_triton_error is_turbo_mode_enabled set_turbo_mode get_kernel_telemetry fast_rmsnorm
    fast_fused_add_rmsnorm FastRMSNorm fast_rope fast_swiglu fast_gelu FastSwiGLU FastGELU fast_cross_entropy chunked_cross_entropy_from_hidden
    FastChunkedCrossEntropyLoss fast_chunk_gla fast_chunk_gated_deltanet fast_recurrent_gated_deltanet fast_zeropower_via_newtonschulz5
    fast_lora_forward fast_lora_linear fast_qkv_lora_linear fast_gate_up_lora_linear is_fp8_available fast_fp8_linear FastFP8Linear nvfp4_quantize
    nvfp4_dequantize nvfp4_linear fwht_16 NVFP4Linear""".split()
    assert sorted(names) == sorted(K.__all__) and all(hasattr(K, n) for n in names)
    assert K.is_triton_available() is False and "Triton" in K.get_triton_error()
    assert K.get_kernel_backend() == "pytorch"  # no GPU here
    assert K.set_turbo_mode(False) is False and K.is_turbo_mode_enabled() is False
    assert K.set_turbo_mode(True) is True and K.get_kernel_telemetry()["turbo_mode"] is True
    assert K.is_fp8_available(torch.device("cpu")) is False


def test_norms_activations_and_rope():
    torch.manual_seed(0)
    x, r, w = torch.randn(3, 5, 32), torch.randn(3, 5, 32), torch.rand(32) + 0.5
    want = F.rms_norm(x, (32,), w, 1e-6)
    assert torch.allclose(K.fast_rmsnorm(x, w), want, atol=1e-5)
    y, s = K.fast_fused_add_rmsnorm(x, r, w)
    assert torch.allclose(s, x + r) and torch.allclose(y, F.rms_norm(x + r, (32,), w, 1e-6), atol=1e-5)
    y, s = K.fast_fused_add_rmsnorm(x, None, w)
    assert s is x and torch.allclose(y, want, atol=1e-5)
    mod = K.FastRMSNorm(32)
    assert torch.allclose(mod(x), F.rms_norm(x, (32,), torch.ones(32), 1e-6), atol=1e-5) and isinstance(mod(x, r), tuple)
    g, u = torch.randn(4, 16), torch.randn(4, 16)
    assert torch.allclose(K.fast_swiglu(g, u), F.silu(g) * u, atol=1e-6) and torch.allclose(K.FastSwiGLU()(g, u), F.silu(g) * u, atol=1e-6)
    assert torch.allclose(K.fast_gelu(g), F.gelu(g, approximate="tanh"), atol=1e-6)
    assert torch.allclose(K.FastGELU()(g), F.gelu(g, approximate="tanh"), atol=1e-6)
    assert torch.allclose(K.FastGELU("none")(g), F.gelu(g), atol=1e-6)
    # head-major rotary: pairs (i, i + D/2) rotate by t * base^(-2i/D)
    B, H, T, D = 2, 3, 7, 8
    q, k = torch.randn(B, H, T, D), torch.randn(B, H, T, D)
    inv = 10000.0 ** (-torch.arange(0, D, 2).float() / D)
    ang = torch.arange(T).float()[:, None] * inv[None]
    cos, sin = ang.cos(), ang.sin()  # [T, D/2]
    qr, kr = K.fast_rope(q, k, cos, sin)
    want_q = torch.cat((q[..., : D // 2] * cos - q[..., D // 2:] * sin, q[..., : D // 2] * sin + q[..., D // 2:] * cos), dim=-1)
    assert qr.shape == q.shape and torch.allclose(qr, want_q, atol=1e-5)
    qr2, _ = K.fast_rope(q, k, torch.cat((cos, cos), -1)[None, None], torch.cat((sin, sin), -1)[None, None])  # [1, 1, T, D] tables
    assert torch.allclose(qr2, want_q, atol=1e-5) and torch.allclose(kr.norm(dim=-1), k.norm(dim=-1), atol=1e-5)


def test_cross_entropy_forms():
    torch.manual_seed(1)
    h = torch.randn(2, 9, 16, requires_grad=True)
    head = torch.nn.Linear(16, 50)
    y = torch.randint(0, 50, (2, 9))
    y[0, :3] = -100
    want = F.cross_entropy(head(h).reshape(-1, 50), y.reshape(-1), ignore_index=-100)
    assert torch.allclose(K.fast_cross_entropy(head(h), y), want, atol=1e-5)
    got = K.chunked_cross_entropy_from_hidden(h, head, y, chunk_size=4, force_chunked=True)
    assert torch.allclose(got, want, atol=1e-5)
    got.backward()
    g1 = h.grad.clone()
    h.grad = None
    want.backward()
    assert torch.allclose(g1, h.grad, atol=1e-5)
    assert torch.allclose(K.chunked_cross_entropy_from_hidden(h, head.weight, y), F.cross_entropy(F.linear(h, head.weight).reshape(-1, 50), y.reshape(-1)), atol=1e-5)
    loss = K.FastChunkedCrossEntropyLoss(chunk_size=4)
    assert torch.allclose(loss(h, y, head), want, atol=1e-5) and torch.allclose(loss(head(h), y), want, atol=1e-5)


def test_sequence_mixers_against_the_token_recurrence():
    torch.manual_seed(2)
    B, T, H, D = 1, 70, 2, 64
    q, k, v = (torch.randn(B, T, H, D) * 0.3 for _ in range(3))
    g = -torch.rand(B, T, H, D) * 0.2
    s0 = torch.randn(B, H, D, D) * 0.1
    o, s = K.fast_chunk_gla(q, k, v, g, initial_state=s0)
    S = s0.clone()
    outs = []
    for t in range(T):  # S <- diag(exp(g_t)) S + k_t v_t^T ; o_t = q_t S
        S = S * g[:, t].exp().unsqueeze(-1) + k[:, t].unsqueeze(-1) * v[:, t].unsqueeze(-2)
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, t], S))
    assert torch.allclose(o, torch.stack(outs, 1), atol=1e-4) and torch.allclose(s, S, atol=1e-4)
    buf = torch.empty_like(o)
    o2, _ = K.fast_chunk_gla(q, k, v, g, initial_state=s0, out=buf)
    assert o2 is buf and torch.allclose(buf, o)
    beta = torch.rand(B, T, H)
    kn = F.normalize(k, dim=-1)  # the delta rule wants unit keys
    oc, sc = K.fast_chunk_gated_deltanet(q, kn, v, g, beta)
    orr, sr = K.fast_recurrent_gated_deltanet(q, kn, v, g, beta)
    assert oc.shape == (B, T, H, D) and torch.allclose(oc, orr, atol=1e-4) and torch.allclose(sc, sr, atol=1e-4)


def test_newton_schulz_and_lora():
    torch.manual_seed(3)
    G = torch.randn(3, 16, 24)
    X = K.fast_zeropower_via_newtonschulz5(G, steps=8)
    sv = torch.linalg.svdvals(X.float())
    assert X.shape == G.shape and float(sv.max()) < 1.3 and float(sv.min()) > 0.5  # singular values pushed towards 1
    X2, scratch = K.fast_zeropower_via_newtonschulz5(G, steps=8, scratch_buffer="mine", return_scratch=True)
    assert scratch == "mine" and torch.allclose(X2, X)
    x, W, b = torch.randn(5, 12), torch.randn(7, 12), torch.randn(7)
    A, Bm = torch.randn(3, 12), torch.randn(7, 3)
    low = (x @ A.t()) @ Bm.t()
    assert torch.allclose(K.fast_lora_forward(x, A, Bm, 2.0), 2.0 * low, atol=1e-5)
    assert torch.allclose(K.fast_lora_linear(x, W, b, A, Bm, 0.5), x @ W.t() + b + 0.5 * low, atol=1e-5)
    qkv = K.fast_qkv_lora_linear(x, W, b, W, None, W, b, A, Bm, A, Bm, A, Bm, 1.0)
    assert qkv.shape == (5, 21) and torch.allclose(qkv[:, 7:14], x @ W.t() + low, atol=1e-5)
    gu = K.fast_gate_up_lora_linear(x, W, None, W, b, A, Bm, A, Bm, 1.0)
    assert torch.allclose(gu, F.silu(x @ W.t() + low) * (x @ W.t() + b + low), atol=1e-5)


def test_fp8_and_nvfp4_layers():
    torch.manual_seed(4)
    x = torch.randn(6, 128)
    lin = torch.nn.Linear(128, 64)
    y0 = lin(x)
    rel = lambda a, b: float((a - b).norm() / b.norm())
    assert rel(K.fast_fp8_linear(x, lin.weight, lin.bias), y0) < 0.06
    f8 = K.FastFP8Linear(128, 64)
    with torch.no_grad():
        f8.weight.copy_(lin.weight)
        f8.bias.copy_(lin.bias)
    assert torch.allclose(f8.train()(x), y0, atol=1e-5)      # training: the plain product
    assert rel(f8.eval()(x), y0) < 0.06 and f8._q is not None  # evaluation: through the E4M3 weight
    w = torch.randn(32, 64)
    packed, scale = K.nvfp4_quantize(w)
    assert packed.shape == (32, 32) and packed.dtype == torch.uint8 and scale.shape == (32, 4) and scale.dtype == torch.bfloat16
    wd = K.nvfp4_dequantize(packed, scale, torch.float32)
    assert rel(wd, w) < 0.15
    x2 = torch.randn(5, 64)
    assert torch.allclose(K.nvfp4_linear(x2, packed, scale, bias=torch.ones(32)), x2 @ wd.t() + 1.0, atol=1e-3)
    # rotated basis: quantise W H, feed x H; H is orthonormal, so the product is that of the unrotated weight up to rounding
    ph, sh = K.nvfp4_quantize(K.fwht_16(w))
    assert rel(K.nvfp4_linear(x2, ph, sh, hadamard=True), x2 @ w.t()) < 0.2
    assert torch.allclose(K.fwht_16(K.fwht_16(w)), w, atol=1e-5)
    q = K.NVFP4Linear.from_linear(torch.nn.Linear(64, 32, bias=False), hadamard=False)
    assert q(x2).shape == (5, 32) and q.in_features == 64
    q2 = K.NVFP4Linear(64, 32)
    assert q2(x2).shape == (5, 32)
