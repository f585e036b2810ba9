"""Chunk-parallel Gated DeltaNet training kernels against the fp64 token recurrence (forward, final state and every
gradient), for head dims 64 and 128, ragged lengths, with and without beta / initial state / a loss on the state."""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _nrel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


@pytest.mark.parametrize("B,T,H,D,with_beta,with_init,state_loss,gate_logits", [
    (1, 64, 1, 64, False, False, False, True),
    (2, 192, 2, 64, True, True, True, True),
    (1, 256, 2, 128, True, False, False, True),
    (2, 128, 1, 128, True, True, True, False),
    (1, 100, 2, 128, True, True, False, True),   # ragged: padded to 128 inside the op
    (1, 200, 1, 64, False, True, True, True),
])
def test_gated_deltanet_chunk_kernels_match_fp64_recurrence(B, T, H, D, with_beta, with_init, state_loss, gate_logits):
    from triune_b200 import ops
    from triune_b200.ops import gla_cuda
    from triune_b200.ops import reference as ref

    dev = torch.device("cuda", 0)
    torch.manual_seed(41)
    q = F.normalize(torch.randn(B, T, H, D, device=dev).abs(), dim=-1).to(torch.bfloat16).requires_grad_(True)
    k = F.normalize(torch.randn(B, T, H, D, device=dev).abs(), dim=-1).to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(B, T, H, D, device=dev).to(torch.bfloat16).requires_grad_(True)
    if gate_logits:
        gx = torch.randn(B, T, H, D, device=dev).to(torch.bfloat16).requires_grad_(True)
    else:
        gx = (-torch.rand(B, T, H, D, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    beta = torch.rand(B, T, H, device=dev).requires_grad_(True) if with_beta else None
    s0 = (torch.randn(B, H, D, D, device=dev) * 0.1).requires_grad_(True) if with_init else None
    w = torch.randn(B, T, H, D, device=dev)
    ws = torch.randn(B, H, D, D, device=dev) * 0.05
    out, fin = ops.gated_deltanet(q, k, v, gx, beta=beta, initial_state=s0, scale=0.5, gate_logits=gate_logits)
    assert int(gla_cuda.last_status.item()) == 0
    loss = (out.float() * w).sum() + ((fin * ws).sum() if state_loss else 0.0)
    loss.backward()
    assert int(gla_cuda.last_status.item()) == 0

    dt = torch.float64
    qf, kf, vf, gf = (t.detach().to(dt).requires_grad_(True) for t in (q, k, v, gx))
    bf = beta.detach().to(dt).requires_grad_(True) if with_beta else None
    sf = s0.detach().to(dt).requires_grad_(True) if with_init else None
    gl = torch.clamp(F.logsigmoid(gf) if gate_logits else gf, min=-5.0, max=0.0)
    o_ref, f_ref = ref.gated_deltanet_recurrent(qf, kf, vf, gl, bf, sf, 0.5)
    l_ref = (o_ref * w.to(dt)).sum() + ((f_ref * ws.to(dt)).sum() if state_loss else 0.0)
    l_ref.backward()

    assert _nrel(out, o_ref) < 2e-2
    assert _nrel(fin, f_ref) < 5e-3
    pairs = [(q.grad, qf.grad, "dq"), (k.grad, kf.grad, "dk"), (v.grad, vf.grad, "dv"), (gx.grad, gf.grad, "dg")]
    if with_beta:
        pairs.append((beta.grad, bf.grad, "dbeta"))
    if with_init:
        pairs.append((s0.grad, sf.grad, "ds0"))
    for a, b_, name in pairs:
        assert a is not None, name
        # The gate gradient is a suffix sum of q dq - k dk_w + k dk_r: a difference of terms of equal size, so the
        # bf16 rounding of the chunk intermediates (about 4e-3 on dq and dk) shows up several times larger there.
        assert _nrel(a, b_) < (8e-2 if name == "dg" else 2e-2), (name, _nrel(a, b_))


def test_gated_deltanet_layer_trains_on_the_chunk_kernels():
    """The dense family's delta-rule mixer (learned beta) takes the kernel path under autograd and agrees with the
    PyTorch operators on output and parameter gradients."""
    from triune_b200 import _ext
    from triune_b200.models import VectorisedGLA

    dev = torch.device("cuda", 0)
    torch.manual_seed(42)
    layer = VectorisedGLA(256, 2, 128, use_delta_rule=True, learn_beta=True).to(dev).to(torch.bfloat16)
    x = torch.randn(2, 192, 256, device=dev).to(torch.bfloat16)
    res = []
    for mode in (False, True):
        _ext.set_reference_ops(mode)
        try:
            xx = x.clone().requires_grad_(True)
            layer.zero_grad()
            y, _ = layer(xx)
            (y.float() ** 2).sum().backward()
            res.append((y.float(), xx.grad.float(), layer.qkvg_weight.grad.float().clone(),
                        layer.beta_proj.weight.grad.float().clone()))
        finally:
            _ext.set_reference_ops(False)
    assert _nrel(res[0][0], res[1][0]) < 3e-2
    assert _nrel(res[0][1], res[1][1]) < 6e-2
    assert _nrel(res[0][2], res[1][2]) < 6e-2
    assert _nrel(res[0][3], res[1][3]) < 8e-2
