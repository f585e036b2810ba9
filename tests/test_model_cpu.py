"""Model semantics on CPU: parameter counts, checkpoint keys, caches, MoE parity, optimizer tiers."""

import os
import sys

import pytest
import torch

from triune_b200.config import ModelConfig, build_config, get_model_config, validate_config
from triune_b200.models import MoE_FFN, TriuneTransformer
from triune_b200.optim import CentroidSteerOptimizer, batched_qr


def tiny(**kw):
    base = dict(vocab_size=256, hidden_dim=64, num_layers=5, num_heads=2, head_dim=32, num_experts=4, top_k=2,
                router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3, expert_hidden=96, dense_hidden=96)
    base.update(kw)
    return ModelConfig(**base)


def test_triune_base_param_count_is_exact():
    cfg = get_model_config("triune-base")
    assert cfg.param_count()[0] == 90_789_271


def test_bench_config_param_count_matches_module():
    cfg = tiny()
    m = TriuneTransformer.from_config(cfg)
    assert m.num_parameters() == cfg.param_count()[0]


def test_state_dict_uses_reference_key_layout():
    m = TriuneTransformer.from_config(tiny())
    keys = set(m.state_dict())
    for k in ("token_embed.weight", "final_head.weight", "final_norm.weight", "router.router_mlp.0.weight",
              "router.target_dist", "router.router_bias", "layers.0.attn.gla.q_proj.weight",
              "layers.0.attn.gla.out_proj.weight", "layers.0.norm1.weight", "layers.0.ffn.0.weight", "layers.0.ffn.2.bias",
              "layers.3.ffn.experts.0.0.weight", "layers.3.ffn.experts.3.2.bias", "layers.3.ffn.shared.0.weight",
              "layers.3.ffn.router.weight", "layers.3.ffn.expert_bias", "layers.3.ffn.expert_load_ratio",
              "layers.3.ffn.last_centroids", "layers.3.ffn._global_step", "layers.2.exit_norm.weight",
              "layers.2.exit_head.bias"):
        assert k in keys, k
    assert not any("qkvg_weight" in k or k.endswith(".w1") for k in keys)
    m2 = TriuneTransformer.from_config(tiny())
    m2.load_state_dict(m.state_dict())
    x = torch.randint(0, 256, (2, 20))
    m.eval(), m2.eval()
    assert torch.equal(m(x, force_depth=2)[0], m2(x, force_depth=2)[0])


def test_reference_checkpoint_keys_match_when_reference_is_installed():
    ref_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "triune")):
        pytest.skip("reference not installed")
    sys.path.insert(0, ref_dir)
    try:
        from triune.model.transformer import TriuneTransformer as Ref
    except Exception as e:  # pragma: no cover
        pytest.skip(f"reference import failed: {e}")
    finally:
        sys.path.remove(ref_dir)
    ref = Ref(vocab_size=256, hidden_dim=64, num_layers=5, num_heads=2, head_dim=32, num_experts=4,
              router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3)
    ours = TriuneTransformer(vocab_size=256, hidden_dim=64, num_layers=5, num_heads=2, head_dim=32, num_experts=4,
                             router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3)
    rs, os_ = ref.state_dict(), ours.state_dict()
    assert set(rs) == set(os_)
    assert all(rs[k].shape == os_[k].shape for k in rs)
    ours.load_state_dict(rs)
    ref.eval(), ours.eval()
    x = torch.randint(0, 256, (2, 24))
    with torch.no_grad():
        a = ref(x, force_depth=2)[0]
        b = ours(x, force_depth=2)[0]
    assert (a - b).abs().max() < 2e-3


@pytest.mark.parametrize("depth", [0, 1, 2])
def test_cached_forward_equals_uncached(depth):
    torch.manual_seed(0)
    m = TriuneTransformer.from_config(tiny()).eval()
    x = torch.randint(0, 256, (2, 50))
    with torch.no_grad():
        full = m(x, force_depth=depth)[0]
        c = m.init_cache(2)
        a, c = m(x[:, :33], force_depth=depth, cache=c)
        outs = [a]
        for t in range(33, 50):
            o, c = m(x[:, t : t + 1], force_depth=depth, cache=c)
            outs.append(o)
    assert (torch.cat(outs, 1) - full).abs().max() < 1e-3


def test_sparse_moe_equals_dense_evaluation():
    torch.manual_seed(1)
    moe = MoE_FFN(64, num_experts=4, top_k=2, expert_hidden=96).eval()
    x = torch.randn(2, 30, 64)
    with torch.no_grad():
        assert (moe(x) - moe.dense_forward(x)).abs().max() < 1e-5


def test_moe_bias_update_and_capacity_stats():
    torch.manual_seed(2)
    moe = MoE_FFN(32, num_experts=4, top_k=1, expert_hidden=48).train()
    moe.router.bias.data[0] = 5.0  # overload expert 0
    x = torch.randn(1, 64, 32)
    moe(x)
    assert int(moe.last_dropped_counts.sum()) > 0 and moe.overflow_counter > 0
    moe.step_bias()
    assert moe.expert_bias[0] < 0 and moe._pending_bias_update is None


def test_dynamic_and_calm_forward_shapes():
    torch.manual_seed(3)
    m = TriuneTransformer.from_config(tiny()).eval()
    x = torch.randint(0, 256, (3, 24))
    with torch.no_grad():
        lg, rl = m(x)
        assert lg.shape == (3, 24, 256) and rl.shape == (3, 3)
        cortex = m(x, force_depth=2)[0]
        lg2, _ = m(x, exit_policy="calm", confidence_threshold=2.0)  # nothing can settle -> all Cortex
        assert (lg2 - cortex).abs().max() < 1e-4 and int(m.last_calm_exit_depths.min()) == 2
        lg3, _ = m(x, exit_policy="calm", confidence_threshold=0.0)  # everything settles at Reflex
        assert (lg3 - m(x, force_depth=0)[0]).abs().max() < 1e-5
        r, l, c, _ = m.forward_all_exits(x)
        assert (c - cortex).abs().max() < 1e-5


def test_config_validation():
    with pytest.raises(ValueError):
        validate_config({"use_fp4": True, "use_fp8": True})
    with pytest.raises(ValueError):
        validate_config({"lr": float("nan")})
    with pytest.raises(ValueError):
        TriuneTransformer(vocab_size=10, hidden_dim=64, num_layers=4, num_heads=2, head_dim=32, router_prefix_layers=2,
                          reflex_exit_layer=1, limbic_exit_layer=3)
    cfg = build_config({"lr": 1e-3}, preset="triune-base")
    assert cfg["hidden_dim"] == 384 and cfg["lr"] == 1e-3


def test_three_tier_partition_and_training_progress():
    torch.manual_seed(4)
    m = TriuneTransformer.from_config(tiny())
    opt = CentroidSteerOptimizer(m, lr=3e-3, rank=8, grad_clip=1.0)
    tiers = {s.name: s.tier for s in opt.arena.segments}
    assert tiers["token_embed.weight"] == "adamw" and tiers["layers.2.exit_head.weight"] == "adamw"
    assert tiers["layers.3.ffn.router.weight"] == "adamw" and tiers["layers.0.norm1.weight"] == "adamw"
    assert tiers["layers.3.ffn.w1"] == "steer" and tiers["layers.3.ffn.w2"] == "steer"
    assert tiers["layers.0.attn.gla.qkvg_weight"] == "muon" and tiers["layers.0.attn.gla.out_proj.weight"] == "muon"
    x = torch.randint(0, 256, (4, 33))
    losses = []
    m.train()
    for _ in range(8):
        loss = m.forward_loss(x[:, :-1], x[:, 1:], 2)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss))
    assert losses[-1] < losses[0] - 0.3
    st = opt.steer_state["layers.3.ffn.w1"]
    Q = st["Q_L"][:, :, : st["rank"]]
    eye = torch.eye(st["rank"])
    assert ((Q.transpose(1, 2) @ Q) - eye).abs().max() < 1e-3
    assert st["step"] == 8 and st["subspace_step"] == 8
    tel = opt.get_telemetry()
    assert tel["tiers"]["steer"]["state_bytes"] < tel["adamw_equivalent_bytes"]
    sd = opt.state_dict()
    opt2 = CentroidSteerOptimizer(m, lr=3e-3, rank=8)
    opt2.load_state_dict(sd)
    assert opt2.step_count == 8


def test_subspace_refresh_resets_subspace_step_not_lifetime_step():
    torch.manual_seed(5)
    m = TriuneTransformer.from_config(tiny())
    opt = CentroidSteerOptimizer(m, lr=1e-3, rank=4, update_gap=2)
    x = torch.randint(0, 256, (2, 17))
    seen = []
    for _ in range(3):
        m.forward_loss(x[:, :-1], x[:, 1:], 2).backward()
        opt.step()
        opt.zero_grad()
        st = opt.steer_state["layers.3.ffn.w1"]
        seen.append((st["step"], st["subspace_step"]))
    assert seen == [(1, 1), (2, 2), (3, 1)]


def test_batched_qr_fast_path_and_fallbacks():
    torch.manual_seed(6)
    good = torch.randn(384, 16)
    collinear = good.clone()
    collinear[:, 3] = collinear[:, 2]
    zero_col = good.clone()
    zero_col[:, 5] = 0
    A = torch.stack((good, collinear, zero_col))
    tel = {"total_qr_calls": 0, "cholesky_fast_path_survivals": 0, "householder_fallbacks": 0,
           "primary_fallback_reasons": {k: 0 for k in ("degenerate_columns", "cholesky_non_positive_definite",
                                                        "condition_ratio_exceeded", "orthogonality_tolerance_exceeded")},
           "overlapping_triggers": {k: 0 for k in ("degenerate_columns", "cholesky_non_positive_definite",
                                                    "condition_ratio_exceeded", "orthogonality_tolerance_exceeded")}}
    Q, info = batched_qr(A, telemetry=tel, return_info=True)
    from triune_b200.optim.subspace import flush_qr_telemetry

    flush_qr_telemetry(tel)  # counters accumulate on the device; the report folds them in
    assert info["fallback_mask"].tolist() == [False, True, True]
    assert sum(tel["primary_fallback_reasons"].values()) == 2 == tel["householder_fallbacks"]
    eye = torch.eye(16)
    assert ((Q.transpose(1, 2) @ Q) - eye).flatten(1).norm(dim=-1).max() < 1e-4
    # kappa = 100 needs no fallback and reaches 1e-5
    U, _ = torch.linalg.qr(torch.randn(384, 16))
    V, _ = torch.linalg.qr(torch.randn(16, 16))
    Ak = U @ torch.diag(torch.logspace(0, -2, 16)) @ V.t()
    Qk, infok = batched_qr(Ak.unsqueeze(0), return_info=True)
    assert not bool(infok["fallback_mask"].any()) and float(infok["orth_err"].max()) < 1e-5


def _loss_backward(m, x):
    m.forward_loss(x[:, :-1], x[:, 1:], 2).backward()


def test_step_parameters_layer_by_layer_equals_one_full_step():
    """Several ``step_parameters`` calls over disjoint parameter subsets (the layers, then the root modules) make the
    same global step as ``step()``: same weights, same optimizer state, one step counted."""
    from triune_b200.optim.subspace import set_sketch_seed

    x = torch.randint(0, 256, (2, 25))
    models, opts = [], []
    for _ in range(2):
        torch.manual_seed(9)
        m = TriuneTransformer.from_config(tiny())
        models.append(m)
        opts.append(CentroidSteerOptimizer(m, lr=2e-3, rank=6))
    for step in range(3):
        for m in models:
            _loss_backward(m, x)
        set_sketch_seed(100 + step)  # both optimizers draw the same Gaussian sketches for their subspace refresh
        opts[0].step()
        opts[0].zero_grad()
        set_sketch_seed(100 + step)
        m1, o1 = models[1], opts[1]
        layer_params = [list(l.parameters()) for l in m1.layers]
        in_layers = {id(p) for ps in layer_params for p in ps}
        root = [p for p in m1.parameters() if id(p) not in in_layers]
        for ps in layer_params:
            o1.step_parameters(ps, is_global_step_end=False)
        o1.step_parameters(root, is_global_step_end=True)
        o1.zero_grad()
        assert o1.step_count == opts[0].step_count == step + 1
        for (n, a), (_, b) in zip(models[0].named_parameters(), m1.named_parameters()):
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-6), (step, n)
    s0, s1 = opts[0].steer_state["layers.3.ffn.w1"], opts[1].steer_state["layers.3.ffn.w1"]
    assert torch.allclose(s0["m"], s1["m"], atol=1e-6) and s0["subspace_step"] == s1["subspace_step"] == 3
    assert torch.allclose(opts[0].exp_avg, opts[1].exp_avg, atol=1e-7)
    # a subset leaves everything else untouched
    before = {n: p.detach().clone() for n, p in m1.named_parameters()}
    _loss_backward(m1, x)
    o1.step_parameters(list(m1.layers[0].parameters()), is_global_step_end=True)
    changed = {n for n, p in m1.named_parameters() if not torch.equal(p, before[n])}
    assert changed and all(n.startswith("layers.0.") for n in changed)


def test_single_sided_low_rank_path_with_basis_transport():
    torch.manual_seed(10)
    m = TriuneTransformer.from_config(tiny())
    opt = CentroidSteerOptimizer(m, lr=3e-3, rank=8, update_gap=3, use_triangular_core=False)
    x = torch.randint(0, 256, (4, 33))
    losses = []
    for _ in range(8):
        loss = m.forward_loss(x[:, :-1], x[:, 1:], 2)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss))
    assert losses[-1] < losses[0] - 0.2
    st = opt.steer_state["layers.3.ffn.w1"]
    assert st["mode"] == "galore" and st["step"] == 8 and st["proj_step"] > 1   # refreshed, moments kept (transported)
    P = st["P"][:, :, : st["rank"]]
    assert ((P.transpose(1, 2) @ P) - torch.eye(st["rank"])).abs().max() < 1e-3
    K, m_, n_ = opt.arena.segments[-1].mat_shape
    assert st["m"].numel() < K * m_ * n_ / 3  # the moments live in the projected space


def test_8bit_adam_tier_tracks_the_fp32_tier():
    x = torch.randint(0, 256, (4, 33))
    finals, state_bytes = [], []
    for eight in (False, True):
        torch.manual_seed(11)
        m = TriuneTransformer.from_config(tiny())
        opt = CentroidSteerOptimizer(m, lr=3e-3, rank=8, use_8bit_adam=eight)
        for _ in range(10):
            loss = m.forward_loss(x[:, :-1], x[:, 1:], 2)
            loss.backward()
            opt.step()
            opt.zero_grad()
        finals.append(float(loss))
        state_bytes.append(opt.get_telemetry()["tiers"]["adamw"]["state_bytes"])
        if eight:
            sd = opt.state_dict()
            opt2 = CentroidSteerOptimizer(m, lr=3e-3, rank=8, use_8bit_adam=True)
            opt2.load_state_dict(sd)
            a, b = opt.moments8.load(0, 4096), opt2.moments8.load(0, 4096)
            assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert abs(finals[0] - finals[1]) < 0.15 and state_bytes[1] < 0.3 * state_bytes[0]
    from triune_b200.optim.adam8bit import BlockwiseMoments

    bm = BlockwiseMoments(1000, torch.device("cpu"))
    mm, vv = torch.randn(1000) * 0.01, torch.rand(1000) ** 4 * 1e-3
    bm.store(0, 1000, mm, vv)
    m2, v2 = bm.load(0, 1000)
    assert float((m2 - mm).abs().max()) < 0.02 * float(mm.abs().max())
    assert float(((v2.sqrt() - vv.sqrt()).abs() / vv.sqrt().clamp_min(1e-4)).median()) < 0.02
    bm.store(300, 420, mm[300:420] * 2, vv[300:420])   # a partial update re-encodes only the touched blocks
    m3, _ = bm.load(0, 1000)
    assert torch.allclose(m3[:256], m2[:256]) and float((m3[300:420] - 2 * mm[300:420]).abs().max()) < 0.05 * float(mm.abs().max())


def test_rank_sensitivity_profile_and_reference_state_layout():
    torch.manual_seed(12)
    m = TriuneTransformer.from_config(tiny())
    opt = CentroidSteerOptimizer(m, lr=2e-3, rank=8)
    x = torch.randint(0, 256, (4, 33))
    _loss_backward(m, x)
    rep = opt.profile_rank_sensitivity(ranks=(2, 4, 8, 16))
    e = [rep["ranks"][r]["energy_ratio"] for r in (2, 4, 8, 16)]
    assert all(b >= a - 1e-4 for a, b in zip(e, e[1:])) and 0.0 < e[0] <= e[-1] <= 1.0 + 1e-4
    assert rep["recommended_rank"] in (2, 4, 8, 16) and opt.get_qr_telemetry()["total_qr_calls"] == 0
    for _ in range(3):
        opt.step()
        opt.zero_grad()
        _loss_backward(m, x)
    ref_sd = opt.reference_state_dict()
    n_experts = sum(s.mat_shape[0] for s in opt.arena.segments if s.tier == "steer")
    assert len(ref_sd["layer_groups"]) == n_experts and ref_sd["step_count"] == 3
    g0 = ref_sd["layer_groups"][0]
    assert g0["Q_L"].dim() == 2 and g0["state"]["momentum"].shape == (g0["Q_L"].shape[1],) * 2
    assert set(ref_sd["base_optimizer"]["state"][0]) == {"step", "exp_avg", "exp_avg_sq"}
    opt2 = CentroidSteerOptimizer(m, lr=2e-3, rank=8)
    opt2.load_reference_state_dict(ref_sd)
    assert torch.allclose(opt2.exp_avg, opt.exp_avg) and torch.allclose(opt2.muon_mom, opt.muon_mom)
    a, b = opt.steer_state["layers.3.ffn.w1"], opt2.steer_state["layers.3.ffn.w1"]
    assert torch.allclose(a["Q_L"], b["Q_L"]) and torch.allclose(a["v"], b["v"]) and a["subspace_step"] == b["subspace_step"]


def test_qr_calls_only_on_refresh_steps_and_unrouted_experts_are_skipped():
    """No QR on a step that reuses its bases, and an expert without gradient never reaches the QR (so it cannot
    trigger the degenerate-column fall-back) -- ``tests/test_triangular_core_integrity.py:362-418`` of the reference."""
    torch.manual_seed(13)
    m = TriuneTransformer.from_config(tiny())
    opt = CentroidSteerOptimizer(m, lr=1e-3, rank=4, update_gap=5)
    x = torch.randint(0, 256, (2, 17))
    calls = []
    for _ in range(3):
        _loss_backward(m, x)
        for seg in opt.arena.segments:
            if seg.tier == "steer":
                seg.param.main_grad[0].zero_()   # expert 0 received no tokens
        opt.step()
        opt.zero_grad()
        tel = opt.get_qr_telemetry()
        calls.append(tel["total_qr_calls"])
        assert tel["primary_fallback_reasons"]["degenerate_columns"] == 0
    assert calls[0] > 0 and calls[1] == calls[0] and calls[2] == calls[0]


def test_steered_bases_meet_the_orthogonality_and_subdiagonal_bars():
    """fp32 bars of the reference (``tests/test_triangular_core_integrity.py:169-240``): the steering-augmented bases
    are orthonormal to 5e-5 and the projected core is upper triangular to 1e-7 of ||G|| below the diagonal; rounded to
    bf16 the bars are 5e-3 and 1e-4."""
    from triune_b200.optim.subspace import reorthogonalise, two_sided_bases

    torch.manual_seed(42)
    mm, nn_, r = 384, 1024, 16
    G16 = torch.randn(1, mm, nn_).to(torch.bfloat16)
    G = G16.float()
    QL, QR = two_sided_bases(G, r)
    c = torch.randn(1, nn_)
    v_orth, _ = reorthogonalise(c, QR)
    u = (G @ v_orth.unsqueeze(-1)).squeeze(-1)
    u_orth, _ = reorthogonalise(u, QL)
    QLb, QRb = torch.cat((QL, u_orth.unsqueeze(-1)), -1)[0], torch.cat((QR, v_orth.unsqueeze(-1)), -1)[0]
    eye = torch.eye(r + 1)
    assert float((QLb.t() @ QLb - eye).norm()) < 5e-5 and float((QRb.t() @ QRb - eye).norm()) < 5e-5
    S = QLb.t() @ G[0] @ QRb
    low = torch.tril(torch.ones(r + 1, r + 1, dtype=torch.bool), diagonal=-1)
    # Q_L = qr(G Q_R) makes Q_L^T G Q_R the triangular factor: nothing below the diagonal of the leading r x r block
    assert float(S[:r, :r][low[:r, :r]].abs().max()) / float(G.norm()) < 1e-7
    l16, r16 = QLb.to(torch.bfloat16).float(), QRb.to(torch.bfloat16).float()
    assert float((l16.t() @ l16 - eye).norm()) < 5e-3 and float((r16.t() @ r16 - eye).norm()) < 5e-3
    S16 = l16.t() @ G[0] @ r16
    assert float(S16[:r, :r][low[:r, :r]].abs().max()) / float(G.norm()) < 1e-4


def test_gla_output_scale_option():
    """``gla_scale="fla"`` multiplies every GLA mixer's output by head_dim ** -0.5 (and its gradients accordingly)."""
    from triune_b200.models.attention import VectorisedGLA, set_gla_scale

    torch.manual_seed(0)
    m = VectorisedGLA(32, 2, 16)
    x = torch.randn(2, 24, 32, requires_grad=True)
    y0, _ = m(x)
    g0 = torch.autograd.grad(y0.square().sum(), [x, m.out_proj.weight])
    wrap = torch.nn.ModuleList([m])
    assert set_gla_scale(wrap, "fla") == 1 and abs(m.out_scale - 0.25) < 1e-12
    y1, _ = m(x)
    g1 = torch.autograd.grad(y1.square().sum(), [x, m.out_proj.weight])
    assert torch.allclose(y1, 0.25 * y0, atol=1e-6)
    for a, b in zip(g1, g0):
        assert torch.allclose(a, 0.0625 * b, atol=1e-6)
    set_gla_scale(wrap, "none")
    assert m.out_scale == 1.0
    d = VectorisedGLA(32, 2, 16, use_delta_rule=True)
    assert set_gla_scale(torch.nn.ModuleList([d]), "fla") == 0 and d.out_scale == 1.0  # the delta-rule path is never scaled


def test_quantised_linears_take_gelu_flag_and_dense_ffn_uses_it():
    import torch.nn.functional as F

    from triune_b200.models.block import DenseFFN
    from triune_b200.models.quant_linear import FP8Linear, NVFP4Linear, convert_to_fp8

    torch.manual_seed(0)
    lin = torch.nn.Linear(64, 48)
    x = torch.randn(5, 64)
    for mod in (FP8Linear.from_linear(lin).eval(), NVFP4Linear.from_linear(lin)):
        with torch.no_grad():
            assert torch.allclose(mod(x, gelu=True), F.gelu(mod(x), approximate="tanh"), atol=1e-6)
    ffn = DenseFFN(64, 128).eval()
    with torch.no_grad():
        want = ffn(x)
        assert convert_to_fp8(ffn) == 2 and getattr(ffn[0], "fused_gelu", False)
        got = ffn(x)
    assert F.cosine_similarity(got.flatten(), want.flatten(), dim=0) > 0.99
