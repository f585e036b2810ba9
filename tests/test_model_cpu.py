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
