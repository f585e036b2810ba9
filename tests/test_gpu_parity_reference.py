"""Loss-curve parity with the reference implementation on a GPU: one initialisation loaded into both models, the same ten
batches, plain AdamW at one learning rate; the bf16 training losses must track each other step by step."""

import os
import sys

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_model_class():
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "triune")):
        pytest.skip("reference not installed")
    sys.path.insert(0, ref_dir)
    try:
        from triune.model.transformer import TriuneTransformer as RefModel
    except Exception as e:  # pragma: no cover
        pytest.skip(f"reference import failed: {e}")
    finally:
        sys.path.remove(ref_dir)
    return RefModel


def test_ten_training_steps_track_the_reference_loss_curve():
    from triune_b200.models import TriuneTransformer

    RefModel = _reference_model_class()
    dev = torch.device("cuda", 0)
    arch = dict(vocab_size=2048, hidden_dim=128, num_layers=5, num_heads=2, head_dim=64, num_experts=4,
                router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3)
    torch.manual_seed(0)
    ref = RefModel(**arch).to(device=dev, dtype=torch.bfloat16)
    ours = TriuneTransformer(**arch)
    ours.load_state_dict(ref.state_dict())
    ours = ours.to(device=dev, dtype=torch.bfloat16)
    import triune.model.attention as ref_attention  # already imported through the model; still in sys.modules
    from triune_b200.models.attention import set_gla_scale

    # with flash-linear-attention installed the reference's CUDA path scales the queries by head_dim ** -0.5
    set_gla_scale(ours, "fla" if getattr(ref_attention, "HAS_FLA", False) else "none")
    g = torch.Generator().manual_seed(5)
    batches = [torch.randint(0, 2048, (4, 257), generator=g).to(dev) for _ in range(3)]  # a small pool: the loss must fall
    opt_ref = torch.optim.AdamW(ref.parameters(), lr=2e-3, betas=(0.9, 0.95), weight_decay=0.0)
    opt_ours = torch.optim.AdamW(ours.parameters(), lr=2e-3, betas=(0.9, 0.95), weight_decay=0.0)
    ref.train(), ours.train()
    curve_ref, curve_ours = [], []
    for step in range(10):
        ids = batches[step % len(batches)]
        x, y = ids[:, :-1], ids[:, 1:]
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = ref(x, force_depth=2)[0]
        l_ref = F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), y.reshape(-1))
        opt_ref.zero_grad(set_to_none=True)
        l_ref.backward()
        opt_ref.step()
        l_ours = ours.forward_loss(x, y, force_depth=2)
        opt_ours.zero_grad(set_to_none=True)
        l_ours.backward()
        opt_ours.step()
        curve_ref.append(float(l_ref))
        curve_ours.append(float(l_ours))
    assert curve_ref[-1] < curve_ref[0] - 0.05 and curve_ours[-1] < curve_ours[0] - 0.05, (curve_ref, curve_ours)
    for a, b in zip(curve_ref, curve_ours):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (curve_ref, curve_ours)
