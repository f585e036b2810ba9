"""C-ABI engine library: every export is exercised on the CPU (the GPU variants are marked gpu)."""

import pytest
import torch

from triune_b200.ops import _c_bridge as cb
from triune_b200.ops import reference as ref

pytestmark = pytest.mark.skipif(not cb.is_available(), reason="libtriune_core.so not built")


def test_version_and_runtime_probe():
    lib = cb.load_library()
    assert b"triune" in lib.triune_engine_version()
    assert lib.triune_has_cuda_runtime() in (0, 1)


def test_steer_update_matches_reference():
    torch.manual_seed(0)
    P, G = torch.randn(37, 19), torch.randn(37, 19)
    exp = ref.steer_update(P.clone(), G, 0.9, 0.2)
    assert (cb.c_centroid_steer_update(P, G, 0.2, 0.9) - exp).abs().max() < 1e-6


def test_route_tiers_and_heatmap_match_reference():
    torch.manual_seed(1)
    lg = torch.randn(257, 3) * 2
    probs, tiers = cb.c_route_tiers(lg, 0.5)
    assert torch.equal(tiers, ref.route_tiers(lg, 0.5))
    assert (probs - torch.softmax(lg, -1)).abs().max() < 1e-6
    act = torch.randn(5000)
    _, rgba = cb.c_neuron_heatmap(act, 64)
    assert torch.equal(rgba, ref.neuron_heatmap(act, 64))
    a2 = torch.randn(8, 33)
    t = torch.randint(0, 3, (8,))
    assert (cb.c_tier_colour_render(a2, t).int() - ref.tier_colour_render(a2, t).int()).abs().max() <= 1


def test_gla_recurrent_step_matches_reference():
    torch.manual_seed(2)
    BH, d = 6, 64
    q, k, v = torch.randn(BH, d), torch.randn(BH, d), torch.randn(BH, d)
    g = -torch.rand(BH, d)
    state = torch.randn(BH, d, d)
    o_ref, s_ref = ref.gla_decode_step(q[None], k[None], v[None], g[None], state[None].clone())
    s = state.clone()
    o = cb.c_gla_recurrent_step(q, k, v, g, s)
    assert (o - o_ref[0]).abs().max() < 1e-4 and (s - s_ref[0]).abs().max() < 1e-5


def test_engine_lifecycle_on_host():
    eng = cb.NativeTriuneEngine(max_seq_len=128, hidden_dim=64, device_id=-1)
    eng.set_losses(3.0, 2.5, 0.5, 1)
    st = eng.step(torch.randint(0, 1000, (2, 64)), torch.randint(0, 1000, (2, 64)))
    assert st["tokens_processed"] == 128 and st["loss"] == 3.0 and st["active_tier"] == 1 and st["step_time_ms"] >= 0
    assert eng.capture_graph(2, 64) != 0  # no device: capture is refused, not faked
    eng.close()


def test_stage_ring_host_fallback_copies_bytes():
    ring = cb.PinnedStageRing(-1, 2, 1 << 16)
    src = torch.arange(1000, dtype=torch.float32)
    dst = torch.zeros(1000)
    for _ in range(3):
        ring.wait(ring.submit(src, dst))
    assert torch.equal(src, dst) and ring.bytes_moved == 3 * 4000
    ring.close()


@pytest.mark.gpu
def test_engine_and_ring_on_device():
    eng = cb.NativeTriuneEngine(max_seq_len=256, hidden_dim=128, device_id=0)
    st = eng.step(torch.randint(0, 1000, (4, 128)))
    assert st["cuda_runtime_bound"] == 1 and st["vram_used_mb"] > 0
    assert eng.capture_graph(4, 128) == 0 and eng.replay_graph() == 0
    st = eng.step(torch.randint(0, 1000, (4, 128)))
    assert st["tokens_processed"] == 512
    eng.close()
    ring = cb.PinnedStageRing(0, 3, 1 << 20)
    src = torch.randn(1 << 18)
    dst = torch.zeros(1 << 18, device="cuda")
    for _ in range(5):
        ring.wait(ring.submit(src, dst))
    torch.cuda.synchronize()
    assert torch.equal(dst.cpu(), src)
    ring.close()
