"""CPU tests of the training loop, checkpoints, schedule, generation, speculative decoding, dense models, layer
streaming, and data parallelism over gloo (world size 2)."""

import math
import os
import subprocess
import sys

import pytest
import torch
import torch.nn.functional as F

from triune_b200.config import ModelConfig
from triune_b200.models import TriuneTransformer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = dict(vocab_size=256, hidden_dim=64, num_layers=5, num_heads=2, head_dim=32, num_experts=4, top_k=2, router_prefix_layers=1,
           reflex_exit_layer=2, limbic_exit_layer=3, expert_hidden=96, dense_hidden=80)


def tiny(seed=0):
    torch.manual_seed(seed)
    return TriuneTransformer.from_config(ModelConfig(**CFG))


class Tok:
    pad_token_id, sep_token_id, eos_token_id = None, None, None

    def encode(self, s):
        return [ord(c) % 256 for c in s]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(int(i) % 128 or 32) for i in ids)


def _trainer(model, **cfg):
    from triune_b200.data import SyntheticTokenSource
    from triune_b200.optim import CentroidSteerOptimizer
    from triune_b200.trainer import Trainer

    run = {"lr": 3e-3, "min_lr": 3e-4, "warmup_steps": 2, "total_steps": 50, "depth_mode": "cortex", "grad_accum_steps": 1,
           "grad_clip": 1.0, "vocab_size": 256, "batch_size": 4, "seq_len": 32}
    run.update(cfg)
    opt = CentroidSteerOptimizer(model, lr=run["lr"], grad_clip=1.0)
    src = SyntheticTokenSource(256, run["batch_size"], run["seq_len"], seed=3, pool=1)  # one repeating batch: loss must fall
    return Trainer(model, run, optimizer=opt, train_loader=src, device=torch.device("cpu"))


@pytest.mark.parametrize("mode", ["cortex", "joint", "dynamic"])
def test_training_modes_reduce_loss(mode):
    tr = _trainer(tiny(), depth_mode=mode)
    losses = [float(tr.engine.step_once()["loss"]) for _ in range(12)]
    assert all(math.isfinite(l) for l in losses) and min(losses[-3:]) < losses[0]
    assert tr.engine.step == 12


def test_dynamic_mode_trains_the_depth_router():
    """The router that picks the exit at inference must receive a gradient in the default depth mode."""
    tr = _trainer(tiny(), depth_mode="dynamic")
    batch = tr.next_batch()
    loss, stats = tr.engine._micro_loss(batch[0], batch[1], None)
    loss.backward()
    router = tr.model.router.router_mlp
    grads = [p.grad if p.grad is not None else getattr(p, "main_grad", None) for p in router.parameters()]
    assert all(g is not None for g in grads)
    assert sum(float(g.float().abs().sum()) for g in grads) > 0.0
    assert "router_loss" in stats and math.isfinite(float(stats["router_loss"]))


def test_lr_schedule_warmup_cosine_and_cycles():
    from triune_b200.trainer.scheduler import lr_schedule

    cfg = {"lr": 1.0, "min_lr": 0.1, "warmup_steps": 10, "total_steps": 110}
    assert lr_schedule(cfg, 0) < lr_schedule(cfg, 5) < lr_schedule(cfg, 10) <= 1.0
    assert abs(lr_schedule(cfg, 10) - 1.0) < 0.11 and abs(lr_schedule(cfg, 109) - 0.1) < 0.02
    mid = lr_schedule(cfg, 60)
    assert 0.1 < mid < 1.0
    assert all(0.1 - 1e-9 <= lr_schedule(cfg, s) <= 1.0 + 1e-9 for s in range(0, 400, 7))  # wraps into new cycles


def test_checkpoint_roundtrip_resume_and_fingerprint(tmp_path):
    from triune_b200.trainer import checkpoint as ckpt

    tr = _trainer(tiny())
    for _ in range(3):
        tr.engine.step_once()
    tr.config["checkpoint_dir"] = str(tmp_path)
    path = tr.save_latest()
    assert os.path.exists(path) and not [p for p in os.listdir(tmp_path) if p.endswith(".tmp")]  # atomic rename
    ref_next = float(tr.engine.step_once()["loss"])
    tr2 = _trainer(tiny(seed=1))
    ck = tr2.resume(path)
    assert tr2.engine.step == 3 and ck["step"] == 3
    for a, b in zip(tr.model.state_dict().values(), tr2.model.state_dict().values()):
        pass  # tr advanced one more step; compare the resumed run's next loss instead
    assert abs(float(tr2.engine.step_once()["loss"]) - ref_next) < 5e-3  # same weights, optimizer state and batch
    fp = ckpt.fingerprint({"hidden_dim": 64, "num_layers": 5, "lr": 1.0})
    assert fp == ckpt.fingerprint({"hidden_dim": 64, "num_layers": 5, "lr": 2.0})  # optimisation settings are not semantics
    assert fp != ckpt.fingerprint({"hidden_dim": 128, "num_layers": 5})
    with pytest.raises(Exception):
        ckpt.load_checkpoint(path, model=TriuneTransformer.from_config(ModelConfig(**{**CFG, "hidden_dim": 32, "num_heads": 1})),
                             config={"hidden_dim": 32, "num_layers": 5})


def test_generation_cache_penalties_and_stop():
    from triune_b200.inference import _apply_penalties, generate_response, generate_tokens, infer_config_from_state_dict

    m = tiny().eval()
    ids = torch.randint(0, 256, (1, 11))
    out, cache, tele = generate_tokens(m, ids, max_new_tokens=6, temperature=0.0, repetition_penalty=1.0, count_penalty=0.0,
                                       prefill_chunk=4)
    # greedy decoding with the recurrent cache equals re-running the whole prefix every step
    seq = ids.clone()
    for _ in range(6):
        nxt = m(seq, force_depth=2)[0][0, -1].argmax().view(1, 1)
        seq = torch.cat((seq, nxt), 1)
    assert out == seq[0, 11:].tolist() and tele["new_tokens"] == 6 and cache is not None
    lg = torch.tensor([2.0, -2.0, 1.0, 0.5])
    pen = _apply_penalties(lg.clone(), torch.tensor([0, 0, 1]), 2.0, 0.5)
    assert pen[0] == 2.0 / 2.0 - 0.5 and pen[1] == -4.0 and pen[2] == 1.0
    seen = []
    r = generate_response(m, Tok(), "hello", max_new_tokens=8, temperature=0.0, stream_callback=seen.append, stop=("zzzz",))
    assert isinstance(r["text"], str) and len(r["tokens"]) <= 8 and "".join(seen).strip().startswith(r["text"][:3])
    cfg = infer_config_from_state_dict(m.state_dict())
    assert (cfg.hidden_dim, cfg.num_layers, cfg.num_experts, cfg.expert_hidden, cfg.dense_hidden) == (64, 5, 4, 96, 80)
    assert (cfg.reflex_exit_layer, cfg.limbic_exit_layer) == (2, 3)


def test_self_speculative_sampling_follows_the_verifier_distribution():
    """Leviathan rejection sampling is exact: the first emitted token of many sampled runs is distributed as the
    verifier's softmax(logits / temperature) (Pearson chi-square with small bins pooled; the reference's bar,
    ``tests/test_self_speculative_decoding.py:126-214``: p > 0.005)."""
    from triune_b200.models.speculative import SelfSpeculativeGenerator

    torch.manual_seed(77)
    vocab, temperature, n_draws = 12, 0.7, 2000
    model = TriuneTransformer(vocab_size=vocab, hidden_dim=32, num_layers=6, num_heads=2, head_dim=16, num_experts=2,
                              router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=4).eval()
    with torch.no_grad():  # make the exits disagree visibly, so that rejections actually occur
        model.final_head.weight.mul_(4.0)
        model.layers[2].exit_head.weight.mul_(4.0)
    prompt = torch.tensor([[1, 3, 7, 2]])
    with torch.no_grad():
        logits = model(prompt, force_depth=2, last_token_only=True)[0]
        p_exact = F.softmax(logits[0, -1].float() / temperature, dim=-1).double()
        q_draft = F.softmax(model(prompt, force_depth=0, last_token_only=True)[0][0, -1].float() / temperature, dim=-1).double()
    assert float((p_exact - q_draft).abs().sum()) > 0.05  # the two exits really differ
    gen = SelfSpeculativeGenerator(model, k_draft=2)
    rng = torch.Generator().manual_seed(2026)
    counts = torch.zeros(vocab, dtype=torch.float64)
    for _ in range(n_draws):
        out = gen.generate(prompt, max_new_tokens=1, temperature=temperature, generator=rng)
        counts[int(out[0, -1])] += 1.0
    assert gen.telemetry["proposed"] > 0 and gen.telemetry["accepted"] < gen.telemetry["proposed"]  # some rejections
    obs, exp = [], []
    tail_o = tail_e = 0.0
    for o_i, e_i in zip(counts.tolist(), (p_exact * n_draws).tolist()):
        if e_i >= 5.0:
            obs.append(o_i)
            exp.append(e_i)
        else:
            tail_o, tail_e = tail_o + o_i, tail_e + e_i
    if tail_e >= 5.0:
        obs.append(tail_o)
        exp.append(tail_e)
    elif tail_e > 0.0 and obs:
        obs[-1] += tail_o
        exp[-1] += tail_e
    df = len(obs) - 1
    assert df >= 3
    chi2 = sum((o - e) ** 2 / e for o, e in zip(obs, exp))
    z = ((chi2 / df) ** (1.0 / 3.0) - (1.0 - 2.0 / (9.0 * df))) / math.sqrt(2.0 / (9.0 * df))  # Wilson-Hilferty
    p_val = 0.5 * math.erfc(z / math.sqrt(2.0))
    assert p_val > 0.005, f"sampled tokens diverge from the verifier distribution (chi2={chi2:.2f}, df={df}, p={p_val:.4g})"


def test_self_speculative_greedy_equals_autoregressive():
    from triune_b200.models.speculative import SelfSpeculativeGenerator

    m = tiny().eval()
    gen = SelfSpeculativeGenerator(m, k_draft=3)
    ids = torch.randint(0, 256, (1, 9))
    a = gen.generate(ids, max_new_tokens=10, temperature=0.0)
    b = gen.generate_autoregressive(ids, max_new_tokens=10)
    assert torch.equal(a[:, : b.shape[1]], b[:, : a.shape[1]])
    assert 0.0 <= gen.acceptance_rate <= 1.0 and gen.telemetry["proposed"] > 0


@pytest.mark.parametrize("mixer,ffn", [("gla", "swiglu"), ("gated_deltanet", "swiglu"), ("sdpa", "gelu")])
def test_universal_dense_models_train_and_cache(mixer, ffn):
    from triune_b200.models.universal import TriuneUniversalEngine, UniversalDenseTransformer

    torch.manual_seed(0)
    cfg = ModelConfig(family="universal", vocab_size=128, hidden_dim=64, num_layers=2, num_heads=2, head_dim=32, mixer=mixer,
                      ffn=ffn, dense_hidden=96, num_experts=1, top_k=1)
    m = UniversalDenseTransformer.from_config(cfg)
    eng = TriuneUniversalEngine(m, lr=5e-3)
    x = torch.randint(0, 128, (2, 17))
    losses = [eng.train_step(x) for _ in range(8)]
    assert losses[-1] < losses[0]
    m.eval()
    full = m(x[:, :12])[0] if isinstance(m(x[:, :12]), tuple) else m(x[:, :12])
    cache = m.init_cache(2)
    lg1, cache = m(x[:, :7], cache=cache)
    lg2, cache = m(x[:, 7:12], cache=cache)
    assert torch.allclose(torch.cat((lg1, lg2), 1), full, atol=2e-4, rtol=1e-3)
    out = eng.generate(x[:1, :5], max_new_tokens=4)
    assert out.shape == (1, 9)


def test_layer_streaming_matches_resident_training():
    from triune_b200.runtime.streaming import StreamingConfig, enable_layer_streaming

    a, b = tiny(), tiny()
    x = torch.randint(0, 256, (2, 16))
    y = torch.randint(0, 256, (2, 16))
    eng = enable_layer_streaming(b, "cpu", config=StreamingConfig(resident_gpu_layers=1, pin_memory=False))
    la = a.forward_loss(x, y, force_depth=2)
    lb = b.forward_loss(x, y, force_depth=2)
    la, lb = (la[0] if isinstance(la, tuple) else la), (lb[0] if isinstance(lb, tuple) else lb)
    assert torch.allclose(la, lb, atol=1e-5)
    la.backward()
    lb.backward()
    # streamed layers hand their gradients to the host store; resident ones keep .grad
    tel = eng.get_telemetry()
    assert tel["d2h_copies"] >= 1 and tel["d2h_bytes"] > 0
    eng.step_streaming_optimizer(None, lr=1e-2)
    lb2 = b.forward_loss(x, y, force_depth=2)
    lb2 = lb2[0] if isinstance(lb2, tuple) else lb2
    assert torch.isfinite(lb2) and float(lb2) != float(lb)  # streamed layers were updated
    eng.detach()
    out = b(x, force_depth=2)[0]
    assert out.shape == (2, 16, 256)


def test_streamed_layers_get_the_tiered_optimizer_with_resident_parity():
    """Streamed layers stepped one at a time through ``step_parameters`` (state sets in host memory, one device arena
    per layer signature) follow the same trajectory as the resident model under one CentroidSteerOptimizer
    (tests/test_streaming_training_parity.py:75-472 of the reference)."""
    from triune_b200.optim import CentroidSteerOptimizer
    from triune_b200.optim.subspace import set_sketch_seed
    from triune_b200.runtime.streaming import StreamingConfig, enable_layer_streaming

    a, b = tiny(), tiny()
    # enough tokens per expert that every expert gradient has full rank: a rank-deficient gradient leaves the trailing
    # basis vectors to rounding noise, and the two sides would then carry their moments in different bases
    kw = dict(lr=3e-3, muon_ns_steps=3, update_gap=2, steer_update_gap=2, rank=16)
    opt_a = CentroidSteerOptimizer(a, grad_clip=0.5, **kw)
    eng = enable_layer_streaming(b, "cpu", config=StreamingConfig(resident_gpu_layers=0, pin_memory=False, grad_clip=0.5))
    streamed = {id(p) for st in eng.stores.values() for p in st.params}
    opt_root = CentroidSteerOptimizer(b, grad_clip=None, only=lambda n, p: id(p) not in streamed, **kw)
    pool = eng.enable_tiered_optimizer(**kw)
    assert len(pool.groups) >= 1 and sum(len(g.layers) for g in pool.groups.values()) == len(eng.stores)
    tiers = {s.tier for g in pool.groups.values() for s in g.opt.arena.segments}
    assert "muon" in tiers and "adamw" in tiers
    for step in range(3):
        x = torch.randint(0, 256, (8, 64), generator=torch.Generator().manual_seed(step))
        y = torch.randint(0, 256, (8, 64), generator=torch.Generator().manual_seed(100 + step))
        la = a.forward_loss(x, y, force_depth=2)
        lb = b.forward_loss(x, y, force_depth=2)
        la, lb = (la[0] if isinstance(la, tuple) else la), (lb[0] if isinstance(lb, tuple) else lb)
        assert torch.allclose(la, lb, atol=2e-4), (step, float(la), float(lb))
        la.backward()
        lb.backward()
        # the resident model takes the same step in the same order (root, then layer by layer), so that the
        # randomised range finder of the CentroidSteer tier draws the same sketches on both sides
        set_sketch_seed(500 + step)
        opt_a.arena.fold_autograd_grads()
        opt_a.compute_clip()
        layer_ids = [{id(p) for p in l.parameters()} for l in a.layers]
        in_layers = set().union(*layer_ids)
        opt_a.step_parameters([p for p in a.parameters() if id(p) not in in_layers])
        for k, l in enumerate(a.layers):
            opt_a.step_parameters(list(l.parameters()), is_global_step_end=(k == len(a.layers) - 1))
        opt_a.zero_grad()
        # root parameters: autograd grads folded into the root arena, clipped by the engine's global coefficient
        set_sketch_seed(500 + step)
        norm = eng.step_streaming_optimizer(_RootStep(opt_root, eng))
        assert abs(norm - float(opt_a.last_grad_norm)) < 1e-3 * max(1.0, norm)
    for (n, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.allclose(pa, pb, atol=5e-4, rtol=1e-3), n
    assert pool.state_bytes() > 0
    sd = pool.state_dict()
    pool.load_state_dict(sd)


class _RootStep:
    """Adapter: the engine scales ``p.grad`` of the root parameters by the global clip coefficient and then calls
    ``step()`` / ``zero_grad()``; the arena optimizer folds those gradients and steps its subset."""

    def __init__(self, opt, eng):
        self.opt, self.eng = opt, eng

    def step(self):
        self.opt.set_clip_coefficient(1.0)
        self.opt.step_parameters([s.param for s in self.opt.arena.segments], is_global_step_end=True)

    def zero_grad(self, set_to_none=True):
        self.opt.zero_grad()


def test_streaming_engine_cleans_up_after_an_exception():
    """A layer that raises on the host in forward or backward, and an optimizer that raises, leave no layer staged or
    bound to a device buffer, and the next step works (tests/test_streaming_exception_cleanup.py:13-116)."""
    from triune_b200.runtime.streaming import StreamingConfig, enable_layer_streaming

    b = tiny()
    eng = enable_layer_streaming(b, "cpu", config=StreamingConfig(resident_gpu_layers=0, pin_memory=False))
    x = torch.randint(0, 256, (2, 16))
    y = torch.randint(0, 256, (2, 16))
    victim = b.layers[1]
    armed = {"fwd": True}
    orig_ffn = victim.ffn.forward

    def raising(*a_, **k_):
        if armed["fwd"]:
            raise RuntimeError("injected forward failure")
        return orig_ffn(*a_, **k_)

    victim.ffn.forward = raising
    try:
        b.forward_loss(x, y, force_depth=2)
        assert False, "the injected failure did not surface"
    except RuntimeError as e:
        assert "injected forward failure" in str(e)
    assert all(v == 0 for v in eng._staged.values())
    assert all(st.device_buf is None for st in eng.stores.values())
    assert all(p.data_ptr() == st.host[off : off + 1].data_ptr() for st in eng.stores.values()
               for p, (off, n, _) in zip(st.params, st.slices))
    # the same layer fails during the recomputation of the backward pass
    armed["fwd"] = False
    loss = b.forward_loss(x, y, force_depth=2)
    loss = loss[0] if isinstance(loss, tuple) else loss
    armed["fwd"] = True
    try:
        loss.backward()
        assert False
    except RuntimeError as e:
        assert "injected forward failure" in str(e)
    assert all(v == 0 for v in eng._staged.values()) and all(st.device_buf is None for st in eng.stores.values())
    armed["fwd"] = False
    eng.cleanup()

    class FaultyOptimizer:
        def step(self):
            raise RuntimeError("injected optimizer failure")

        def zero_grad(self, set_to_none=True):
            pass

    loss = b.forward_loss(x, y, force_depth=2)
    (loss[0] if isinstance(loss, tuple) else loss).backward()
    try:
        eng.step_streaming_optimizer(FaultyOptimizer())
        assert False
    except RuntimeError as e:
        assert "injected optimizer failure" in str(e)
    assert all(st.device_buf is None for st in eng.stores.values())
    assert all(p.grad is None for st in eng.stores.values() for p in st.params)
    # the engine is reusable
    loss = b.forward_loss(x, y, force_depth=2)
    (loss[0] if isinstance(loss, tuple) else loss).backward()
    assert eng.step_streaming_optimizer(None, lr=1e-2) > 0


GLOO_WORKER = r'''
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from triune_b200.config import ModelConfig
from triune_b200.models import TriuneTransformer
from triune_b200.optim import CentroidSteerOptimizer
from triune_b200.parallel import setup_distributed, all_reduce_dict
from triune_b200.parallel.data_parallel import ShardedDataParallel
from triune_b200.trainer import Trainer
ctx = setup_distributed(backend="gloo")
cfg = dict(vocab_size=256, hidden_dim=64, num_layers=5, num_heads=2, head_dim=32, num_experts=4, top_k=2, router_prefix_layers=1,
           reflex_exit_layer=2, limbic_exit_layer=3, expert_hidden=96, dense_hidden=80)
torch.manual_seed(100 + ctx.rank)           # different initial weights per rank: attach() must broadcast rank 0's
model = TriuneTransformer.from_config(ModelConfig(**cfg))
dp = ShardedDataParallel(ctx, mode="nccl")   # collective all-reduce path (gloo here)
opt = CentroidSteerOptimizer(model, lr=3e-3, grad_clip=1.0)
run = {"lr": 3e-3, "min_lr": 3e-4, "warmup_steps": 2, "total_steps": 50, "depth_mode": "cortex", "grad_accum_steps": 1,
       "grad_clip": 1.0, "vocab_size": 256}
tr = Trainer(model, run, optimizer=opt, device=torch.device("cpu"), dp=dp)
g = torch.Generator().manual_seed(7)
data = torch.randint(0, 256, (4, 33), generator=g)        # global batch of 4, two rows per rank
mine = data[ctx.rank * 2:(ctx.rank + 1) * 2]
losses = []
for _ in range(6):
    losses.append(tr.train_step(mine[:, :-1].contiguous(), mine[:, 1:].contiguous()))
avg = all_reduce_dict({"loss": losses[-1]}, ctx)
chk = float(sum(p.double().sum() for p in model.parameters()))
print("RESULT " + json.dumps({"rank": ctx.rank, "losses": losses, "avg": avg["loss"], "checksum": chk}), flush=True)
dist.barrier(); dist.destroy_process_group()
'''


def test_gloo_data_parallel_matches_single_process_large_batch(tmp_path):
    """Two gloo ranks with half the batch each follow the same loss curve as one process with the whole batch."""
    import json

    worker = tmp_path / "w.py"
    worker.write_text(GLOO_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29731", str(worker), ROOT]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    import re

    dec = json.JSONDecoder()  # two ranks share the pipe: records can land on one line
    res = sorted((dec.raw_decode(p.stdout, m.end())[0] for m in re.finditer(r"RESULT (?=\{)", p.stdout)), key=lambda r: r["rank"])
    assert p.returncode == 0 and len(res) == 2, p.stdout[-2000:] + p.stderr[-2000:]
    assert abs(res[0]["checksum"] - res[1]["checksum"]) < 1e-6 * max(1.0, abs(res[0]["checksum"]))  # replicas stay identical
    # single process, same initial weights as rank 0, whole batch
    torch.manual_seed(100)
    model = TriuneTransformer.from_config(ModelConfig(**CFG))
    tr = _trainer(model)
    g = torch.Generator().manual_seed(7)
    data = torch.randint(0, 256, (4, 33), generator=g)
    single = [tr.train_step(data[:, :-1].contiguous(), data[:, 1:].contiguous()) for _ in range(6)]
    dp_mean = [(a + b) / 2 for a, b in zip(res[0]["losses"], res[1]["losses"])]
    assert abs(dp_mean[0] - single[0]) < 2e-3                      # same weights, same data: same first loss
    assert dp_mean[-1] < dp_mean[0] and abs(dp_mean[-1] - single[-1]) < 0.15  # same trajectory up to routing / capacity effects
    assert abs(res[0]["avg"] - dp_mean[-1]) < 1e-5


def test_layer_store_keeps_every_tensor_on_a_vector_boundary():
    """The flat per-layer buffers pad every tensor to 64 elements, so a tensor packed behind an odd-sized one (a
    3-element bias) still starts on a 16-byte boundary; the kernels read parameters in 16-byte vectors."""
    import torch.nn as nn

    from triune_b200.runtime.streaming import LayerStore

    layer = nn.Sequential(nn.Linear(16, 3), nn.Linear(3, 24), nn.LayerNorm(24)).to(torch.bfloat16)
    before = [p.detach().clone() for p in layer.parameters()]
    st = LayerStore(layer, pin=False)
    assert [off % 64 for off, _, _ in st.slices] == [0] * len(st.slices)
    assert st.numel % 64 == 0 and st.host.numel() == st.numel and st.host_grad.numel() == st.numel
    for p, q in zip(layer.parameters(), before):
        assert torch.equal(p.detach(), q)
        assert (p.data_ptr() - st.host.data_ptr()) % 16 == 0
    dev = torch.zeros(st.numel, dtype=torch.bfloat16)
    dev.copy_(st.host)
    st.bind(dev)
    for p, q in zip(layer.parameters(), before):
        assert torch.equal(p.detach(), q) and (p.data_ptr() - dev.data_ptr()) % 16 == 0
    st.bind_host()


def test_tensor_parallel_dense_model_matches_unsharded_on_gloo():
    """Two gloo ranks: the tensor-parallel dense model (sequence-parallel rows, column / row parallel projections) gives
    the loss and every gradient of the unsharded model, for GLA + SwiGLU and Gated DeltaNet + GELU blocks."""
    import json
    import re

    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2", TRIUNE_TP_DEVICE="cpu")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29733", os.path.join(ROOT, "tests", "mp_tp_model_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    dec = json.JSONDecoder()
    res = [dec.raw_decode(p.stdout, m.end())[0] for m in re.finditer(r"RESULT (?=\{)", p.stdout)]
    assert p.returncode == 0 and len(res) == 2, p.stdout[-2000:] + p.stderr[-2000:]
    for r in res:
        for k, v in r.items():
            if k == "rank" or k.endswith("_status"):
                continue
            assert v < 1e-4, (k, v)


def test_sharded_checkpoints_merge_to_the_canonical_single_file_on_gloo(tmp_path):
    """Two gloo ranks save rank-local shards of a tensor-parallel dense model and of an expert-parallel MoE model;
    ``python -m triune_b200 checkpoint merge`` assembles the canonical file (reference key layout), which loads
    strictly into the unsharded model and reproduces its logits; each rank resumes from its own shard."""
    import json
    import re

    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29751", os.path.join(ROOT, "tests", "mp_shard_ckpt_worker.py"), str(tmp_path)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    dec = json.JSONDecoder()
    res = [dec.raw_decode(p.stdout, m.end())[0] for m in re.finditer(r"RESULT (?=\{)", p.stdout)]
    assert p.returncode == 0 and len(res) == 2, p.stdout[-2000:] + p.stderr[-3000:]
    r0 = [r for r in res if r["rank"] == 0][0]
    for key in ("tp_gla_swiglu", "tp_gated_deltanet_gelu"):
        assert r0[key + "_merged_logits"] < 1e-5 and r0[key + "_step"] == 7, r0
        for r in res:
            assert r[key + "_resume"] == 0.0 and r[key + "_resume_step"] == 7, r
    assert r0["ep_merged_logits"] < 1e-5 and r0["ep_keys_equal"] == 1 and r0["ep_has_per_expert_keys"] == 1, r0
    assert sorted(f for f in os.listdir(tmp_path / "ep") if f.startswith("shard-")) == [
        "shard-00000-of-00002.pt", "shard-00001-of-00002.pt"]


@pytest.mark.parametrize("kernel_like", [False, True])
def test_context_parallel_gla_matches_whole_sequence_on_gloo(kernel_like):
    """Three gloo ranks, one sequence segment each: the state hand-off reproduces outputs, final state and all input
    gradients of the whole-sequence recurrence (fp64), with and without an autograd graph. ``kernel_like`` makes the
    local pass return its state without a gradient, as the CUDA kernels do, so the analytic state gradient carries the
    dependence of later segments on earlier keys, values and decays."""
    import json
    import re

    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2", CP_EMULATE_KERNEL_STATE="1" if kernel_like else "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29735", os.path.join(ROOT, "tests", "mp_cp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    dec = json.JSONDecoder()
    res = [dec.raw_decode(p.stdout, m.end())[0] for m in re.finditer(r"RESULT (?=\{)", p.stdout)]
    assert p.returncode == 0 and len(res) == 3, p.stdout[-2000:] + p.stderr[-2000:]
    assert any("state" in r for r in res)
    for r in res:
        for k, v in r.items():
            if k != "rank":
                assert v < 1e-9, (k, v)


def test_tensor_parallel_times_data_parallel_on_gloo():
    """Four gloo ranks as tensor parallel 2 x data parallel 2: after the tensor-parallel sum of the replicated
    gradients and the average over replicas, every gradient equals that of the unsharded model on the whole batch."""
    import json
    import re

    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", "29737", os.path.join(ROOT, "tests", "mp_tp_dp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    dec = json.JSONDecoder()
    res = [dec.raw_decode(p.stdout, m.end())[0] for m in re.finditer(r"RESULT (?=\{)", p.stdout)]
    assert p.returncode == 0 and len(res) == 4, p.stdout[-2000:] + p.stderr[-2000:]
    for r in res:
        for k, v in r.items():
            if k != "rank":
                assert v < 1e-4, (k, v)


def test_pipeline_schedule_properties():
    """1F1B as data: every stage runs each micro-batch forward once and backward once, backward after forward and in
    order; a stage never holds more than (stages - stage) micro-batches; the layer split covers every layer once."""
    from triune_b200.parallel.pipeline import one_f_one_b, peak_live_micro_batches, split_layers

    for stages in (1, 2, 3, 4, 8):
        for micro in (1, 2, 4, 8, 16):
            for s in range(stages):
                steps = one_f_one_b(s, stages, micro)
                assert [i for k, i in steps if k == "F"] == list(range(micro))
                assert [i for k, i in steps if k == "B"] == list(range(micro))
                for i in range(micro):
                    assert steps.index(("F", i)) < steps.index(("B", i))
                assert peak_live_micro_batches(s, stages, micro) == min(stages - s, micro)
    assert split_layers(24, 4) == [(0, 6), (6, 12), (12, 18), (18, 24)]
    assert split_layers(5, 3) == [(0, 2), (2, 4), (4, 5)]
    b = split_layers(24, 4, weights=[1, 1, 1, 1.5])
    assert b[0][0] == 0 and b[-1][1] == 24 and all(b[i][1] == b[i + 1][0] for i in range(3))
    assert b[-1][1] - b[-1][0] < b[0][1] - b[0][0]
    with pytest.raises(ValueError):
        split_layers(2, 3)


@pytest.mark.parametrize("family", ["dense", "triune"])
def test_pipeline_parallel_on_gloo(family):
    """Three gloo ranks, four micro-batches: loss and every gradient of every stage equal those of the whole model on
    the whole batch, two steps in a row, and the number of live micro-batches follows the schedule. ``triune`` is the
    multi-exit MoE family, whose tied embedding / head weight lives on the first and the last stage and has its two
    gradients summed after every step."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1", PP_MICRO="4", PP_FAMILY=family)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29741", os.path.join(ROOT, "tests", "mp_pp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0 and "PP_OK 3 4" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]


def test_rescue_checkpoint_stages():
    """Continuation rescue: on learnable synthetic data the three stages lower the loss of every exit, the report
    carries before / per-stage / after metrics, block packing keeps separators and drops the ragged tail."""
    from triune_b200.config import ModelConfig
    from triune_b200.models import TriuneTransformer
    from triune_b200.trainer.rescue import cosine_lr, evaluate_all_depths, pack_blocks, rescue_checkpoint

    blocks = pack_blocks([[1, 2, 3], [4, 5, 6, 7], [8]], seq_len=3, sep_id=0)
    assert blocks.shape == (2, 4) and blocks[0].tolist() == [1, 2, 3, 0]
    assert cosine_lr(0, 100, 10, 1.0, 0.1) == pytest.approx(0.1) and cosine_lr(99, 100, 10, 1.0, 0.1) < 0.11
    assert cosine_lr(10, 100, 10, 1.0, 0.1) == pytest.approx(1.0)

    torch.manual_seed(0)
    V, T = 32, 24
    cfg = ModelConfig(vocab_size=V, hidden_dim=32, num_layers=5, num_heads=2, head_dim=16, num_experts=2, reflex_exit_layer=2,
                      limbic_exit_layer=3, router_prefix_layers=1)
    model = TriuneTransformer.from_config(cfg)
    start = torch.randint(0, V, (96, 1))
    seq = [start]
    for _ in range(T):
        seq.append((seq[-1] * 5 + 3) % V)  # a fixed next-token rule: learnable by every exit
    data = torch.cat(seq, dim=1)
    train, val = data[:80], data[80:]
    before = evaluate_all_depths(model, val)
    rep = rescue_checkpoint(model, train, val, deepen_steps=30, align_steps=10, joint_steps=10, lr=3e-3, batch_size=8)
    assert set(rep["stages"]) == {"deepen", "align", "joint"} and rep["tokens_trained"] == 50 * 8 * T
    assert rep["before"]["cortex"]["loss"] == pytest.approx(before["cortex"]["loss"])
    assert rep["after"]["cortex"]["loss"] < before["cortex"]["loss"] - 0.5
    assert rep["stages"]["align"]["val"]["reflex"]["loss"] < rep["stages"]["deepen"]["val"]["reflex"]["loss"]
    assert all(rep["improved"][n] > 0 for n in ("reflex", "limbic", "cortex"))
    assert rep["config_update"]["depth_mode"] == "joint" and all(p.requires_grad for p in model.parameters())


@pytest.mark.parametrize("victim,mode,strict", [(2, "between", "0"), (0, "midstep", "0"), (1, "between", "1")])
def test_elastic_data_parallel_survives_a_lost_rank(tmp_path, victim, mode, strict):
    """Three gloo ranks; one leaves without notice (between steps, or when the others are already inside the step's
    all-reduce; once the lowest rank, which also writes the checkpoints). The survivors detect it by heartbeat or by
    the process group's timeout, re-form as two ranks, reload the last checkpoint, finish all steps and agree on the
    weights. The store lives in this process, so it outlives every rank."""
    import json
    import re

    from triune_b200.parallel.elastic import connect_store
    from triune_b200.desktop import find_free_port

    port = find_free_port(29800, attempts=100)
    store = connect_store("127.0.0.1", port, is_master=True)  # noqa: F841  (kept alive for the workers)
    env = dict(os.environ, OMP_NUM_THREADS="1", EL_PORT=str(port), EL_WORLD="3", EL_VICTIM=str(victim), EL_DIE_AT="5",
               EL_MODE=mode, EL_CKPT=str(tmp_path / "ck.pt"), EL_STEPS="8", EL_STRICT=strict)  # strict: meet on the store before every step
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "mp_elastic_worker.py")], env=dict(env, EL_IDENT=str(i)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for i in range(3)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=240))
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate())
    assert procs[victim].returncode == 17
    res = []
    for i, (p, (so, se)) in enumerate(zip(procs, outs)):
        if i == victim:
            continue
        assert p.returncode == 0, (i, so[-1500:], se[-1500:])
        res.append(json.loads(re.search(r"RESULT (\{.*\})", so).group(1)))
    survivors = sorted(set(range(3)) - {victim})
    for r in res:
        assert r["steps"] == 8 and r["world"] == 2 and r["members"] == survivors and r["generation"] == 1
        assert r["failures"] == [[victim]]
    assert res[0]["w"] == res[1]["w"] and any(abs(v) > 1e-3 for v in res[0]["w"])


def test_elastic_training_command_survives_a_killed_rank(tmp_path):
    """`triune_b200 train` under the elastic environment, three gloo ranks: one process is killed (by its exact handle)
    once the first checkpoint exists; the others re-form as two ranks, reload that checkpoint and finish all steps."""
    import json
    import re
    import time

    from triune_b200.desktop import find_free_port
    from triune_b200.parallel.elastic import connect_store

    port = find_free_port(29900, attempts=100)
    store = connect_store("127.0.0.1", port, is_master=True)  # noqa: F841
    ck = tmp_path / "ck"
    tiny = json.dumps(dict(vocab_size=256, hidden_dim=64, num_layers=5, num_heads=2, head_dim=32, num_experts=4, reflex_exit_layer=2,
                           limbic_exit_layer=3, router_prefix_layers=1))
    cmd = [sys.executable, "-m", "triune_b200", "train", "--model", "triune-nano", "--overrides", tiny, "--batch-size", "2",
           "--seq-len", "32", "--steps", "60", "--log-every", "5", "--checkpoint-dir", str(ck)]
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=ROOT, TRIUNE_ELASTIC_STORE=f"127.0.0.1:{port}", TRIUNE_ELASTIC_WORLD="3",
               TRIUNE_ELASTIC_HB_TIMEOUT="1.0", TRIUNE_ELASTIC_PG_TIMEOUT="6.0", TRIUNE_ELASTIC_CKPT_EVERY="2")
    procs = [subprocess.Popen(cmd, env=dict(env, TRIUNE_ELASTIC_IDENT=str(i)), stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for i in range(3)]
    try:
        end = time.time() + 180
        while not (ck / "latest.pt").exists() and time.time() < end and all(p.poll() is None for p in procs):
            time.sleep(0.05)
        assert (ck / "latest.pt").exists(), "no checkpoint appeared"
        procs[1].kill()  # this exact child, mid-run and without notice
        outs = [p.communicate(timeout=300) for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    assert procs[0].returncode == 0 and procs[2].returncode == 0, (outs[0][1][-1500:], outs[2][1][-1500:])
    rep = json.loads(outs[0][0][outs[0][0].rindex('{\n  "steps"'):])
    assert rep["steps"] == 60 and rep["world"] == 2 and rep["members"] == [0, 2] and rep["failures"] == [[1]]
    assert rep["generation"] == 1 and "world 2" in outs[0][0]


def test_pipeline_times_data_parallel_on_gloo():
    """Four gloo ranks as two pipelines of two stages: each pipeline trains its own batch; after the average over the
    replicas every stage's gradients equal those of the whole model on both batches together."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1", PP_MICRO="4", PP_FAMILY="dense", PP_SIZE="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", "29743", os.path.join(ROOT, "tests", "mp_pp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0 and "PP_OK 4 4 pp2xdp2" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]


def _reference_checkpoint_module():
    import sys

    ref_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "triune")):
        pytest.skip("reference not installed")
    sys.path.insert(0, ref_dir)
    try:
        from triune.model.transformer import TriuneTransformer as RefModel
        from triune.trainer import checkpoint as ref_ckpt
    except Exception as e:  # pragma: no cover
        pytest.skip(f"reference import failed: {e}")
    finally:
        sys.path.remove(ref_dir)
    return RefModel, ref_ckpt


def test_checkpoint_fingerprint_and_files_interoperate_with_the_reference(tmp_path):
    """Schema-v2 contract: equal fingerprints for equal configs, and a file written by either project loads in the
    other through that project's own ``load_checkpoint`` (weights-only and with the fingerprint gate active)."""
    from types import SimpleNamespace

    from triune_b200.trainer import checkpoint as ckpt

    RefModel, ref_ckpt = _reference_checkpoint_module()
    arch = dict(vocab_size=256, hidden_dim=64, num_layers=5, num_heads=2, head_dim=32, num_experts=4,
                router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3)
    cfg = dict(arch, top_k=1, use_rope=True, shared_expert=True, target_depth_dist=(0.34, 0.33, 0.33), use_muon=True,
               muon_lr=0.02, lr=3e-4)
    assert ckpt.fingerprint(cfg) == ref_ckpt.compute_checkpoint_fingerprint(cfg)
    assert ckpt.canonical_semantics(cfg) == ref_ckpt.extract_canonical_semantics(cfg)
    assert ckpt.model_fingerprint(cfg) == ref_ckpt.compute_model_fingerprint(cfg)

    torch.manual_seed(0)
    ours = TriuneTransformer(**arch)
    ref = RefModel(**arch)
    x = torch.randint(0, 256, (2, 24))

    # ours -> reference
    p1 = ckpt.save_checkpoint(str(tmp_path / "ours.pt"), ours, None, step=7, loss=1.5, config=cfg)
    ref_trainer = SimpleNamespace(model=ref, optimizer=None, config=dict(cfg))
    got = ref_ckpt.load_checkpoint(ref_trainer, p1, load_optimizer=False)
    assert got["step"] == 7
    ours.eval(), ref.eval()
    with torch.no_grad():
        assert (ours(x, force_depth=2)[0] - ref(x, force_depth=2)[0]).abs().max() < 2e-3
    with pytest.raises(ValueError):
        ref_ckpt.load_checkpoint(SimpleNamespace(model=ref, optimizer=None, config=dict(cfg, hidden_dim=128)), p1,
                                 load_optimizer=False)

    # reference -> ours
    torch.manual_seed(1)
    ref2 = RefModel(**arch)
    eng = SimpleNamespace(best_eval_loss=2.0, depth_usage_ema=None)
    tr = SimpleNamespace(model=ref2, optimizer=None, config=dict(cfg, checkpoint_dir=str(tmp_path)), logger=None)
    p2 = ref_ckpt.save_latest(tr, eng, 11, 0.9)
    ours2 = TriuneTransformer(**arch)
    ck = ckpt.load_checkpoint(str(p2), model=ours2, config=dict(cfg))
    assert ck["step"] == 11
    ours2.eval(), ref2.eval()
    with torch.no_grad():
        assert (ours2(x, force_depth=2)[0] - ref2(x, force_depth=2)[0]).abs().max() < 2e-3
    with pytest.raises(ValueError, match="architecture.num_layers"):
        ckpt.load_checkpoint(str(p2), model=None, config=dict(cfg, num_layers=6))
    # an optimizer-only difference is tolerated when only the weights are loaded
    ckpt.load_checkpoint(str(p2), model=None, config=dict(cfg, muon_lr=0.5))


def test_checkpoint_loader_refuses_pickled_code(tmp_path):
    """A file that needs the unrestricted unpickler is refused instead of executed."""
    import pickle

    from triune_b200.trainer import checkpoint as ckpt

    class Boom:
        def __reduce__(self):
            return (os.system, ("true",))

    path = tmp_path / "evil.pt"
    torch.save({"model_state": {}, "payload": Boom()}, path)
    with pytest.raises(Exception) as e:
        ckpt.load_checkpoint(str(path))
    assert isinstance(e.value, (pickle.UnpicklingError, RuntimeError))


def test_graphed_speculative_decoder_equals_greedy_and_accepts_agreeing_drafts():
    """The device-resident speculative round (drafts by the Reflex exit, one batched verification with per-token
    recurrent states, acceptance count as a device index) reproduces plain full-depth greedy decoding token for token:
    with random weights (drafts mostly rejected) and with a model whose early exit agrees with the full depth (every
    draft accepted, k + 1 tokens per round)."""
    from triune_b200.inference import GraphedGreedyDecoder, GraphedSpeculativeDecoder

    m = tiny().eval()
    prompt = torch.randint(0, 256, (1, 9), generator=torch.Generator().manual_seed(4))
    want = GraphedGreedyDecoder(m, batch_size=1, decode_depth=2).generate(prompt, 24)
    spec = GraphedSpeculativeDecoder(m, k_draft=3)
    got = spec.generate(prompt, 24)
    assert torch.equal(got, want)
    low = spec.acceptance_rate
    # make the layers after the Reflex exit the identity and give the Reflex exit the final head: drafts always agree
    with torch.no_grad():
        r = m.exit_layers[0]
        for blk in m.layers[r + 1 :]:
            blk.attn.gla.out_proj.weight.zero_()
            for p in blk.ffn.parameters():
                p.zero_()
        ex = m.layers[r]
        ex.exit_norm.load_state_dict(m.final_norm.state_dict())
        ex.exit_head.weight.copy_(m.final_head.weight)
        if ex.exit_head.bias is not None:
            ex.exit_head.bias.zero_() if m.final_head.bias is None else ex.exit_head.bias.copy_(m.final_head.bias)
    want2 = GraphedGreedyDecoder(m, batch_size=1, decode_depth=2).generate(prompt, 24)
    spec2 = GraphedSpeculativeDecoder(m, k_draft=3)
    got2 = spec2.generate(prompt, 24)
    assert torch.equal(got2, want2)
    assert spec2.acceptance_rate == 1.0 and spec2.acceptance_rate >= low
    assert int(spec2.rounds.item()) <= 8  # 23 tokens at 4 per round, checked every 8 rounds


def test_streaming_finds_the_layer_stack_of_foreign_models():
    """Layer streaming locates the block stack of models it did not build: Hugging Face style nesting, or any longest
    list of same-typed blocks; streamed layers of such a model still train."""
    import torch.nn as nn

    from triune_b200.runtime.streaming import StreamingConfig, enable_layer_streaming, find_layer_list

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(16, 16)

        def forward(self, x):
            return x + torch.tanh(self.lin(x))

    class Inner(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed_tokens = nn.Embedding(32, 16)
            self.layers = nn.ModuleList([Block() for _ in range(4)])

    class HFLike(nn.Module):
        def __init__(self):
            super().__init__()
            self.model = Inner()
            self.lm_head = nn.Linear(16, 32)

        def forward(self, ids):
            x = self.model.embed_tokens(ids)
            for l in self.model.layers:
                x = l(x)
            return self.lm_head(x)

    class Odd(nn.Module):
        def __init__(self):
            super().__init__()
            self.stem = nn.ModuleList([nn.Linear(4, 4)])
            self.tower = nn.ModuleList([Block() for _ in range(3)])

    torch.manual_seed(0)
    m = HFLike()
    assert find_layer_list(m) is m.model.layers
    assert find_layer_list(Odd()) is not None and len(find_layer_list(Odd())) == 3
    try:
        find_layer_list(m, "transformer.h")
        assert False
    except AttributeError:
        pass
    eng = enable_layer_streaming(m, "cpu", config=StreamingConfig(resident_gpu_layers=1, pin_memory=False))
    assert len(eng.stores) == 3
    ids = torch.randint(0, 32, (2, 6))
    before = m.model.layers[2].lin.weight.detach().clone()
    loss = torch.nn.functional.cross_entropy(m(ids).reshape(-1, 32), ids.reshape(-1))
    loss.backward()
    eng.step_streaming_optimizer(None, lr=1e-2)
    assert not torch.equal(before, m.model.layers[2].lin.weight.detach())


def test_streaming_fp8_weight_staging_and_bf16_gradient_staging():
    """``fp8_weights``: the forward / backward passes receive an E4M3 copy (one fp32 scale per 128 elements, 1-D tensors
    beside it unquantised) and about half the bytes; ``grad_dtype="bf16"`` halves the gradient traffic. The master copy
    keeps training: the loss of the streamed model stays close to the unquantised one and falls."""
    from triune_b200.runtime.streaming import StreamingConfig, enable_layer_streaming

    x = torch.randint(0, 256, (2, 16), generator=torch.Generator().manual_seed(0))
    y = torch.randint(0, 256, (2, 16), generator=torch.Generator().manual_seed(1))

    def run(cfg, steps=3):
        m = tiny()
        eng = enable_layer_streaming(m, "cpu", config=cfg)
        losses = []
        for _ in range(steps):
            l = m.forward_loss(x, y, force_depth=2)
            l = l[0] if isinstance(l, tuple) else l
            l.backward()
            eng.step_streaming_optimizer(None, lr=5e-3)
            losses.append(float(l))
        return losses, eng

    base, e0 = run(StreamingConfig(resident_gpu_layers=0, pin_memory=False))
    q, e1 = run(StreamingConfig(resident_gpu_layers=0, pin_memory=False, fp8_weights=True, grad_dtype="bf16"))
    assert abs(q[0] - base[0]) < 5e-2 and q[-1] < q[0]          # FP8 weights perturb the loss a little; it still falls
    t0, t1 = e0.get_telemetry(), e1.get_telemetry()
    st = next(iter(e1.stores.values()))
    assert st.host_q.dtype == torch.float8_e4m3fn and st.host_grad.dtype == torch.bfloat16
    assert st.fp8_stage_bytes() < 0.3 * st.numel * 4            # fp32 test model: 1.03 bytes per weight against 4
    assert t1["h2d_bytes"] < 0.75 * t0["h2d_bytes"]             # weights in: 2 x 1.03 instead of 2 x 4 bytes; gradient back in bf16
    assert t1["d2h_bytes"] < 0.97 * t0["d2h_bytes"]             # gradient out in bf16, plus the refreshed FP8 copy
    # norm weights and biases are staged exactly
    for p, (off, n, shape) in zip(st.params, st.slices):
        if p.dim() < 2:
            assert torch.equal(st.expand_fp8("cpu")[off : off + n].view(shape), st.host[off : off + n].view(shape))


def test_streamed_model_keeps_dynamic_depth_forced_exits_all_exits_cached_decode_and_jev():
    """With its layers streamed from the host, the model still chooses a depth per sequence, honours a forced depth, gives
    all three exits at once, decodes step by step through the recurrent cache with the logits of the resident model, and
    runs the JEV exit policy; afterwards no layer stays staged (tests/test_streaming_dynamic_depth.py:13-108)."""
    from triune_b200.runtime.streaming import LayerStreamingEngine, StreamingConfig

    ref, m = tiny(3).eval(), tiny(3).eval()
    eng = LayerStreamingEngine(m, device="cpu", config=StreamingConfig(enabled=True, async_prefetch=True, pin_memory=False))
    eng.attach()
    x = torch.randint(0, 256, (2, 16))
    with torch.no_grad():
        logits, route = m(x)
        assert logits.shape == (2, 16, 256) and route.shape == (2, 3)
        assert m.last_depth_choice is not None and bool(torch.isin(m.last_depth_choice, torch.tensor([0, 1, 2])).all())
        for depth in (0, 1, 2):
            forced, froute = m(x, force_depth=depth)
            assert forced.shape == (2, 16, 256) and froute.shape == (2, 3) and bool((m.last_depth_choice == depth).all())
            assert torch.allclose(forced, ref(x, force_depth=depth)[0], atol=1e-5)
        outs = m.forward_all_exits(x)
        assert [tuple(o.shape) for o in outs] == [(2, 16, 256)] * 3 + [(2, 3)]
        for o, r in zip(outs, ref.forward_all_exits(x)):
            assert torch.allclose(o, r, atol=1e-5)
        cache, rcache = m.init_cache(2), ref.init_cache(2)
        for t in range(3):
            tok = x[:, t : t + 1]
            out, cache = m(tok, cache=cache, force_depth=2)
            rout, rcache = ref(tok, cache=rcache, force_depth=2)
            assert out.shape == (2, 1, 256) and torch.allclose(out, rout, atol=1e-5)
        assert len(cache) == len(m.layers) and all(c is not None for c in cache)
        m.enable_jev_routing(threshold=0.0)
        jl, _ = m(x, exit_policy="jev")
        assert jl.shape == (2, 16, 256) and bool(torch.isfinite(jl).all())
    assert all(v == 0 for v in eng._staged.values())
    assert sum(st.device_buf is not None for st in eng.stores.values()) <= 1  # at most the layer prefetched past an exit
    eng.drop_prefetched()
    assert all(st.device_buf is None for st in eng.stores.values())
    eng.detach()
