"""CPU tests of the framework components around the model core: zoo, exits, JEV, conversion, LoRA, tokenizers, data,
export, staging, planning, session state, callbacks."""

import json
import os
import sys

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from triune_b200.config import ModelConfig
from triune_b200.models import TriuneTransformer

CFG = dict(vocab_size=256, hidden_dim=64, num_layers=5, num_heads=2, head_dim=32, num_experts=4, top_k=2, router_prefix_layers=1,
           reflex_exit_layer=2, limbic_exit_layer=3, expert_hidden=96, dense_hidden=80)


def tiny():
    torch.manual_seed(0)
    return TriuneTransformer.from_config(ModelConfig(**CFG))


class Tok:
    def encode(self, s):
        return [ord(c) % 256 for c in s]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(int(i)) for i in ids)


# ------------------------------------------------------------------------------------------------ zoo / specs
def test_model_specs_clamp_and_resolve(tmp_path):
    from triune_b200.models.zoo import CANONICAL_MODEL_SPECS, get_model_spec, load_model, register_model

    assert len(CANONICAL_MODEL_SPECS) == 11 and CANONICAL_MODEL_SPECS["triune-base"].compute_exact_params()[0] == 90_789_271
    s = get_model_spec("triune-micro", num_layers=3, reflex_exit_layer=9, limbic_exit_layer=9)
    assert s.num_layers == 4 and 0 < s.router_prefix_layers < s.reflex_exit_layer < s.limbic_exit_layer < s.num_layers
    assert get_model_spec("triune-nano", precision="float8_e4m3").use_fp8
    assert get_model_spec("triune-nano", hidden_dim=384).head_dim == 128  # 3 heads kept, head_dim follows hidden_dim
    m = load_model("triune-nano", vocab_size=512)
    assert sum(p.numel() for p in m.parameters()) == get_model_spec("triune-nano", vocab_size=512).compute_exact_params()[0]

    @register_model("unit-test-arch")
    class Toy(nn.Module):
        def __init__(self, n=3):
            super().__init__()
            self.l = nn.Linear(n, n)

    assert isinstance(load_model("unit-test-arch", n=5), Toy)
    p = tmp_path / "m.pt"
    torch.save({"model_state": m.state_dict(), "config": {}}, p)
    m2 = load_model(str(p))
    assert all(torch.equal(a, b) for a, b in zip(m.state_dict().values(), m2.state_dict().values()))
    with pytest.raises(ValueError):
        load_model("definitely-not-a-model")


# ------------------------------------------------------------------------------------------------ JEV / exits
def test_jev_objective_and_router():
    from triune_b200.models.jev import JEVExitRouter, JEVLatentPredictor, JEVObjective

    torch.manual_seed(0)
    p = JEVLatentPredictor(32)
    z, t = torch.randn(4, 7, 32), torch.randn(4, 7, 32)
    for mode in ("euclidean", "geodesic", "stiefel"):
        loss, parts = JEVObjective(stp_mode=mode)(p(z), t, return_dict=True)
        assert torch.isfinite(loss) and set(parts) == {"l_sim", "l_stp", "l_cov", "total_loss"}
    assert float(JEVObjective().compute_sim_loss(t, t)) < 1e-6 and float(JEVObjective().compute_stp_loss(t, t)) == 0.0
    for metric in ("cosine", "euclidean", "geodesic", "stp_tube", "learned"):
        r = JEVExitRouter(32, distance_metric=metric)(z, z)
        assert r.should_exit.shape == (4, 7)
        if metric != "learned":
            assert bool(r.should_exit.all())  # identical latents are always confident
    with pytest.raises(ValueError):
        JEVExitRouter(32, distance_metric="manhattan")


def test_early_exit_adapters_on_foreign_model():
    from triune_b200.models.adapters import WeightTiedExitProjection, attach_early_exits

    class Blk(nn.Module):
        def __init__(self):
            super().__init__()
            self.l = nn.Linear(32, 32)

        def forward(self, x):
            return (x + torch.tanh(self.l(x)),)

    class LM(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb, self.layers, self.lm_head = nn.Embedding(100, 32), nn.ModuleList(Blk() for _ in range(8)), nn.Linear(32, 100, bias=False)

        def forward(self, ids):
            x = self.emb(ids)
            for l in self.layers:
                x = l(x)[0]
            return self.lm_head(x)

    torch.manual_seed(0)
    m = attach_early_exits(LM(), rank=8, use_jev=True)
    assert m.reflex_layer_idx == 2 and m.limbic_layer_idx == 4
    x = torch.randn(2, 5, 32)
    head = m.reflex_head
    assert isinstance(head, WeightTiedExitProjection) and len(head.adapter_parameters()) == 3
    assert torch.allclose(head(x), m.lm_head(head.norm(x)), atol=1e-6)  # zero-initialised up-projection
    out = m.generate_adaptive(torch.randint(0, 100, (1, 4)), max_new_tokens=5, use_jev=False)
    assert sum(out["exit_counts"].values()) == len(out["generated_token_ids"]) <= 5
    out = m.generate_adaptive(torch.randint(0, 100, (1, 4)), max_new_tokens=3, confidence_threshold=0.0)
    assert out["exit_counts"]["reflex"] == 3 and out["flops_saved_pct"] > 50


def test_low_rank_embedding_factorisation():
    from triune_b200.models.manifold_embedding import UniversalAdaptiveEmbedding

    torch.manual_seed(0)
    W = torch.randn(300, 12) @ torch.randn(12, 40)
    e = UniversalAdaptiveEmbedding.from_pretrained_weights(W, rank=12)
    assert (e(torch.arange(300)) - W).abs().max() < 1e-3
    h = torch.randn(3, 40)
    assert torch.allclose(e.compute_logits(h), h @ e(torch.arange(300)).t(), atol=1e-3)
    vals, idx = e.compute_logits(h, top_k=5)
    assert idx.shape == (3, 5)


def test_transmuter_weight_surgery_and_distillation():
    transformers = pytest.importorskip("transformers")
    from triune_b200.models.transmuter import (distill_native_triune_step, expand_gqa_weight, ollama_to_hf_candidate,
                                                transfer_weights_to_native_triune, transmute_hf_to_triune)

    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=300, hidden_size=128, intermediate_size=256, num_hidden_layers=6,
                                   num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=False)
    teacher = transformers.LlamaForCausalLM(cfg)
    student, rep = transfer_weights_to_native_triune(teacher, num_experts=4, top_k=2)
    assert rep["weights_transferred"] and rep["lm_head_untied"] and rep["student_layers"] == 6
    hd = 128
    k_t = teacher.model.layers[0].self_attn.k_proj.weight
    assert torch.equal(student.layers[0].attn.gla.qkvg_weight[hd : 2 * hd], expand_gqa_weight(k_t, 4, 2))
    assert torch.equal(student.token_embed.weight, teacher.model.embed_tokens.weight)
    ids = torch.randint(0, 300, (2, 16))
    opt = torch.optim.AdamW(student.parameters(), lr=1e-3)
    a = distill_native_triune_step(student, teacher, ids, opt)
    b = distill_native_triune_step(student, teacher, ids, opt)
    assert b["loss"] < a["loss"]
    m, meta = transmute_hf_to_triune(teacher, use_jev=False)
    assert meta["transmute_mode"] == "early_exit" and hasattr(m, "generate_adaptive")
    assert ollama_to_hf_candidate("ollama:gemma3:4b-instruct-q4_K_M") == "google/gemma-3-4b-it"
    assert ollama_to_hf_candidate("org/repo") == "org/repo" and ollama_to_hf_candidate("nonexistent:1b") is None


# ------------------------------------------------------------------------------------------------ LoRA / quantised modules
DATA = [{"prompt": "hello ", "completion": "world!"}, {"instruction": "say hi", "output": "hi there"},
        {"messages": [{"role": "user", "content": "a"}, {"role": "assistant", "content": "bcd"}]}, "plain text sample"] * 3


def test_lora_finetune_save_load_merge(tmp_path):
    from triune_b200.trainer.finetune import LoRAConfig, TriuneFineTuner, list_adapters, merge_adapter_checkpoint

    m = tiny()
    n_base = sum(p.numel() for p in m.parameters())
    ft = TriuneFineTuner(m, LoRAConfig(rank=8, dropout=0.0), tokenizer=Tok())
    assert all(not p.requires_grad for n, p in m.named_parameters() if "lora" not in n)
    assert 0 < ft.count_trainable_parameters() < 0.2 * n_base
    ex = ft.build_examples(DATA, max_seq_len=32)
    assert any((y == -100).any() for _, y in ex)  # prompt tokens are masked
    r = ft.fit(DATA, epochs=6, batch_size=4, lr=5e-3)
    assert r["final_loss"] < r["first_loss"]
    x = torch.randint(0, 256, (1, 9))
    m.eval()
    y_adapted = m(x, force_depth=2)[0]
    d = ft.save_adapter(tmp_path / "ad")
    cfg = json.loads((d / "adapter_config.json").read_text())
    assert cfg["peft_type"] == "LORA" and cfg["r"] == 8 and (d / "adapter_model.safetensors").is_file()
    assert list_adapters([str(tmp_path)])[0]["rank"] == 8
    ft.detach_lora()
    assert not any("lora" in k for k in m.state_dict())
    y_base = m(x, force_depth=2)[0]
    assert (y_base - y_adapted).abs().max() > 1e-4
    merge_adapter_checkpoint(m, d)
    assert torch.allclose(m(x, force_depth=2)[0], y_adapted, atol=1e-4)


def test_qlora_and_quantised_converters():
    from triune_b200.models.quant_linear import FP4Linear, NVFP4Linear, convert_to_fp8, convert_to_nvfp4
    from triune_b200.trainer.finetune import LoRAConfig, TriuneFineTuner

    m = tiny()
    ft = TriuneFineTuner(m, LoRAConfig(rank=8, use_qlora=True, quantization="4-bit NVFP4", dropout=0.0), tokenizer=Tok())
    assert sum(isinstance(getattr(a, "original_layer", None), NVFP4Linear) for a in ft.applied_adapters.values()) > 0
    r = ft.fit(DATA, epochs=2, batch_size=4, lr=5e-3)
    assert torch.isfinite(torch.tensor(r["final_loss"]))
    m2 = tiny().eval()
    x = torch.randint(0, 256, (2, 8))
    want = m2(x, force_depth=2)[0]
    assert convert_to_fp8(m2) > 0
    assert torch.nn.functional.cosine_similarity(m2(x, force_depth=2)[0].flatten(), want.flatten(), dim=0) > 0.99
    m3 = tiny().eval()
    n = convert_to_nvfp4(m3, hadamard=True)
    assert n > 0 and not any(isinstance(mod, NVFP4Linear) for name, mod in m3.named_modules() if "exit_head" in name or "router" in name)
    assert torch.nn.functional.cosine_similarity(m3(x, force_depth=2)[0].flatten(), want.flatten(), dim=0) > 0.9
    lin = FP4Linear(32, 16)
    lin(torch.randn(3, 32)).sum().backward()
    assert lin.weight.grad is not None and NVFP4Linear.from_linear(nn.Linear(64, 8)).bits_per_weight() == 4.5


# ------------------------------------------------------------------------------------------------ tokenizers / data
CORPUS = ["the quick brown fox jumps over the lazy dog. " * 6, "héllo wörld — naïve café 日本語 🙂 snake_case",
          "def f(x):\n    return x + 123456\n" * 4] * 4


def test_bpe_tokenizer_roundtrip_and_fast_parity(tmp_path):
    from triune_b200.data.tokenizer import SPECIAL_TOKENS, load_tokenizer, train_bpe

    tok = train_bpe(CORPUS, vocab_size=400)
    assert len(SPECIAL_TOKENS) == 21 and tok.token_to_id("[PAD]") == 0
    s = "<|user|>the quick café 🙂 12345 a_b\n<|eot_id|>"
    ids = tok.encode(s)
    assert ids.ids == list(ids) and tok.decode(ids, skip_special_tokens=False) == s and "<|user|>" not in tok.decode(ids)
    tok.save(tmp_path / "t.json")
    slow = load_tokenizer(tmp_path / "t.json", prefer_fast=False)
    assert list(slow.encode(s)) == list(ids)
    pytest.importorskip("tokenizers")
    fast = load_tokenizer(tmp_path / "t.json")
    for t in ("the quick café 12345", "def f(x):\n    return  x_1 + 99\n\n", "日本語 🙂 it's"):
        assert fast.encode(t).ids == list(slow.encode(t)) and fast.decode(fast.encode(t).ids) == t
    buf, out = bytearray(), ""
    for i in tok.encode("café 🙂 ok"):
        buf, piece = tok.decode_stream_step(buf, i)
        out += piece
        assert "�" not in piece  # never half a UTF-8 sequence
    assert out == "café 🙂 ok"
    assert tok.apply_chat_template([{"role": "user", "content": "hi"}]).endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")


def test_token_stream_dataset_packing_and_holdout(tmp_path):
    from triune_b200.data.dataset import TokenStreamDataset, build_dataloader
    from triune_b200.data.tokenizer import train_bpe

    tok = train_bpe(CORPUS, vocab_size=350)
    ds = TokenStreamDataset(tok, seq_len=32, sep_token_id=tok.sep_token_id, texts=CORPUS, shuffle_buffer=8)
    items = list(ds)
    assert len(items) > 4 and all(x.shape == (32,) and torch.equal(x[1:], y[:-1]) for x, y in items)
    p = tmp_path / "c.jsonl"
    p.write_text("\n".join(json.dumps({"text": t}) for t in CORPUS))
    from_file = list(TokenStreamDataset(tok, seq_len=32, sep_token_id=tok.sep_token_id, dataset_name=str(p), shuffle_buffer=1))
    assert len(from_file) == len(items)
    two = [len(list(TokenStreamDataset(tok, seq_len=32, sep_token_id=3, texts=CORPUS, rank=r, world_size=2))) for r in (0, 1)]
    assert abs(two[0] - two[1]) <= 2 and sum(two) <= len(items) + 2  # ranks read disjoint documents
    cfg = {"batch_size": 2, "seq_len": 32, "eval_batches": 2}
    hold = list(build_dataloader(tok, cfg, tok.sep_token_id, is_holdout=True, texts=CORPUS))
    assert len(hold) == 2 and hold[0][0].shape == (2, 32)


def test_dynamic_tokenizer_is_lossless():
    from triune_b200.data.dynamic_tokenizer import DynamicTokenizer
    from triune_b200.data.tokenizer import train_bpe

    dt = DynamicTokenizer(train_bpe(CORPUS, vocab_size=350))
    s = "the quick brown fox jumps over the lazy dog. " * 8 + "def f(x):\n    return x\n"
    o = dt.encode(s, return_chunks=True)
    assert 2.2 <= o.compression_ratio <= 4.5 and dt.decode(o.input_ids) == s and dt.decode(dt.unpack_chunks(o.chunks)) == s
    assert all(len(c) == dt.chunk_size for c in o.chunks) and max(o.input_ids) >= dt.dynamic_id_start
    b = dt.encode_batch([s, "hello world"])
    assert dt.decode_batch(b["input_ids"], b["attention_mask"]) == [s, "hello world"]
    assert dt.learn_ngrams(CORPUS, max_new_rules=10) > 0
    tab = dt.lookup_vector(8)
    first = dt.dynamic_id_start
    assert tab[0, 1 : 1 + min(8, int(tab[0, 0]))].tolist() == dt._expand_token(first)[:8]
    fallback = DynamicTokenizer()
    t = "héllo héllo héllo héllo wörld"
    assert fallback.decode(fallback.encode(t).input_ids) == t


# ------------------------------------------------------------------------------------------------ export
def test_safetensors_io_and_hf_bundle(tmp_path):
    from triune_b200.export import export_model, export_to_huggingface, load_file, load_from_huggingface, save_file

    t = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7), "s": torch.tensor(3), "e": torch.empty(0, 3)}
    save_file(t, str(tmp_path / "x.safetensors"), {"format": "pt"})
    back = load_file(str(tmp_path / "x.safetensors"))
    assert all(torch.equal(back[k], t[k]) for k in t)
    st = pytest.importorskip("safetensors.torch")
    assert all(torch.equal(v, t[k]) for k, v in st.load_file(str(tmp_path / "x.safetensors")).items())
    m = tiny().eval()
    d = export_to_huggingface(m, tmp_path / "hf")
    assert {"config.json", "generation_config.json", "configuration_triune.py", "modeling_triune.py", "model.safetensors"} <= set(os.listdir(d))
    keys = set(load_file(str(d / "model.safetensors")))
    assert "transformer.layers.0.attn.gla.q_proj.weight" in keys and "transformer.layers.3.ffn.experts.0.0.weight" in keys
    assert "transformer.final_head.weight" in keys and "transformer.token_embed.weight" in keys  # tied tensors stored twice
    m2 = load_from_huggingface(d)
    x = torch.randint(0, 256, (2, 12))
    assert torch.equal(m(x, force_depth=2)[0], m2(x, force_depth=2)[0])
    with pytest.raises(NotImplementedError):
        export_model(m, tmp_path / "m.gguf", "gguf")
    with pytest.raises(ValueError):
        export_model(m, tmp_path / "l.safetensors", "lora")


# ------------------------------------------------------------------------------------------------ runtime services
@pytest.mark.parametrize("kw,min_cos", [({}, 0.99999), ({"use_fp8": True}, 0.995), ({"use_fp4": True}, 0.97)])
def test_parameter_stager_roundtrip(kw, min_cos):
    from triune_b200.runtime.staging import ParameterStager

    torch.manual_seed(0)
    ref_layer = nn.Sequential(nn.Linear(512, 256), nn.BatchNorm1d(256), nn.Linear(256, 64))
    layer = nn.Sequential(nn.Linear(512, 256), nn.BatchNorm1d(256), nn.Linear(256, 64))
    layer.load_state_dict(ref_layer.state_dict())
    x = torch.randn(8, 512)
    want = ref_layer(x)
    st = ParameterStager("cpu", min_quant_numel=1000, **kw)
    st.register_module(layer)
    st.stage_layer(layer)
    y = layer(x)
    assert torch.nn.functional.cosine_similarity(y.flatten(), want.flatten(), dim=0) > min_cos
    st.release_layer(layer, clear_snapshot=True)
    s = st.get_memory_summary()
    assert s["gpu_bytes"] == 0 and s["h2d_bytes_transferred"] == s["transfer_bytes_per_pass"]
    assert (s["transfer_bytes_per_pass"] < 0.5 * s["cpu_master_bytes"]) == bool(kw)
    assert torch.allclose(layer[1].running_mean, ref_layer[1].running_mean, atol=5e-2) and layer[1].running_mean.abs().sum() > 0  # written back
    assert torch.equal(layer[0].weight, ref_layer[0].weight)  # masters untouched by compressed staging


def test_memory_planner_and_resource_manager():
    from triune_b200.config import get_model_config
    from triune_b200.runtime.memory_planner import MemoryPlanner
    from triune_b200.runtime.resource_manager import DynamicResourceManager, HardwareProfile, VRAMBudgetExceededError

    small = MemoryPlanner.estimate_vram({**get_model_config("bench-90m").to_dict(), "batch_size": 16, "seq_len": 2048}, available_vram_gb=180)
    assert small.fits and small.recommended_mode == "resident" and small.total_params == 99_663_531
    big = MemoryPlanner.estimate_vram({**get_model_config("triune-70b").to_dict(), "batch_size": 16, "seq_len": 2048}, available_vram_gb=180)
    assert not big.fits and big.recommended_mode in ("layer_streaming", "disk_streaming")
    hf = MemoryPlanner.estimate_hf_model({"hidden_size": 4096, "num_hidden_layers": 32, "vocab_size": 128256, "intermediate_size": 14336,
                                          "num_attention_heads": 32, "num_key_value_heads": 8}, available_vram_gb=180)
    assert abs(hf["total_params"] - 8.03e9) < 0.05e9 and hf["fits"]
    hw = HardwareProfile("B200", 180, 178, 2, (10, 0), True, True, False, 148, 8)
    cfg = {**get_model_config("triune-7b").to_dict(), "batch_size": 16, "seq_len": 2048}
    a = DynamicResourceManager.assess_feasibility(cfg, hardware=hw)
    assert not a.is_feasible and a.suggested_batch_size * a.suggested_grad_accum >= 16
    with pytest.raises(VRAMBudgetExceededError):
        DynamicResourceManager.validate_and_allot(cfg, hardware=hw)
    assert DynamicResourceManager.validate_and_allot(cfg, hardware=hw, force=True).forced_override
    plan = DynamicResourceManager.validate_and_allot(cfg, hardware=hw, auto_fit=True)
    assert plan.auto_fitted and plan.batch_size == a.suggested_batch_size


def test_session_state_manager_lru_ttl_and_queue():
    import time

    from triune_b200.serve.srsm import ServingRequestQueue, SessionRecurrentStateManager

    m = SessionRecurrentStateManager(max_active_sessions=2, session_ttl_seconds=0.3)
    c = [(torch.randn(2, 3, 4, 4), 7), (None, 7), (torch.randn(2, 3, 4, 4), 7)]
    m.update_session_cache("a", c, depth=2)
    got, depth = m.get_session_cache("a", "cpu")
    assert depth == 2 and torch.equal(got[0][0], c[0][0]) and got[1] == (None, 7) and got[2][1] == 7
    got[0][0].zero_()  # a caller mutating its copy must not corrupt the parked state
    assert torch.equal(m.get_session_cache("a", "cpu")[0][0][0], c[0][0])
    m.update_session_cache("b", c)
    m.update_session_cache("c", c)
    assert m.get_session_cache("a", "cpu") is None and m.stats()["active_sessions"] == 2
    time.sleep(0.35)
    assert m.get_session_cache("c", "cpu") is None
    q = ServingRequestQueue(1)
    ev = q.register_request("r")
    assert q.acquire(0.05) and not q.acquire(0.05) and q.cancel_request("r") and ev.is_set() and not q.cancel_request("zz")


def test_callbacks_events_and_loggers(tmp_path):
    from triune_b200.callbacks import Callback, CallbackList, EventEmitter, TelemetryCallback
    from triune_b200.trainer.logger import JsonlLogger, NullLogger

    class Count(Callback):
        n = 0

        def on_step_end(self, trainer, step, logs):
            Count.n += 1

    tel = TelemetryCallback()
    cl = CallbackList([Count(), tel])
    cl.on_train_begin(None)
    cl.on_step_end(type("T", (), {"device": None})(), 3, {"loss": torch.tensor(1.5)})
    assert Count.n == 1 and tel.history[0]["loss"] == 1.5 and tel.history[0]["step"] == 3
    em, got = EventEmitter(), []
    em.on("on_loss_update", got.append)
    em.on("on_loss_update", lambda p: 1 / 0)  # a failing listener is isolated
    em.emit_loss_update(1, 2.0)
    assert got[0]["loss"] == 2.0 and "timestamp" in got[0]
    lg = JsonlLogger(tmp_path / "run.jsonl", config={"lr": 1e-3})
    lg.log({"loss": torch.tensor(0.5)}, step=4)
    lg.finish()
    lines = [json.loads(l) for l in (tmp_path / "run.jsonl").read_text().splitlines()]
    assert lines[0]["config"]["lr"] == 1e-3 and lines[1] == {**lines[1], "step": 4, "loss": 0.5}
    assert NullLogger().log({}, step=0) is None


def test_sandbox_validation_and_limits():
    from triune_b200.runtime.sandbox import PythonSandbox

    sb = PythonSandbox(timeout=5)
    ok = sb.execute_code("import math\nresult = math.sqrt(x) + 1\nprint('hi')", {"x": 16})
    assert ok["success"] and ok["result"] == 5.0 and ok["stdout"] == "hi\n"
    for bad in ("import os", "open('/etc/passwd')", "().__class__", "from subprocess import run", "eval('1')"):
        assert not sb.execute_code(bad)["success"]
    assert sb.execute_code("while True: pass")["timed_out"]
    assert "ZeroDivisionError" in sb.execute_code("result = 1/0")["error"]


# ------------------------------------------------------------------------------------------------ DAG / plugins / agents / engines
def test_dag_validation_execution_and_signed_plugins(tmp_path):
    from triune_b200.execution.dag import DAGValidationError, execute_dag, node_catalog, parse_dag
    from triune_b200.plugins.registry import PluginError, PluginRegistry, file_sha256, sign_manifest

    over = {"vocab_size": 256, "hidden_dim": 64, "num_heads": 2, "head_dim": 32}
    spec = {"nodes": [{"id": "m", "type": "load_model", "params": {"model": "triune-nano", "overrides": over}}, {"id": "i", "type": "model_info"},
                      {"id": "t", "type": "text", "params": {"text": "hi"}}, {"id": "g", "type": "generate", "params": {"max_new_tokens": 3}},
                      {"id": "p", "type": "python", "params": {"code": "result = value['parameters'] > 0"}}],
            "edges": [{"from": "m.model", "to": "i.model"}, {"from": "m.model", "to": "g.model"}, {"from": "t.out", "to": "g.prompt"},
                      {"from": "i.out", "to": "p.value"}]}
    r = execute_dag(spec)
    assert r["order"].index("m") < r["order"].index("g") and r["outputs"]["p.out"] is True and isinstance(r["outputs"]["g.text"], str)
    for bad in ({"nodes": [{"id": "a", "type": "nope"}]}, {"nodes": [{"id": "a", "type": "concat_text"}]},
                {"nodes": [{"id": "a", "type": "text"}, {"id": "b", "type": "model_info"}], "edges": [{"from": "a.out", "to": "b.model"}]},
                {"nodes": [{"id": "a", "type": "python"}, {"id": "b", "type": "python"}],
                 "edges": [{"from": "a.out", "to": "b.value"}, {"from": "b.out", "to": "a.value"}]}):
        with pytest.raises(DAGValidationError):
            parse_dag(bad)
    assert any(n["type"] == "train_steps" for n in node_catalog())
    (tmp_path / "p1").mkdir()
    (tmp_path / "p1" / "main.py").write_text("def register(api):\n    @api.register_node('double', {'x': 'any'}, {'out': 'any'})\n"
                                              "    def f(i, p, c):\n        return {'out': i['x'] * 2}\n")
    sha = file_sha256(tmp_path / "p1" / "main.py")
    key = "k" * 32
    (tmp_path / "p1" / "plugin.json").write_text(json.dumps({"name": "p1", "version": "1", "entry": "main.py", "sha256": sha,
                                                              "signature": sign_manifest("p1", "1", sha, key)}))
    reg = PluginRegistry(key=key)
    reg.discover(tmp_path)
    assert reg.load("p1").nodes == ["p1.double"]
    out = execute_dag({"nodes": [{"id": "c", "type": "constant", "params": {"value": 21}}, {"id": "d", "type": "p1.double"}],
                       "edges": [{"from": "c.out", "to": "d.x"}]})
    assert out["outputs"]["d.out"] == 42
    wrong = PluginRegistry(key="z" * 32)
    wrong.discover(tmp_path)
    with pytest.raises(PluginError):
        wrong.load("p1")
    (tmp_path / "p1" / "main.py").write_text("def register(api):\n    pass\n# tampered\n")
    fresh = PluginRegistry(key=key)
    fresh.discover(tmp_path)
    with pytest.raises(PluginError):
        fresh.load("p1")


def test_agent_tools_and_url_guard():
    from triune_b200.agents import Agent, AgentMemory, MultiAgentOrchestrator, build_integrated_toolbelt, is_safe_public_url

    urls = ("http://127.0.0.1/x", "http://10.0.0.5", "https://224.0.0.1", "https://239.1.1.1", "ftp://example.com", "http://[ff02::1]/",
            "http://localhost:8000", "http://169.254.169.254/latest")
    assert not any(is_safe_public_url(u, resolve=False) for u in urls) and is_safe_public_url("http://93.184.216.34/", resolve=False)
    replies = iter(['<|tool_call|>{"tool": "python", "args": {"code": "result = 6*7"}}\n', "The answer is 42.", "ok"])
    a = Agent(lambda p: next(replies), tools=build_integrated_toolbelt())
    r = a.run("what is 6*7?")
    assert r["text"] == "The answer is 42." and r["tool_calls"][0]["result"]["result"] == 42
    assert MultiAgentOrchestrator({"a": a}).run("again")[0]["text"] == "ok"
    mem = AgentMemory(max_items=2)
    for k in "abc":
        mem.set(k, k)
    assert mem.get("a") is None and mem.get("c") == "c" and mem.delete("c") and not mem.delete("c")


def test_parallel_engine_and_disk_streaming(tmp_path):
    from triune_b200.runtime.disk_streaming import DiskNVFP4StreamingEngine, build_nvfp4_disk_cache, describe_cache
    from triune_b200.runtime.model_scanner import scan_models
    from triune_b200.runtime.parallel_engine import ParallelEngine

    torch.manual_seed(0)
    e = ParallelEngine(dim=64, heads=2, head_dim=32, num_experts=4, device="cpu")
    x = torch.randn(3, 64, 64)
    o, s = e.prefill_batched(x)
    assert o.shape == (3, 64, 64) and s.shape == (3, 2, 32, 32) and e.forward(x).shape == x.shape
    r = e.score_draft_chunks(torch.ones(2, 4, 8), torch.ones(2, 4, 8), 0.9)
    assert r["contiguous_accepted"].tolist() == [4, 4] and float(r["acceptance_rate"]) == 1.0
    assert e.benchmark_throughput(2, 64, iters=1, warmup=1)["tokens_per_s"] > 0
    transformers = pytest.importorskip("transformers")
    cfg = transformers.LlamaConfig(vocab_size=300, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                                   num_key_value_heads=2, tie_word_embeddings=False)
    m = transformers.LlamaForCausalLM(cfg).eval()
    m.save_pretrained(tmp_path / "hf", safe_serialization=True)
    man = build_nvfp4_disk_cache(tmp_path / "hf", tmp_path / "cache", hadamard=False, device="cpu")
    assert man["num_layers"] == 3 and man["compression"] > 2.5 and "mlp.up_proj" in man["quantized_modules"][0]
    assert build_nvfp4_disk_cache(tmp_path / "hf", tmp_path / "cache", hadamard=False, device="cpu") == man  # reused, not rebuilt
    eng = DiskNVFP4StreamingEngine(tmp_path / "cache", "cpu", dtype=torch.float32, prefetch=1, resident_budget_gb=0)
    st = eng.layer_state(0)
    w, ref_w = st["self_attn.q_proj.weight"], m.model.layers[0].self_attn.q_proj.weight
    assert torch.nn.functional.cosine_similarity(w.flatten(), ref_w.flatten(), dim=0) > 0.99
    assert torch.allclose(st["input_layernorm.weight"], m.model.layers[0].input_layernorm.weight, atol=1e-2)
    for i in range(3):
        eng.layer_state(i)
    assert eng.telemetry["layers_loaded"] >= 3 and eng.telemetry["evictions"] >= 1
    assert "model.embed_tokens.weight" in eng.root_state()
    eng.close()
    assert describe_cache(tmp_path / "cache")["num_layers"] == 3
    counts = scan_models([str(tmp_path)])["counts"]
    assert counts.get("hf_model") == 1 and counts.get("nvfp4_cache") == 1


def test_expert_parallel_positions_match_one_hot_cumsum():
    """Position of an assignment inside its expert, from one stable sort, equals the cumulative one-hot count."""
    import torch

    from triune_b200.parallel.expert_parallel import _positions

    torch.manual_seed(0)
    E = 16
    idx = torch.randint(-1, E, (5000,), dtype=torch.int32)  # -1 = dropped assignment
    pos, counts = _positions(idx, E)
    onehot = idx.view(-1, 1) == torch.arange(E, dtype=idx.dtype).view(1, -1)
    csum = onehot.to(torch.int32).cumsum(0, dtype=torch.int32)
    want = (csum.gather(1, idx.clamp_min(0).long().view(-1, 1)).view(-1) - 1).to(torch.int32)
    want = torch.where(idx >= 0, want, torch.full_like(want, -1))
    assert pos.dtype == torch.int32 and counts.dtype == torch.int32
    assert torch.equal(pos, want) and torch.equal(counts, csum[-1])


def test_launcher_starts_reuses_and_stops_the_server(tmp_path):
    """The launcher starts the API server as a child on a free port, recognises it as its own service on a second call
    (no second child), moves away from a port held by a foreign program, and stops the child it started."""
    import socket

    from triune_b200 import desktop

    pytest.importorskip("fastapi")
    pytest.importorskip("uvicorn")
    port = desktop.find_free_port(18700, attempts=200)
    with desktop.start_session(port, startup_timeout=180.0, quiet=True) as first:
        assert not first.reused and first.port == port and desktop.server_alive(port)
        again = desktop.start_session(port, quiet=True)
        assert again.reused and again.proc is None and again.port == port
        again.stop()  # must not touch the server it did not start
        assert desktop.server_alive(port)
    assert first.proc.poll() is not None and not desktop.server_alive(port)

    # a foreign listener on the wanted port: not our service, so the launcher would move on to another port
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        s.listen(1)
        held = s.getsockname()[1]
        assert desktop.port_in_use(held) and not desktop.server_alive(held, timeout=0.3)
        assert desktop.find_free_port(held, attempts=50) != held
    cmd = desktop.server_command(9001, model="bench-90m", static_dir="web", precision="bf16")
    assert cmd[1:4] == ["-m", "triune_b200", "serve"] and "--static-dir" in cmd and "9001" in cmd


def test_packaging_bundles(tmp_path):
    """Every platform bundle is generated as plain files with an entry that runs the desktop command; the POSIX
    launchers are executable and syntactically valid shell."""
    import subprocess

    from triune_b200.packaging import build_native_targets

    res = build_native_targets("all", out_dir=tmp_path)
    assert sorted(res) == ["linux", "macos", "windows"]
    for name, rec in res.items():
        entry = open(rec["entry"]).read()
        assert "-m triune_b200 desktop" in entry, name
    for name in ("linux", "macos"):
        assert os.access(res[name]["entry"], os.X_OK)
        assert subprocess.run(["bash", "-n", res[name]["entry"]]).returncode == 0
    assert os.path.isfile(os.path.join(res["linux"]["bundle"], "triune-b200.desktop"))
    assert os.path.isfile(os.path.join(res["macos"]["bundle"], "Contents", "Info.plist"))
    assert build_native_targets("mac", out_dir=tmp_path / "again").keys() == {"macos"}
    with pytest.raises(ValueError):
        build_native_targets("amiga", out_dir=tmp_path)


def test_mqar_recall_separates_the_mixers():
    """Analytic associative recall: every mixer answers the plain task; after a key is re-bound only the delta rule is
    guaranteed to return the fresh value (additive mixers keep the stale one in superposition)."""
    from triune_b200.evals import mqar

    tokens, answers = mqar.make_task(4, 128, 6, overwrite=True, seed=3)
    assert tokens.shape == (4, 128) and ((tokens[:, -1] >= mqar.KEYS[0]) & (tokens[:, -1] < mqar.KEYS[1])).all()
    for b in range(4):  # the queried key occurs twice before the query and its LAST binding is the answer
        pos = (tokens[b, :-1] == tokens[b, -1]).nonzero().flatten()
        assert len(pos) == 2 and tokens[b, pos[-1] + 1] == answers[b] and tokens[b, pos[0] + 1] >= mqar.STALE[0]
    res = {m: mqar.evaluate(m, 128, 6, dim=64, heads=2, batch=8, device="cpu", reps=1, warmup=0) for m in mqar.MIXERS}
    assert all(r["recall"] == 1.0 for r in res.values()), res
    assert res["gated_deltanet"]["overwrite_recall"] == 1.0
    assert res["gla"]["overwrite_recall"] <= 1.0 and res["softmax"]["overwrite_recall"] < 1.0
    with pytest.raises(ValueError):
        mqar.make_task(1, 16, 12)


def test_failure_detector_and_status_word():
    """Heartbeat bookkeeping against a fake store and a fake clock: a rank is overdue only after its counter stood
    still for longer than the timeout; a moving counter resets it; a never-seen rank counts from construction.
    A non-zero status word of a fused kernel becomes CollectiveTimeout on the host."""
    from triune_b200.parallel.elastic import CollectiveTimeout, FailureDetector, RankFailure, raise_on_status

    class Store(dict):
        def check(self, keys):
            return all(k in self for k in keys)

        def get(self, k):
            return str(self[k]).encode()

    now = [0.0]
    st = Store({"hb/1": 1, "hb/2": 1})
    det = FailureDetector(st, [1, 2, 3], timeout=2.0, clock=lambda: now[0])
    assert det.poll() == []
    now[0] = 1.5
    st["hb/1"] = 2                        # rank 1 keeps beating, rank 2 stands still, rank 3 never appeared
    assert det.poll() == []               # nobody has been silent for more than 2 s yet
    now[0] = 2.5
    assert det.poll() == [2, 3]           # rank 2 last moved at t=0, rank 3 never did; rank 1 moved at t=1.5
    now[0] = 3.6
    assert det.poll() == [1, 2, 3]        # now rank 1 is overdue too ...
    st["hb/1"] = 3
    assert det.poll() == [2, 3]           # ... until its next beat
    st["hb/2"] = 2                        # a late beat revives it
    assert det.poll() == [3]
    det.forget([3])
    assert det.poll() == []
    raise_on_status(0)
    with pytest.raises(CollectiveTimeout) as e:
        raise_on_status(0x30002, "test kernel")
    assert e.value.status == 0x30002 and "test kernel" in str(e.value)
    assert RankFailure([2, 1]).dead == [1, 2]


def test_dag_component_nodes(tmp_path):
    """The component node library: a training graph (model -> optimizer -> batch -> step -> perplexity -> checkpoint
    -> reload), operator nodes on random tensors, inspectors, a nested subgraph; every node type has typed ports."""
    import torch

    from triune_b200.execution.dag import NODE_TYPES, execute_dag

    assert len(NODE_TYPES) >= 45
    tiny = dict(vocab_size=64, hidden_dim=32, num_layers=5, num_heads=2, head_dim=16, num_experts=2, reflex_exit_layer=2,
                limbic_exit_layer=3, router_prefix_layers=1)
    ck = str(tmp_path / "g.pt")
    train = {"nodes": [
        {"id": "m", "type": "load_model", "params": {"model": "triune-nano", "overrides": tiny}},
        {"id": "opt", "type": "adamw_optimizer", "params": {"lr": 1e-2}},
        {"id": "data", "type": "synthetic_tokens", "params": {"vocab_size": 64, "batch_size": 2, "seq_len": 16}},
        {"id": "b", "type": "next_batch"}, {"id": "insp", "type": "token_batch_inspector"},
        {"id": "step", "type": "training_step"}, {"id": "ppl", "type": "perplexity"},
        {"id": "joint", "type": "joint_exit_loss"}, {"id": "acc", "type": "gradient_accumulator", "params": {"micro_batches": 2}},
        {"id": "save", "type": "checkpoint_save", "params": {"path": ck, "step": 1}},
    ], "edges": [
        {"from": "m.model", "to": "opt.model"}, {"from": "data.loader", "to": "b.loader"}, {"from": "b.input_ids", "to": "insp.input_ids"},
        {"from": "opt.model", "to": "step.model"}, {"from": "opt.optimizer", "to": "step.optimizer"},
        {"from": "b.input_ids", "to": "step.input_ids"}, {"from": "b.labels", "to": "step.labels"},
        {"from": "step.model", "to": "ppl.model"}, {"from": "b.input_ids", "to": "ppl.input_ids"}, {"from": "b.labels", "to": "ppl.labels"},
        {"from": "step.model", "to": "joint.model"}, {"from": "b.input_ids", "to": "joint.input_ids"}, {"from": "b.labels", "to": "joint.labels"},
        {"from": "step.model", "to": "acc.model"}, {"from": "data.loader", "to": "acc.loader"},
        {"from": "acc.model", "to": "save.model"},
    ]}
    out = execute_dag(train)["outputs"]
    assert out["insp.out"]["shape"] == [2, 16] and out["step.loss"] > 0 and out["ppl.out"]["ppl"] > 1
    assert len(out["joint.parts"]) == 3 and out["acc.loss"] > 0 and os.path.isfile(ck)
    re = execute_dag({"nodes": [{"id": "l", "type": "checkpoint_load", "params": {"path": ck}}, {"id": "i", "type": "model_info"}],
                      "edges": [{"from": "l.model", "to": "i.model"}]})["outputs"]
    assert re["i.out"]["layers"] == 5

    def rnd(i, shape, scale=1.0):
        return {"id": i, "type": "random_tensor", "params": {"shape": shape, "seed": len(i), "scale": scale}}

    ops_graph = {"nodes": [rnd("q", [1, 32, 2, 16]), rnd("kk", [1, 32, 2, 16]), rnd("vvv", [1, 32, 2, 16]), rnd("gggg", [1, 32, 2, 16]),
                           {"id": "gla", "type": "gla"}, {"id": "gdn", "type": "gated_deltanet"}, {"id": "rope", "type": "rope"},
                           {"id": "norm", "type": "rmsnorm"}, {"id": "see", "type": "tensor_inspector"},
                           rnd("lg", [8, 6]), {"id": "route", "type": "moe_route", "params": {"top_k": 2}},
                           {"id": "z", "type": "router_z_loss"}, rnd("w", [32, 64], 0.1), {"id": "fp4", "type": "nvfp4_roundtrip"},
                           {"id": "lr", "type": "cosine_lr", "params": {"step": 10, "total_steps": 100, "warmup_steps": 10, "lr": 1.0}},
                           {"id": "hw", "type": "resource_manager"}, {"id": "vram", "type": "vram_profiler"}],
                 "edges": [{"from": "q.x", "to": "rope.x"}, {"from": "rope.y", "to": "gla.q"}, {"from": "kk.x", "to": "gla.k"},
                           {"from": "vvv.x", "to": "gla.v"}, {"from": "gggg.x", "to": "gla.g"},
                           {"from": "q.x", "to": "gdn.q"}, {"from": "kk.x", "to": "gdn.k"}, {"from": "vvv.x", "to": "gdn.v"},
                           {"from": "gggg.x", "to": "gdn.g"}, {"from": "gla.out", "to": "norm.x"}, {"from": "norm.y", "to": "see.x"},
                           {"from": "lg.x", "to": "route.logits"}, {"from": "lg.x", "to": "z.logits"}, {"from": "w.x", "to": "fp4.w"}]}
    o = execute_dag(ops_graph)["outputs"]
    assert o["see.out"]["shape"] == [1, 32, 2, 16] and o["see.out"]["finite"] and abs(o["see.out"]["std"] - 1.0) < 0.2
    assert list(o["gdn.state"].shape) == [1, 2, 16, 16] and list(o["route.indices"].shape) == [8, 2]
    assert float(o["z.loss"]) > 0 and 0 < o["fp4.error"] < 0.2 and o["lr.lr"] == pytest.approx(1.0)
    assert "available" in o["vram.out"] and isinstance(o["hw.out"], dict)

    inner = {"nodes": [{"id": "input", "type": "constant"}, {"id": "py", "type": "python", "params": {"code": "result = value * 2"}}],
             "edges": [{"from": "input.out", "to": "py.value"}]}
    sub = execute_dag({"nodes": [{"id": "c", "type": "constant", "params": {"value": 21}},
                                 {"id": "s", "type": "subgraph", "params": {"dag": inner, "output": "py.out"}}],
                       "edges": [{"from": "c.out", "to": "s.value"}]})["outputs"]
    assert sub["s.out"] == 42
    for t in NODE_TYPES.values():
        if "." in t.name:  # nodes that plugins of other tests registered
            continue
        assert all(isinstance(v, str) for v in list(t.inputs.values()) + list(t.outputs.values())) and t.description


def test_plugin_scaffold_sign_load_and_tamper(tmp_path):
    """A scaffolded plugin loads under its signing key and its node runs in a graph; an edited entry file is refused
    until the manifest is re-signed; a wrong key is refused; the CLI drives the same functions."""
    from triune_b200.cli import main as cli
    from triune_b200.execution.dag import execute_dag
    from triune_b200.plugins.registry import PluginError, PluginRegistry, create_plugin, write_manifest

    d = create_plugin(tmp_path, "scaf", key="secret")
    reg = PluginRegistry("secret")
    assert [p.name for p in reg.discover(tmp_path)] == ["scaf"]
    info = reg.load("scaf")
    assert info.loaded and info.nodes == ["scaf.echo"]
    out = execute_dag({"nodes": [{"id": "c", "type": "constant", "params": {"value": 7}}, {"id": "e", "type": "scaf.echo"}],
                       "edges": [{"from": "c.out", "to": "e.value"}]})["outputs"]
    assert out["e.out"] == 7
    with pytest.raises(PluginError):
        create_plugin(tmp_path, "scaf")
    with pytest.raises(PluginError):
        create_plugin(tmp_path, "../evil")
    (d / "plugin.py").write_text((d / "plugin.py").read_text() + "\n# changed\n")
    fresh = PluginRegistry("secret")
    fresh.discover(tmp_path)
    with pytest.raises(PluginError):
        fresh.verify(fresh.plugins["scaf"])
    write_manifest(d, "secret")
    again = PluginRegistry("secret")
    again.discover(tmp_path)
    again.verify(again.plugins["scaf"])
    other = PluginRegistry("other-key")
    other.discover(tmp_path)
    with pytest.raises(PluginError):
        other.verify(other.plugins["scaf"])
    assert cli(["plugin", "verify", "--dir", str(tmp_path), "--key", "secret"]) == 0
    assert cli(["plugin", "verify", "--dir", str(tmp_path), "--key", "nope"]) == 1


def test_agent_memory_skills_and_providers(tmp_path):
    """Lessons are recalled by similarity and survive a reload; skills are parsed from markdown headers and picked by
    triggers; provider records hide their keys and refuse to send without an injected transport."""
    from triune_b200.agents import AgentMemoryStore, ProviderManager, SkillLibrary

    path = tmp_path / "mem" / "store.json"
    mem = AgentMemoryStore(str(path))
    mem.add_lesson("when the loss is NaN lower the learning rate and check the gate clamp", ["training"])
    mem.add_lesson("prefill is faster with larger chunks on long prompts", ["serving"])
    mem.add_lesson("tokenizer files must be saved next to the checkpoint")
    mem.set_preference("tone", "brief")
    assert mem.record_tool("http_get", ok=False) == {"calls": 1, "failures": 1}
    top = mem.recall("my training loss became nan, what about the learning rate?", k=2)
    assert top and "NaN" in top[0][1] and (len(top) == 1 or top[0][0] >= top[1][0])
    assert mem.recall("completely unrelated zebra question") == []
    again = AgentMemoryStore(str(path))
    assert again.data["preferences"] == {"tone": "brief"} and len(again.data["lessons"]) == 3

    (tmp_path / "skills").mkdir()
    (tmp_path / "skills" / "ckpt.md").write_text("---\nname: checkpoint-care\ndescription: saving and resuming runs\n"
                                                 "triggers: resume, save checkpoint\n---\nAlways save the tokenizer too.\n")
    (tmp_path / "skills" / "plain.md").write_text("Write short answers.\n")
    lib = SkillLibrary(str(tmp_path / "skills"))
    assert set(lib.skills) == {"checkpoint-care", "plain"}
    assert [s.name for s in lib.select("how do I resume my run?")] == ["checkpoint-care"]
    assert "Always save the tokenizer" in lib.prompt_block("please save checkpoint now")
    assert lib.select("zebra") == []

    pm = ProviderManager()
    pm.save("Example", "https://api.example.com/v1/", "m-1", "sk-abcdef123456")
    assert pm.describe()[0]["key_hint"] == "...3456" and "abcdef" not in json.dumps(pm.describe())
    with pytest.raises(ValueError):
        pm.save("bad", "http://evil.example.com", "m", "k")
    with pytest.raises(RuntimeError):
        pm.chat("example", [{"role": "user", "content": "hi"}])
    pm.transport = lambda p, msgs, opt: f"{p.model}:{msgs[-1]['content']}"
    assert pm.chat("example", [{"role": "user", "content": "hi"}]) == "m-1:hi"


def test_convergence_evaluation_all_optimizers_learn():
    """The synthetic Markov language has a known entropy floor; 30 steps of each optimizer move a small dense model
    from the uniform loss towards it, and the report carries the curve, the floor and the step time."""
    import math

    from triune_b200.evals import convergence as cv

    succ, probs, floor = cv.markov_language(64, branching=4, seed=1)
    assert succ.shape == (64, 4) and torch.allclose(probs.sum(-1), torch.ones(64)) and 0 < floor < math.log(4) + 1e-6
    x = cv.sample_batch(succ, probs, 4, 16, torch.Generator().manual_seed(0))
    assert x.shape == (4, 17) and all(int(x[b, t + 1]) in succ[int(x[b, t])].tolist() for b in range(4) for t in range(16))
    for opt in cv.OPTIMIZERS:
        r = cv.run(opt, "dense", steps=30, vocab=64, width=32, layers=2, batch=8, seq_len=32, lr=3e-3, device="cpu")
        assert abs(r["loss_start"] - math.log(64)) < 0.5 and r["loss_end"] < r["loss_start"] - 0.5, r
        assert r["loss_end"] > r["entropy_floor"] - 0.05 and r["ms_per_step"] > 0 and r["optimizer_state_bytes"] > 0


def test_merge_shards_rejects_incomplete_and_mixed_sets(tmp_path):
    """The merge tool refuses a directory with a missing rank, shard sets of two sizes, and slices that do not cover a
    parameter exactly once."""
    import pytest

    from triune_b200.trainer.checkpoint import _atomic_save
    from triune_b200.trainer.sharded_checkpoint import FORMAT, merge_shards, shard_path

    def shard(rank, world, pieces, replicated=None):
        _atomic_save({"format": FORMAT, "rank": rank, "world": world, "step": 1, "loss": 0.0, "pieces": pieces,
                      "replicated": replicated or {}, "optimizer_state": None, "config": {}, "architecture": None},
                     shard_path(str(tmp_path), rank, world))

    w = torch.arange(24.0).view(6, 4)
    shard(0, 2, [("w", 0, 0, 3, 6, w[:3].clone())], {"b": torch.ones(2)})
    with pytest.raises(ValueError, match="expected shards"):
        merge_shards(str(tmp_path))
    shard(1, 2, [("w", 0, 3, 6, 6, w[3:].clone())])
    merged = merge_shards(str(tmp_path), str(tmp_path / "m.pt"))
    assert torch.equal(merged["model_state"]["w"], w) and torch.equal(merged["model_state"]["b"], torch.ones(2))
    assert merged["merged_from"]["shards"] == 2 and (tmp_path / "m.pt").exists()
    shard(1, 2, [("w", 0, 3, 5, 6, w[3:5].clone())])  # one row never written
    with pytest.raises(ValueError, match="incomplete or overlapping"):
        merge_shards(str(tmp_path))
    shard(0, 3, [])
    with pytest.raises(ValueError, match="different sizes"):
        merge_shards(str(tmp_path))
    with pytest.raises(FileNotFoundError):
        merge_shards(str(tmp_path / "nothing"))


def test_expert_parallel_reduction_runs_follow_the_received_counts():
    """The run list of the bounded weight-gradient reductions: one run per (local expert, source rank) segment of the
    expert-major buffer, as many 64-row blocks as hold rows, counts above the capacity clamped."""
    from types import SimpleNamespace

    from triune_b200.parallel.expert_parallel import EPContext

    W, El, cap = 3, 2, 256
    cnt_all = torch.tensor([[0, 65], [64, 300], [1, 128]], dtype=torch.int32).reshape(-1)  # [source rank, local expert]
    runs, offs = EPContext.reduction_runs(SimpleNamespace(experts_per_rank=El, world=W), cnt_all, cap)
    assert runs.dtype == torch.int32 and offs.dtype == torch.int32
    assert offs.tolist() == [0, 3, 6]
    # segment order is expert-major: (e0, r0), (e0, r1), (e0, r2), (e1, r0), ...
    assert runs[:, 0].tolist() == [0, 256, 512, 768, 1024, 1280]
    assert runs[:, 1].tolist() == [0, 1, 1, 2, 4, 2]


def test_installer_plan_run_and_scripts(tmp_path):
    """The installer on fake machines: what it detects, the plan it makes (kernels only where they can be built, wheel
    directory and offline flags, existing environment reused), how a run stops or carries on, and what it writes."""
    from triune_b200 import installer as ins

    def machine(smi=None, nvcc=True):
        def run(argv, cwd=None, timeout=0):
            if argv[0] == "nvidia-smi":
                return (0, smi) if smi else (127, "not found")
            if argv[0] == "nvcc":
                return (0, "nvcc: NVIDIA (R) Cuda compiler driver\nCuda compilation tools, release 12.9, V12.9.86\n") if nvcc else (127, "")
            raise AssertionError(argv)
        return run

    b200 = ins.probe_machine(machine("NVIDIA B200, 183359, 580.159, 10.0\nNVIDIA B200, 183359, 580.159, 10.0\n"), os_type="Linux", proc_version="Linux version 6.1")
    assert len(b200.gpus) == 2 and b200.gpus[0]["memory_gb"] == 179.1 and b200.driver == "580.159" and b200.nvcc == "12.9"
    assert b200.blackwell and b200.can_build_kernels and not b200.is_wsl and not b200.notes
    h100 = ins.probe_machine(machine("NVIDIA H100, 81559, 550.54, 9.0\n"), os_type="Linux", proc_version="Linux ... microsoft-standard-WSL2")
    assert h100.is_wsl and not h100.blackwell and not h100.can_build_kernels and "10.x" in h100.notes[0]
    cpu = ins.probe_machine(machine(None, nvcc=False), os_type="Darwin")
    assert not cpu.gpus and "no NVIDIA GPU" in cpu.notes[0]
    no_nvcc = ins.probe_machine(machine("NVIDIA B200, 183359, 580.159, 10.0\n", nvcc=False), os_type="Linux", proc_version="")
    assert no_nvcc.blackwell and not no_nvcc.can_build_kernels and "nvcc was not found" in no_nvcc.notes[0]

    venv = tmp_path / "env"
    names = lambda steps: [s.name for s in steps]
    plan = ins.plan_install(b200, venv, base_python="/usr/bin/python3")
    assert names(plan) == ["create-venv", "install-torch", "install-core", "install-serve", "install-extras", "build-kernels", "launcher", "verify"]
    assert plan[0].argv == ["/usr/bin/python3", "-m", "venv", str(venv)] and plan[1].argv[0] == str(venv / "bin" / "python")
    assert "--index-url" in plan[1].argv and plan[5].argv[-2:] == ["triune_b200", "native"] and plan[6].argv[-1] == "linux"
    assert [s.optional for s in plan] == [False, False, False, True, True, False, True, False]
    assert "build-kernels" not in names(ins.plan_install(h100, venv)) and "build-kernels" not in names(ins.plan_install(b200, venv, build=False))
    off = ins.plan_install(b200, venv, find_links="/wheels", offline=True, extras=False, shortcuts=False)
    assert names(off) == ["create-venv", "install-torch", "install-core", "install-serve", "build-kernels", "verify"]
    assert off[1].argv[-4:] == ["--no-index", "--find-links", "/wheels", "torch"] and "--index-url" not in off[1].argv
    bare = ins.plan_install(cpu, None, offline=True, shortcuts=True)
    assert names(bare) == ["check-torch", "launcher", "verify"] and bare[1].argv[-1] == "macos"
    (venv / "bin").mkdir(parents=True)
    (venv / "bin" / "python").write_text("")
    assert names(ins.plan_install(b200, venv))[0] == "check-venv"
    win = ins.plan_install(ins.MachineProfile(os_type="Windows", python=(3, 12)), tmp_path / "w")
    assert win[1].argv[0].endswith("Scripts/python.exe") and win[-2].argv[-1] == "windows"

    calls, lines = [], []

    def runner(fail):
        def run(argv, cwd=None, timeout=0):
            calls.append(argv)
            step = next(s.name for s in plan if s.argv == argv)
            return (1, "boom\nlast line") if step in fail else (0, "fine")
        return run

    plan = ins.plan_install(b200, tmp_path / "e2", base_python="py")
    rec = ins.run_plan(plan, runner({"install-extras", "launcher"}), lines.append)
    assert rec["ok"] and [r["status"] for r in rec["steps"]] == ["done", "done", "done", "done", "skipped", "done", "skipped", "done"]
    assert any("warning: exit code 1" in l and "last line" in l for l in lines)
    calls.clear()
    rec = ins.run_plan(plan, runner({"install-core"}), lines.append)
    assert not rec["ok"] and rec["steps"][-1] == {"step": "install-core", "status": "failed", "exit_code": 1, "output": "boom\nlast line"}
    assert len(calls) == 3  # nothing ran after the failing required step
    calls.clear()
    rec = ins.run_plan(plan, runner(set()), lines.append, dry_run=True)
    assert rec["ok"] and not calls and all(r["status"] == "planned" for r in rec["steps"])

    s = ins.write_bootstrap_scripts(tmp_path / "dist")
    sh, bat = open(s["sh"]).read(), open(s["bat"], newline="").read()
    assert sh.startswith("#!/usr/bin/env sh") and "-m triune_b200 install --venv" in sh and os.access(s["sh"], os.X_OK)
    assert "wsl.exe --status" in bat and "\r\n" in bat and "-m triune_b200 install" in bat
    real = tmp_path / "venv_real"
    real.mkdir()
    (real / "pyvenv.cfg").write_text("home = /usr/bin\n")
    plain = tmp_path / "not_a_venv"
    plain.mkdir()
    assert ins.uninstall(str(plain), str(tmp_path / "dist"), dry_run=True)["kept"] and plain.exists()
    out = ins.uninstall(str(real), str(tmp_path / "dist"))
    assert not real.exists() and not os.path.exists(s["sh"]) and len(out["removed"]) == 3


def test_desktop_wsl_discovery_and_launch(monkeypatch):
    """The launcher's WSL path: path translation, choice of the interpreter inside WSL (one that sees a GPU wins; one
    that cannot import the package is skipped), the command line, and a session started through it on a fake Windows."""
    from triune_b200 import desktop as d

    assert d.to_wsl_path("C:\\Users\\me\\repo") == "/mnt/c/Users/me/repo"
    assert d.to_wsl_path("\\\\wsl$\\Ubuntu\\home\\me\\repo") == "/home/me/repo"
    assert d.to_wsl_path("\\\\wsl.localhost\\Ubuntu-24.04\\srv") == "/srv" and d.to_wsl_path("/opt/x") == "/opt/x"

    info = {"/home/me/venvs/triune/bin/python": {"torch": "2.11", "cuda": False, "package": True},
            "/home/me/.venv/bin/python": {"torch": None, "cuda": False, "package": True},
            "/mnt/c/w/.venv/bin/python": {"torch": "2.11", "cuda": True, "package": False},
            "/usr/bin/python3": {"torch": "2.11", "cuda": True, "package": True}}
    seen = []

    def run(argv, timeout=0):
        seen.append(list(argv))
        if argv[:2] == ["wsl.exe", "--status"]:
            return 0, ""
        if argv[:3] == ["wsl.exe", "-e", "sh"]:
            return (0, "/home/me") if "HOME" in argv[-1] else (0, "/usr/bin/python3\n")
        if argv[:3] == ["wsl.exe", "-e", "test"]:
            return (0 if argv[-1] in info else 1), ""
        if argv[:2] == ["wsl.exe", "-e"] and argv[2] in info:
            return 0, "warning line\n" + json.dumps(info[argv[2]]) + "\n"
        return 1, ""

    monkeypatch.delenv("TRIUNE_WSL_PYTHON", raising=False)
    got = d.find_wsl_python("C:\\w", run=run)
    assert got == {"python": "/usr/bin/python3", "cuda": True, "torch": "2.11", "workspace": "/mnt/c/w"}
    assert all(c[-1] == "/mnt/c/w" for c in seen if len(c) > 3 and c[2] in info)  # every probe was told where the package lives
    info["/usr/bin/python3"]["cuda"] = False
    assert d.find_wsl_python("C:\\w", run=run)["python"] == "/home/me/venvs/triune/bin/python"  # first usable one without a GPU
    assert d.find_wsl_python("C:\\w", run=lambda a, t=0: (1, "")) is None  # no WSL
    cmd = d.wsl_server_command(got, 8123, model="triune-nano", precision="fp8")
    assert cmd == ["wsl.exe", "--cd", "/mnt/c/w", "-e", "/usr/bin/python3", "-m", "triune_b200", "serve", "--host", "127.0.0.1", "--port", "8123",
                   "--model", "triune-nano", "--precision", "fp8"]

    started = []

    class FakeProc:
        def poll(self):
            return None

        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0

        def kill(self):
            pass

    monkeypatch.setattr(d, "port_in_use", lambda port, host="127.0.0.1": False)
    monkeypatch.setattr(d, "wait_for_server", lambda *a, **k: True)
    monkeypatch.setattr(d, "_local_cuda", lambda: False)
    info["/usr/bin/python3"]["cuda"] = True
    ses = d.start_session(8123, quiet=True, allow_wsl=True, run=run, popen=lambda cmd, **kw: started.append(cmd) or FakeProc(), platform="win32")
    assert started[0][0] == "wsl.exe" and started[0][started[0].index("-e") + 1] == "/usr/bin/python3" and not ses.reused
    started.clear()
    d.start_session(8123, quiet=True, allow_wsl=True, run=run, popen=lambda cmd, **kw: started.append(cmd) or FakeProc(), platform="linux")
    assert started[0][0] == sys.executable  # WSL is only considered on a Windows host


def test_calm_calibration_pieces():
    """Statistics of the confidence-exit calibration on constructed data: Wilson bound, AUROC with ties, calibration
    error, the threshold choice, and the whole evaluation on a tiny model."""
    from triune_b200.evals import calm

    assert calm.wilson_lower(0, 0) == 0.0 and 0.83 < calm.wilson_lower(95, 100) < 0.95 and calm.wilson_lower(100, 100) < 1.0
    s = torch.tensor([0.1, 0.2, 0.3, 0.4, 0.5, 0.6])
    assert calm.auroc(s, torch.tensor([0, 0, 0, 1, 1, 1], dtype=torch.bool)) == 1.0
    assert calm.auroc(s, torch.tensor([1, 1, 1, 0, 0, 0], dtype=torch.bool)) == 0.0
    assert calm.auroc(torch.tensor([0.5, 0.5, 0.5, 0.5]), torch.tensor([1, 0, 1, 0], dtype=torch.bool)) == 0.5  # all tied
    assert calm.auroc(s, torch.ones(6, dtype=torch.bool)) is None
    conf = torch.cat([torch.full((100,), 0.95), torch.full((100,), 0.15)])
    agree = torch.cat([torch.ones(95), torch.zeros(5), torch.ones(15), torch.zeros(85)]).bool()
    assert calm.reliability(conf, agree)["ece"] < 1e-6  # confidence equals the observed agreement in both bins
    assert calm.reliability(conf, ~agree)["ece"] > 0.7
    # margins above 0.4 always agree, below they agree half of the time: the smallest qualifying threshold is 0.4
    g = torch.Generator().manual_seed(0)
    margin = torch.rand(4000, generator=g)
    ok = (margin >= 0.4) | (torch.rand(4000, generator=g) < 0.5)
    assert calm.calibrate(margin, ok, 0.99) == 0.4
    assert calm.calibrate(margin, ok, 0.99, min_positions=10**6) is None
    rows = calm.curve(margin, ok)
    assert rows[0]["coverage"] > rows[-1]["coverage"] and rows[-1]["agreement"] == 1.0

    torch.manual_seed(0)
    model = TriuneTransformer.from_config(ModelConfig(vocab_size=64, hidden_dim=32, num_layers=5, num_heads=1, head_dim=32, num_experts=2,
                                                      router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3))
    cal = calm.synthetic_batches(64, 2, 4, 24, seed=1)
    held = calm.synthetic_batches(64, 2, 4, 24, seed=2)
    assert not torch.equal(cal[0], held[0]) and cal[0].shape == (4, 25)
    res = calm.evaluate(model, calm.collect(model, cal), calm.collect(model, held), (0.5,), min_positions=1)
    assert res["positions"] == {"calibration": 192, "held_out": 192} and set(res["exits"]) == {"reflex", "limbic"}
    assert 0.0 <= res["exits"]["reflex"]["agreement_all_positions"] <= 1.0
    assert calm.layers_saved(model, 1.0, 0.0) == 0.4 and calm.layers_saved(model, 0.0, 1.0) == 0.2
    lat = calm.policy_latency(model, held[0][:, :-1], 0.3, iters=1)
    assert lat["full_depth_ms"] > 0 and lat["where_tokens_left"]["total_tokens"] == 96


def test_qr_residuals_and_dynamic_exit_evals():
    from triune_b200.evals import dynamic_exits, qr_residuals

    rows = qr_residuals.sweep(K=6, d=96, r=8, conds=(1e1, 1e3, 1e6))
    assert rows[0]["fast_path"] == 6 and rows[0]["fast_path_max"]["orthogonality"] < 1e-5 and rows[0]["fast_path_max"]["projector_distance"] < 1e-4
    assert rows[1]["all_max"]["reconstruction"] < 1e-5
    assert rows[2]["fallbacks"] == 6 and rows[2]["all_max"]["orthogonality"] < 1e-5  # ill-conditioned slices go to Householder QR
    deg = qr_residuals.degenerate_cases()
    assert deg["caught"] == [True, True, True] and deg["finite"]
    A = qr_residuals.conditioned(2, 40, 5, 100.0, torch.Generator().manual_seed(0))
    sv = torch.linalg.svdvals(A)
    assert torch.allclose(sv[:, 0] / sv[:, -1], torch.full((2,), 100.0, dtype=torch.float64), rtol=1e-6)

    torch.manual_seed(0)
    model = TriuneTransformer.from_config(ModelConfig(vocab_size=64, hidden_dim=32, num_layers=5, num_heads=1, head_dim=32, num_experts=2,
                                                      router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3))
    res = dynamic_exits.measure(model, torch.randint(0, 64, (3, 16)), iters=1, calm_tau=0.5)
    assert set(res["exits"]) == {"reflex", "limbic", "cortex"} and sum(res["router"]["sequences_per_depth"]) == 3
    assert res["calm"]["where_tokens_left"]["total_tokens"] == 48


def test_local_ollama_probe_and_chat_stream():
    """A stand-in daemon on the loopback address: tag listing, streamed chat pieces, a daemon-side error; nothing else is contacted."""
    import threading
    from http.server import BaseHTTPRequestHandler, HTTPServer

    from triune_b200.runtime import model_scanner as ms

    seen = {}

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_GET(self):
            body = json.dumps({"models": [{"name": "gemma3:4b"}, {"name": "qwen3:8b"}, {"nope": 1}]}).encode() if self.path == "/api/tags" else b"{}"
            self.send_response(200)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_POST(self):
            req = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            seen["req"] = req
            lines = ([{"error": "model not found"}] if req["model"] == "missing" else
                     [{"message": {"content": "Hel"}}, {"message": {"content": "lo"}}, {"message": {"content": ""}, "done": True}, {"message": {"content": "late"}}])
            body = "".join(json.dumps(l) + "\n" for l in lines).encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

    srv = HTTPServer(("127.0.0.1", 0), H)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    url = f"http://127.0.0.1:{srv.server_port}"
    try:
        assert ms.query_ollama_running_tags(url, timeout=2.0) == ["gemma3:4b", "qwen3:8b"]
        msgs = [{"role": "user", "content": "hi"}]
        assert "".join(ms.stream_ollama_chat("gemma3:4b", msgs, url, options={"temperature": 0}, timeout=5.0)) == "Hello"
        assert seen["req"]["stream"] is True and seen["req"]["messages"] == msgs and seen["req"]["options"] == {"temperature": 0}
        with pytest.raises(RuntimeError, match="model not found"):
            list(ms.stream_ollama_chat("missing", msgs, url, timeout=5.0))
    finally:
        srv.shutdown()
    assert ms.query_ollama_running_tags(url, timeout=0.3) == []  # the daemon is gone
    assert ms.query_ollama_running_tags("http://example.com:11434") == []  # never leaves the machine
    with pytest.raises(ValueError):
        list(ms.stream_ollama_chat("m", [], "http://example.com:11434"))
    with pytest.raises(ConnectionError):
        list(ms.stream_ollama_chat("m", [], url, timeout=0.5))


def test_cli_reference_command_names_doctor_and_agent(tmp_path, capsys):
    """The command names of the reference's CLI resolve here (aliases), `doctor` reports a healthy CPU installation,
    and `agent` runs a goal through one persona and through a team, keeping a lesson for the next run."""
    from triune_b200 import cli

    p = cli.build_parser()
    for argv in (["studio", "--no-browser"], ["benchmark"], ["build-native", "--target", "linux"], ["info"], ["cache-nvfp4", "--help"]):
        if "--help" in argv:
            with pytest.raises(SystemExit):
                p.parse_args(argv)
            capsys.readouterr()
            continue
        assert callable(p.parse_args(argv).fn), argv
    assert p.parse_args(["studio"]).fn is cli.cmd_desktop and p.parse_args(["info"]).fn is cli.cmd_doctor
    assert cli.main(["doctor"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["status"] == "healthy" and rep["tiny_forward"] and rep["studio_page"] and rep["model_zoo"]["presets"] >= 10
    store = tmp_path / "agent"
    base = ["agent", "--device", "cpu", "--model", "triune-nano", "--max-tokens", "4", "--store-dir", str(store)]
    assert cli.main(base + ["list the files", "--workspace", str(tmp_path)]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["persona"] == "engineer" and isinstance(out["text"], str) and "read_file" in out["tools_offered"]  # "list the files": engineer by keyword
    assert cli.main(base + ["--team", "architect,engineer", "--goal", "list the files", "--read-only", "--workspace", str(tmp_path)]) == 0
    out = json.loads(capsys.readouterr().out)
    assert [o["agent"] for o in out] == ["architect", "engineer"]
    mem = json.loads((store / "memory.json").read_text())
    assert len(mem["lessons"]) == 2
    assert cli.main(["agent", "--device", "cpu"]) == 2  # no goal


def test_agent_harness_personas_tools_memory_and_skills(tmp_path):
    """The harness with a scripted generator: persona choice, workspace confinement, read-only and shell switches, the
    public-URL guard, tool statistics, lessons recalled by a later run, and a skill written from a successful run."""
    from triune_b200.agents.harness import AgentHarness, choose_persona, resolve_persona, workspace_tools

    assert choose_persona("why does the kernel hang with a traceback").name == "debugger"
    assert choose_persona("make the decode loop faster, profile the latency").name == "optimizer"
    assert choose_persona("hello").name == "assistant"
    assert resolve_persona("sentinel").name == "sentinel" and resolve_persona("auto", "design the module layout").name == "architect"
    custom = resolve_persona("poet=Answer in verse.")
    assert custom.name == "poet" and custom.system_prompt == "Answer in verse."
    assert resolve_persona("navigator").system_prompt.startswith("You are the navigator")

    ws = tmp_path / "ws"
    (ws / "src").mkdir(parents=True)
    (ws / "src" / "a.py").write_text("def f():\n    return 41  # TODO fix\n")
    (tmp_path / "secret.txt").write_text("outside")
    tools = workspace_tools(str(ws), fetch=lambda url: "fetched " + url)
    assert tools.call("list_dir", path=".") == ["src/"] and tools.call("read_file", path="src/a.py").startswith("def f")
    assert tools.call("search", pattern="TODO")[0] == {"file": "src/a.py", "line": 2, "text": "    return 41  # TODO fix"}
    for bad in ("../secret.txt", "/etc/passwd", "src/../../secret.txt"):
        with pytest.raises(PermissionError):
            tools.call("read_file", path=bad)
    with pytest.raises(PermissionError):
        tools.call("write_file", path="../evil.txt", content="x")
    assert "edited" in tools.call("edit_file", path="src/a.py", old="41", new="42") and "42" in (ws / "src" / "a.py").read_text()
    with pytest.raises(ValueError):
        tools.call("edit_file", path="src/a.py", old="zzz", new="y")
    with pytest.raises(PermissionError):
        tools.call("http_get", url="http://127.0.0.1:8000/v1/models")
    with pytest.raises(PermissionError):
        tools.call("http_get", url="http://169.254.169.254/latest/meta-data")
    assert tools.call("http_get", url="https://8.8.8.8/x") == "fetched https://8.8.8.8/x"
    ro = workspace_tools(str(ws), read_only=True, allow_shell=True)
    assert "write_file" not in ro.tools and "shell" not in ro.tools and "read_file" in ro.tools
    sh = workspace_tools(str(ws), allow_shell=True)
    assert sh.call("shell", command="ls src")["stdout"].strip() == "a.py"

    script = ['I will look. <|tool_call|> {"tool": "search", "args": {"pattern": "TODO"}}', "The TODO is in src/a.py line 2."]
    prompts = []

    def generate(prompt):
        prompts.append(prompt)
        return script[min(len(prompts) - 1, len(script) - 1)] if len(prompts) <= 2 else "done"

    h = AgentHarness(generate, str(tmp_path / "store"), workspace=str(ws))
    out = h.run("debug the TODO bug: find where it fails")
    assert out["persona"] == "debugger" and out["text"] == "The TODO is in src/a.py line 2."
    assert out["tool_calls"][0]["result"][0]["file"] == "src/a.py" and "<|tool_return|>" in prompts[1]
    assert out["new_skill"] and (tmp_path / "store" / "skills" / f"{out['new_skill']}.md").is_file()
    assert h.memory.data["tool_stats"]["search"] == {"calls": 1, "failures": 0}
    # a second harness on the same store starts from the lesson and the skill of the first run
    prompts.clear()
    h2 = AgentHarness(lambda p: (prompts.append(p), "ok")[1], str(tmp_path / "store"), workspace=str(ws))
    h2.memory.set_preference("style", "terse")
    out2 = h2.run("find the TODO in the code again")
    assert "Notes from earlier runs" in prompts[0] and "## Skill: " in prompts[0] and "style = terse" in prompts[0]
    assert out2["new_skill"] is None  # no tool was used this time
    team = h2.run_team("review the code for risk", ["engineer", "sentinel"])
    assert [t["agent"] for t in team] == ["engineer", "sentinel"] and team[1]["persona"] == "sentinel"


def test_staging_invariants_identity_restoration_and_backward_after_master_mutation():
    """Parameters keep their identity through stage / release, the host master comes back unchanged, gradients flow
    through staged weights, and a backward pass that runs after the layer was released and its host master overwritten
    still differentiates the weights the forward pass used."""
    from triune_b200.runtime.staging import ParameterStager

    class Two(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin1, self.lin2 = nn.Linear(16, 16), nn.Linear(16, 16)

        def forward(self, x):
            return self.lin2(torch.relu(self.lin1(x)))

    torch.manual_seed(42)
    ref_layer, layer = Two(), Two()
    layer.load_state_dict(ref_layer.state_dict())
    ids = [id(p) for p in layer.parameters()]
    before = [p.detach().clone() for p in layer.parameters()]
    st = ParameterStager("cpu")
    st.register_module(layer)
    st.stage_layer(layer)
    assert [id(p) for p in layer.parameters()] == ids
    x_ref = torch.randn(4, 16, requires_grad=True)
    x = x_ref.detach().clone().requires_grad_(True)
    (ref_layer(x_ref) ** 2).sum().backward()
    out = layer(x)
    st.release_layer(layer)
    assert [id(p) for p in layer.parameters()] == ids
    assert all(torch.equal(a, b) for a, b in zip(before, layer.parameters()))
    for b in st.buffers.values():  # something rewrites the host masters between this layer's forward and its backward
        b.cpu_master.add_(torch.randn_like(b.cpu_master) * 10.0)
    st.stage_layer(layer, is_backward=True)  # the backward pass re-stages the weights the forward pass saw
    assert all(torch.equal(a, b) for a, b in zip(before, layer.parameters()))
    (out ** 2).sum().backward()
    st.release_layer(layer, clear_snapshot=True)
    assert [id(p) for p in layer.parameters()] == ids
    assert not any(torch.equal(a, b) for a, b in zip(before, layer.parameters()))  # the masters are the rewritten ones
    assert st.get_memory_summary()["snapshot_bytes"] == 0
    assert torch.allclose(x.grad, x_ref.grad, atol=1e-6)
    for (n, p), (_, q) in zip(layer.named_parameters(), ref_layer.named_parameters()):
        assert p.grad is not None and torch.allclose(p.grad, q.grad, atol=1e-6), n


def test_profile_summaries_carry_their_commands_and_name_existing_files():
    """Every measurement summary says what it ran on, gives at least one full command, and every repository file or
    module a command names exists, so that each figure can be taken again from the committed tree."""
    import re
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    files = sorted((root / "profiles").glob("*.md"))
    assert len(files) >= 10
    for f in files:
        text = f.read_text()
        assert "B200" in text, f.name
        assert "_work/" not in text, f.name
        cmds = [ln.strip() for ln in text.splitlines() if re.match(r"\s*(python|ncu|nvcc)\s", ln)]
        cmds += re.findall(r"`((?:python|ncu|nvcc) [^`]+)`", text)
        assert cmds, f"{f.name}: no command line"
        for c in cmds:
            for script in re.findall(r"(?<![\w/.-])((?:[\w-]+/)*[\w-]+\.py)\b", c):
                assert (root / script).exists(), f"{f.name}: {script}"
            for mod in re.findall(r"-m (triune_b200[\w.]*)", c):
                p = root / mod.replace(".", "/")
                assert p.with_suffix(".py").exists() or (p / "__main__.py").exists() or (p / "__init__.py").exists(), f"{f.name}: {mod}"
        cells = [c.strip().lower() for ln in text.splitlines() if ln.lstrip().startswith("|") for c in ln.split("|")]
        assert not any(c in ("nan", "inf", "-inf") or re.fullmatch(r"-\d[\d.]*( ?[a-zµ/%]+)?", c) for c in cells), f.name


def test_whole_model_streams_from_an_nvfp4_disk_cache(tmp_path):
    """``load_disk_streamed_model`` builds the cache from a Hugging Face directory, creates the model without storage,
    serves each decoder layer from disk for the duration of its forward pass and reproduces the resident model's logits to
    NVFP4 accuracy, with and without the Hadamard rotation; afterwards no layer holds storage."""
    from transformers import LlamaConfig, LlamaForCausalLM

    from triune_b200.runtime.disk_streaming import load_disk_streamed_model, resolve_hf_model_dir

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                      max_position_embeddings=64, tie_word_embeddings=False)
    ref = LlamaForCausalLM(cfg).eval()
    ref.save_pretrained(tmp_path / "hf", safe_serialization=True)
    assert resolve_hf_model_dir(tmp_path / "hf") == tmp_path / "hf"
    with pytest.raises(FileNotFoundError):
        resolve_hf_model_dir("nobody/not-on-this-disk")
    x = torch.randint(0, 128, (2, 10))
    with torch.no_grad():
        want = ref(x).logits
    for had in (False, True):
        model, eng, cache = load_disk_streamed_model(tmp_path / "hf", cache_dir=tmp_path / f"cache{int(had)}", device="cpu", hadamard=had)
        assert (cache / "manifest.json").is_file() and eng.manifest["hadamard"] is had
        with torch.no_grad():
            got = model(x).logits
            again = model(x).logits
        assert F.cosine_similarity(got.flatten().float(), want.flatten(), dim=0) > 0.97 and torch.equal(got, again)
        assert eng.telemetry["layers_loaded"] == 6 and len(eng._resident) == 0
        assert all(p.is_meta for lay in model.model.layers for p in lay.parameters())
        model2, eng2, cache2 = load_disk_streamed_model(cache, device="cpu")  # a cache directory is accepted as it is
        assert cache2 == cache
        eng.close(), eng2.close()


def test_model_scanner_reads_sizes_from_headers(tmp_path):
    from triune_b200.export.safetensors_io import save_file
    from triune_b200.runtime.gguf_loader import build_hf_tokenizer_from_gguf, write_gguf
    from triune_b200.runtime.model_scanner import inspect_model_spec_for_upgrade, parse_gguf_header, resolve_ollama_host, scan_pc_models

    meta = {"general.architecture": "llama", "general.name": "tiny", "llama.block_count": 2, "llama.embedding_length": 64,
            "llama.attention.head_count": 4, "llama.feed_forward_length": 128, "llama.context_length": 512, "llama.vocab_size": 100}
    write_gguf(tmp_path / "m.gguf", {"token_embd.weight": (torch.randn(100, 64), 0), "blk.0.attn_q.weight": (torch.randn(64, 64), 8),
                                     "blk.1.attn_q.weight": (torch.randn(64, 64), 8)}, meta)
    head = parse_gguf_header(tmp_path / "m.gguf")
    assert (head["num_layers"], head["hidden_dim"], head["num_heads"], head["ffn_dim"], head["vocab_size"], head["quantization"]) == (2, 64, 4, 128, 100, "Q8_0")
    assert inspect_model_spec_for_upgrade(str(tmp_path / "m.gguf")) == (2, 64, 4, 128, 100, "LLAMA GGUF (m.gguf)")
    save_file({"model.embed_tokens.weight": torch.randn(50, 32), "model.layers.2.mlp.gate_proj.weight": torch.randn(96, 32)}, str(tmp_path / "x.safetensors"))
    assert inspect_model_spec_for_upgrade(str(tmp_path / "x.safetensors"))[:5] == (3, 32, 1, 96, 50)
    torch.save({"model_state": {"embed.weight": torch.randn(40, 16), "layers.1.ffn.w1": torch.randn(4, 16, 48)}}, tmp_path / "c.pt")
    assert inspect_model_spec_for_upgrade(str(tmp_path / "c.pt"))[:5] == (2, 16, 1, 48, 40)
    assert inspect_model_spec_for_upgrade(str(tmp_path / "c.pt"), checkpoint_arch_fn=lambda ck, fb: ("x", {"num_layers": 7, "hidden_dim": 128}))[:3] == (7, 128, 2)
    assert inspect_model_spec_for_upgrade("") is None and inspect_model_spec_for_upgrade(str(tmp_path / "nothing")) is None
    assert parse_gguf_header(tmp_path / "c.pt") is None
    rep = scan_pc_models([str(tmp_path)], include_wsl=False, installed_modules=[{"id": "m1"}])
    by_id = {m["id"].split(":")[0]: m for m in rep["models"]}
    assert by_id["gguf"]["num_layers"] == 2 and "checkpoint" in by_id and by_id["module"]["id"] == "module:m1" and str(tmp_path) in rep["scanned_roots"]
    assert resolve_ollama_host("localhost:11434/") == "http://localhost:11434"
    toks = ["<unk>", "<s>", "</s>"] + ["▁" + w for w in ("hello", "world")] + list("helowrd") + ["▁"]
    tk = build_hf_tokenizer_from_gguf({"tokenizer.ggml.tokens": toks, "tokenizer.ggml.scores": [0.0] * 3 + [-1.0] * 2 + [-5.0] * 8,
                                       "tokenizer.ggml.token_type": [2, 3, 3] + [1] * 10, "tokenizer.ggml.bos_token_id": 1,
                                       "tokenizer.ggml.eos_token_id": 2, "tokenizer.ggml.unknown_token_id": 0, "tokenizer.chat_template": "{{ messages }}"})
    ids = tk.encode("hello world")
    assert tk.decode(ids) == "hello world" and max(ids) < len(toks) and tk.bos_token == "<s>" and tk.chat_template == "{{ messages }}"
    with pytest.raises(ValueError):
        build_hf_tokenizer_from_gguf({})


def test_curated_modules_install_offline_and_register_plain_node_names(tmp_path):
    from triune_b200.execution.dag import NODE_TYPES, execute_dag
    from triune_b200.plugins.curated import CURATED, curated_path
    from triune_b200.plugins.curated.custom_loss_nodes.custom_loss_nodes import CentroidBalanceLoss, FocalCrossEntropyLoss, anneal_temperature
    from triune_b200.plugins.registry import PluginRegistry, file_sha256

    import json
    import shutil

    man = json.loads((curated_path("custom-loss-nodes") / "plugin.json").read_text())
    assert man["sha256"] == file_sha256(curated_path("custom_loss_nodes") / man["entry"])  # the shipped manifest matches the shipped file
    assert {c["id"] for c in CURATED} == {"custom_loss_nodes", "code_assistant_lora"}
    assert json.loads((curated_path("code_assistant_lora") / "adapter_config.json").read_text())["r"] == 16
    shutil.copytree(curated_path("custom_loss_nodes"), tmp_path / "custom_loss_nodes")
    reg = PluginRegistry(key="")
    reg.discover(tmp_path)
    try:
        info = reg.load("custom_loss_nodes")
        assert {"FocalCrossEntropyLoss", "custom_loss_nodes.FocalCrossEntropyLoss", "TemperatureAnnealer"} <= set(info.nodes)
        out = execute_dag({"nodes": [{"id": "t", "type": "TemperatureAnnealer", "params": {"global_step": 2500}}], "edges": []})
        assert out["outputs"]["t.temperature"] == pytest.approx(0.55)
    finally:
        for n in ("FocalCrossEntropyLoss", "CentroidBalanceLoss", "TemperatureAnnealer"):
            NODE_TYPES.pop(n, None), NODE_TYPES.pop(f"custom_loss_nodes.{n}", None)
    # an edited copy is an ordinary plugin: its nodes get the plugin's prefix only
    (tmp_path / "other").mkdir()
    shutil.copytree(curated_path("custom_loss_nodes"), tmp_path / "other" / "custom_loss_nodes")
    entry = tmp_path / "other" / "custom_loss_nodes" / man["entry"]
    entry.write_text(entry.read_text() + "\n# edited\n")
    from triune_b200.plugins.registry import write_manifest

    write_manifest(tmp_path / "other" / "custom_loss_nodes", key="")
    reg2 = PluginRegistry(key="")
    reg2.discover(tmp_path / "other")
    try:
        assert "FocalCrossEntropyLoss" not in reg2.load("custom_loss_nodes").nodes
    finally:
        for n in ("FocalCrossEntropyLoss", "CentroidBalanceLoss", "TemperatureAnnealer"):
            NODE_TYPES.pop(f"custom_loss_nodes.{n}", None)
    logits, tgt = torch.randn(2, 5, 7), torch.randint(0, 7, (2, 5))
    assert torch.allclose(FocalCrossEntropyLoss(0.0)(logits, tgt), F.cross_entropy(logits.view(-1, 7), tgt.view(-1)))
    assert FocalCrossEntropyLoss(2.0)(logits, tgt) < FocalCrossEntropyLoss(0.0)(logits, tgt)
    assert float(CentroidBalanceLoss(1.0)(torch.full((6, 4), 0.25))) == 0.0 and float(CentroidBalanceLoss(1.0)(torch.eye(4)[[0, 0, 0]])) == pytest.approx(0.75)
    assert anneal_temperature(0) == 1.0 and anneal_temperature(10 ** 6) == pytest.approx(0.1)


def test_upgrade_model_keeps_gemma_and_llama_logits():
    """Patching a third-party model must not change what it computes: Gemma stores its norm scale as an offset from one
    and gates its MLP with GELU, Llama uses the plain scale and SiLU."""
    from transformers import GemmaConfig, GemmaForCausalLM, LlamaConfig, LlamaForCausalLM

    from triune_b200.inference import IncrementalStreamingDecoder, optimize_hf_model_for_inference
    from triune_b200.models.universal import upgrade_model

    torch.manual_seed(0)
    for C, M, swiglu in ((GemmaConfig, GemmaForCausalLM, 0), (LlamaConfig, LlamaForCausalLM, 2)):
        cfg = C(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, head_dim=16,
                max_position_embeddings=64)
        m = M(cfg).eval()
        with torch.no_grad():
            for p in m.parameters():
                p.add_(torch.randn_like(p) * 0.05)
        x = torch.randint(0, 128, (2, 12))
        with torch.no_grad():
            want = m(x).logits
            optimize_hf_model_for_inference(m)
            assert torch.allclose(m(x).logits, want, atol=1e-5)
            upgrade_model(m)
            assert torch.allclose(m(x).logits, want, atol=1e-5)
        assert m._triune_upgrade["rmsnorm"] == 5 and m._triune_upgrade["swiglu"] == swiglu

    class Tk:
        def decode(self, ids):
            return bytes(ids).decode("utf-8", errors="replace")

    dec = IncrementalStreamingDecoder(Tk())
    pieces = [dec.step(b)[1] for b in "hé there".encode("utf-8")]
    assert "".join(pieces) + dec.flush()[1] == "hé there" and "" in pieces and dec.cumulative_text == "hé there"


def test_terminal_rendering_plain_and_rich(capsys, monkeypatch):
    from triune_b200 import cli_ui

    for rich in (cli_ui.HAS_RICH, False):
        monkeypatch.setattr(cli_ui, "HAS_RICH", rich)
        cli_ui.render_banner("TITLE", "sub", "badge")
        cli_ui.render_kv_panel("card", [("key", 1), ("longer key", "v")], footer="foot")
        cli_ui.render_table("tab", [("name", "left", "cyan"), ("n", "right", "")], [["a", 1], ["bbb", 22]], caption="cap")
        cli_ui.render_notice("done", "success")
        cli_ui.render_telemetry_bar("limbic", tok_sec=12.3, ttft_ms=4.5, tokens=7, latency_ms=99, vram_gb=1.5, load_s=0.2, extra="x")
        cli_ui.render_rule("rule")
        with cli_ui.status_spinner("working"):
            pass
        out = capsys.readouterr().out
        for piece in ("TITLE", "badge", "sub", "card", "longer key", "foot", "tab", "bbb", "22", "cap", "done", "LIMBIC", "12.3 tok/s", "4.5ms", "1.50GB", "rule", "working"):
            assert piece in out, (rich, piece)
        assert "\x1b[" not in out and "[bold" not in out  # no colour codes or markup when stdout is not a terminal
    assert cli_ui.route_badge_ansi("reflex") == "[REFLEX]" and "CORTEX" in cli_ui.route_badge_markup("cortex") and "OLLAMA" in cli_ui.route_badge_markup("ollama:x")
    cli_ui.render_help_overview()
    overview = capsys.readouterr().out
    assert all(c in overview for c in ("train", "finetune", "serve", "doctor", "plugin"))
    from triune_b200.cli import main

    assert main([]) == 0 and "chat" in capsys.readouterr().out
