"""More node types for the DAG executor: one small handler per framework component, so a graph can wire operators,
losses, optimizers, data sources, runtime services and exports together.

Every handler has the executor's signature ``(inputs, params, context) -> outputs`` and only forwards to code that
lives elsewhere in the package; nothing here computes on its own. The set mirrors the node catalogue of the
reference's executor (``triune/execution/dag.py:474-541``: data sources, tokenizer, loaders, model parts, optimizers,
schedule, losses, runtime services, inspectors, evaluation, fine-tuning, exports); names are this package's own.
Importing this module registers the nodes (``execution/dag.py`` does so at the end of its own definitions).
"""

from __future__ import annotations

import math
from typing import Any, Dict

from .dag import ANY, register_node

T = "tensor"


def _torch():
    import torch

    return torch


# ---------------------------------------------------------------------------------------------------- data
@register_node("local_file_reader", {}, {"texts": "json"}, "documents of a .jsonl / .txt / .parquet file or directory (params: path, limit)")
def _local_files(i, p, c):
    from ..data.dataset import iter_local_texts

    out = []
    for t in iter_local_texts(str(p["path"])):
        out.append(t)
        if len(out) >= int(p.get("limit", 1000)):
            break
    return {"texts": out}


@register_node("synthetic_tokens", {}, {"loader": "loader"}, "endless random token batches (params: vocab_size, batch_size, seq_len, seed)")
def _synthetic(i, p, c):
    from ..data import SyntheticTokenSource

    return {"loader": SyntheticTokenSource(int(p.get("vocab_size", 256)), int(p.get("batch_size", 2)), int(p.get("seq_len", 32)),
                                           seed=int(p.get("seed", 0)), pool=int(p.get("pool", 4)))}


@register_node("cycling_loader", {"batches": "json"}, {"loader": "loader"}, "repeat a finite list of batches for ever")
def _cycling(i, p, c):
    from ..data.dataloader import CyclingDataLoader

    return {"loader": CyclingDataLoader(list(i["batches"]))}


@register_node("next_batch", {"loader": "loader"}, {"input_ids": T, "labels": T}, "draw one (inputs, labels) batch")
def _next_batch(i, p, c):
    b = next(iter(i["loader"])) if not hasattr(i["loader"], "__next__") else next(i["loader"])
    x, y = (b[0], b[1]) if isinstance(b, (tuple, list)) else (b[:, :-1], b[:, 1:])
    return {"input_ids": x, "labels": y}


@register_node("bpe_tokenizer", {"text": "text"}, {"ids": "tokens", "count": "json"}, "tokenise with params['tokenizer_path'] (bytes when absent)")
def _bpe(i, p, c):
    if p.get("tokenizer_path"):
        from ..data.tokenizer import load_tokenizer

        out = load_tokenizer(p["tokenizer_path"]).encode(i["text"])
        ids = list(getattr(out, "ids", out))
    else:
        ids = list(i["text"].encode("utf-8"))
    return {"ids": ids, "count": len(ids)}


@register_node("token_batch_inspector", {"input_ids": T}, {"out": "json"}, "shape, range and repetition of a token batch")
def _tok_inspect(i, p, c):
    x = i["input_ids"]
    return {"out": {"shape": list(x.shape), "min": int(x.min()), "max": int(x.max()), "unique": int(x.unique().numel())}}


@register_node("tensor_inspector", {"x": T}, {"out": "json", "x": T}, "shape, dtype, mean, std, finite check; passes the tensor on")
def _tensor_inspect(i, p, c):
    x = i["x"]
    f = x.detach().float()
    return {"x": x, "out": {"shape": list(x.shape), "dtype": str(x.dtype), "mean": float(f.mean()), "std": float(f.std()) if f.numel() > 1 else 0.0,
                            "abs_max": float(f.abs().max()), "finite": bool(_torch().isfinite(f).all())}}


@register_node("random_tensor", {}, {"x": T}, "normal noise (params: shape, seed, scale)")
def _random(i, p, c):
    torch = _torch()
    return {"x": torch.randn(*[int(s) for s in p.get("shape", [2, 8])], generator=torch.Generator().manual_seed(int(p.get("seed", 0))))
            * float(p.get("scale", 1.0))}


# ---------------------------------------------------------------------------------------------------- operators
@register_node("rmsnorm", {"x": T}, {"y": T}, "RMS normalisation with unit weight (params: eps)")
def _rmsnorm(i, p, c):
    from .. import ops

    x = i["x"]
    return {"y": ops.rmsnorm(x, _torch().ones(x.shape[-1], dtype=x.dtype, device=x.device), float(p.get("eps", 1e-6)))}


@register_node("rope", {"x": T}, {"y": T}, "rotary embedding of [B, T, H, D] (params: base, offset)")
def _rope(i, p, c):
    from .. import ops

    x = i["x"]
    cos, sin = ops.rope_tables(x.shape[1], x.shape[-1], float(p.get("base", 10000.0)), int(p.get("offset", 0)), x.device)
    return {"y": ops.apply_rope(x, cos, sin)}


@register_node("gla", {"q": T, "k": T, "v": T, "g": T}, {"out": T, "state": T}, "gated linear attention over [B, T, H, D]")
def _gla(i, p, c):
    from .. import ops

    o, s = ops.gla(i["q"], i["k"], i["v"], i["g"], scale=float(p.get("scale", 1.0)), gate_logits=bool(p.get("gate_logits", True)))
    return {"out": o, "state": s}


@register_node("gated_deltanet", {"q": T, "k": T, "v": T, "g": T, "beta": T}, {"out": T, "state": T}, "delta-rule linear attention", optional=("beta",))
def _gdn(i, p, c):
    from .. import ops

    o, s = ops.gated_deltanet(i["q"], i["k"], i["v"], i["g"], beta=i.get("beta"), scale=float(p.get("scale", 1.0)),
                              gate_logits=bool(p.get("gate_logits", True)))
    return {"out": o, "state": s}


@register_node("moe_route", {"logits": T}, {"indices": T, "weights": T}, "top-k expert routing (params: top_k, temperature)")
def _route(i, p, c):
    from .. import ops

    lg = i["logits"]
    out = ops.moe_route(lg, _torch().zeros(lg.shape[-1], dtype=lg.dtype, device=lg.device), int(p.get("top_k", 2)), float(p.get("temperature", 1.0)))
    return {"indices": out[0], "weights": out[1]}


@register_node("fp8_linear", {"x": T, "w": T}, {"y": T}, "block-scaled FP8 weight, bf16 activations")
def _fp8(i, p, c):
    from ..models.quant_linear import FP8Linear

    torch = _torch()
    w = i["w"]
    lin = torch.nn.Linear(w.shape[1], w.shape[0], bias=False, device=w.device, dtype=w.dtype)
    with torch.no_grad():
        lin.weight.copy_(w)
    return {"y": FP8Linear.from_linear(lin, int(p.get("block", 128)))(i["x"])}


@register_node("nvfp4_roundtrip", {"w": T}, {"w": T, "error": "json"}, "quantise a weight to NVFP4 and back; reports the relative error")
def _fp4(i, p, c):
    from .. import ops

    w = i["w"]
    packed, scales, ts = ops.nvfp4_quantize(w, hadamard=bool(p.get("hadamard", False)))[:3]
    back = ops.nvfp4_dequantize(packed, scales, ts, dtype=w.dtype)
    back = back[: w.shape[0], : w.shape[1]]
    return {"w": back, "error": float((back.float() - w.float()).norm() / w.float().norm().clamp_min(1e-12))}


# ---------------------------------------------------------------------------------------------------- losses
@register_node("cross_entropy", {"logits": T, "labels": T}, {"loss": T}, "mean next-token cross entropy")
def _ce(i, p, c):
    from .. import ops

    lg = i["logits"]
    return {"loss": ops.cross_entropy(lg.reshape(-1, lg.shape[-1]), i["labels"].reshape(-1))}


@register_node("joint_exit_loss", {"model": "model", "input_ids": T, "labels": T}, {"loss": T, "parts": "json"},
               "weighted sum of the losses at the three exits (params: weights)")
def _joint(i, p, c):
    losses, _ = i["model"].exit_losses(i["input_ids"], i["labels"], update_stats=False)
    w = p.get("weights", [0.2, 0.3, 0.5])
    return {"loss": sum(float(a) * l for a, l in zip(w, losses)), "parts": [float(l.detach()) for l in losses]}


@register_node("router_z_loss", {"logits": T}, {"loss": T}, "mean squared log-partition of router logits")
def _zloss(i, p, c):
    return {"loss": _torch().logsumexp(i["logits"].float(), dim=-1).pow(2).mean() * float(p.get("coef", 1.0))}


@register_node("perplexity", {"model": "model", "input_ids": T, "labels": T}, {"out": "json"}, "loss and perplexity at one depth (params: depth)")
def _ppl(i, p, c):
    torch = _torch()
    with torch.no_grad():
        m = i["model"]
        was = m.training
        m.eval()
        try:
            loss = float(m.forward_loss(i["input_ids"], i["labels"], force_depth=int(p.get("depth", 2))))
        finally:
            m.train(was)
    return {"out": {"loss": loss, "ppl": math.exp(min(loss, 50.0))}}


# ---------------------------------------------------------------------------------------------------- optimizers, schedule, steps
def _make_opt(kind: str):
    def handler(i, p, c):
        from ..optim import build_optimizer

        cfg = {"optimizer": kind, "lr": float(p.get("lr", 1e-4)), "weight_decay": float(p.get("weight_decay", 0.05))}
        cfg.update({k: v for k, v in p.items() if k not in cfg})
        return {"optimizer": build_optimizer(i["model"], cfg), "model": i["model"]}

    return handler


for _name, _kind in (("centroid_steer_optimizer", "centroid_steer"), ("muon_optimizer", "muon"), ("adamw_optimizer", "adamw")):
    register_node(_name, {"model": "model"}, {"optimizer": "optimizer", "model": "model"}, f"build the {_kind} optimizer (params: lr, weight_decay)")(_make_opt(_kind))


@register_node("cosine_lr", {}, {"lr": "json"}, "warm-up + cosine learning rate at params['step']")
def _cos(i, p, c):
    from ..trainer.rescue import cosine_lr

    lr = float(p.get("lr", 1e-4))
    return {"lr": cosine_lr(int(p.get("step", 0)), int(p.get("total_steps", 1000)), int(p.get("warmup_steps", 10)), lr, lr * float(p.get("min_ratio", 0.1)))}


@register_node("training_step", {"model": "model", "optimizer": "optimizer", "input_ids": T, "labels": T}, {"model": "model", "loss": "json"},
               "one forward / backward / update at params['depth']")
def _step(i, p, c):
    m, opt = i["model"], i["optimizer"]
    m.train()
    opt.zero_grad()
    loss = m.forward_loss(i["input_ids"], i["labels"], force_depth=int(p.get("depth", 2)))
    loss.backward()
    opt.step()
    return {"model": m, "loss": float(loss.detach())}


@register_node("gradient_accumulator", {"model": "model", "loader": "loader"}, {"model": "model", "loss": "json"},
               "accumulate gradients over params['micro_batches'] batches without stepping")
def _accum(i, p, c):
    m, n, tot = i["model"], int(p.get("micro_batches", 2)), 0.0
    m.train()
    it = iter(i["loader"])
    for _ in range(n):
        b = next(it)
        x, y = (b[0], b[1]) if isinstance(b, (tuple, list)) else (b[:, :-1], b[:, 1:])
        loss = m.forward_loss(x, y, force_depth=int(p.get("depth", 2))) / n
        loss.backward()
        tot += float(loss.detach())
    return {"model": m, "loss": tot}


# ---------------------------------------------------------------------------------------------------- runtime services
@register_node("checkpoint_save", {"model": "model"}, {"path": "text"}, "write a training checkpoint (params: path, step)")
def _ck_save(i, p, c):
    from ..trainer import checkpoint as ckpt

    return {"path": ckpt.save_checkpoint(str(p["path"]), model=i["model"], step=int(p.get("step", 0)), config=dict(p.get("config", {})))}


@register_node("checkpoint_load", {}, {"model": "model"}, "build the model a checkpoint describes and load it (params: path)")
def _ck_load(i, p, c):
    from ..inference import load_checkpoint_model

    return {"model": load_checkpoint_model(str(p["path"]))[0]}


@register_node("vram_profiler", {}, {"out": "json"}, "device memory statistics")
def _vram(i, p, c):
    from ..runtime.vram import VRAMProfiler

    return {"out": VRAMProfiler.get_vram_stats(p.get("device", "cuda"))}


@register_node("resource_manager", {}, {"out": "json"}, "hardware profile of the machine")
def _resources(i, p, c):
    from dataclasses import asdict

    from ..runtime.resource_manager import DynamicResourceManager

    return {"out": asdict(DynamicResourceManager.probe_hardware(p.get("device")))}


@register_node("layer_streaming", {"model": "model"}, {"model": "model", "out": "json"}, "keep layers in host memory and stream them through the device")
def _streaming(i, p, c):
    from ..runtime.streaming import StreamingConfig, enable_layer_streaming

    eng = enable_layer_streaming(i["model"], p.get("device", "cuda" if _torch().cuda.is_available() else "cpu"),
                                 config=StreamingConfig(resident_gpu_layers=int(p.get("resident_layers", 2))))
    return {"model": i["model"], "out": dict(eng.get_telemetry())}


@register_node("lora_adapter", {"model": "model"}, {"model": "model", "out": "json"}, "attach LoRA adapters (params: rank, alpha)")
def _lora(i, p, c):
    from ..trainer.finetune import LoRAConfig, TriuneFineTuner

    ft = TriuneFineTuner(i["model"], LoRAConfig(rank=int(p.get("rank", 8)), alpha=float(p.get("alpha", 16.0))))
    c.setdefault("finetuners", []).append(ft)
    return {"model": i["model"], "out": {"adapters": len(ft.applied_adapters), "trainable": ft.count_trainable_parameters()}}


@register_node("subgraph", {"value": ANY}, {"out": ANY}, "run params['dag'] with `value` offered to its node 'input'; returns its port params['output']", optional=("value",))
def _subgraph(i, p, c):
    from .dag import execute_dag

    spec = {"nodes": list(p["dag"].get("nodes", [])), "edges": list(p["dag"].get("edges", []))}
    spec["nodes"] = [dict(n, params=dict(n.get("params", {}), value=i.get("value"))) if n["id"] == "input" else n for n in spec["nodes"]]
    res = execute_dag(spec, c)
    return {"out": res["outputs"].get(str(p.get("output", "")))}


# ---------------------------------------------------------------------------------------------------- exports that refuse politely
@register_node("gguf_export", {"model": "model"}, {"path": "text"}, "not supported: raises NotImplementedError like the exporter")
def _gguf(i, p, c):
    from ..export import export_model

    return {"path": str(export_model(i["model"], p.get("output", "model.gguf"), "gguf"))}


@register_node("onnx_export", {"model": "model"}, {"path": "text"}, "ONNX export of the forward pass")
def _onnx(i, p, c):
    from ..export import export_model

    return {"path": str(export_model(i["model"], p["output"], "onnx"))}


@register_node("safetensors_export", {"model": "model"}, {"path": "text"}, "weights as one .safetensors file")
def _st(i, p, c):
    from ..export import export_model

    return {"path": str(export_model(i["model"], p["output"], "safetensors"))}
