"""Command line interface: ``python -m triune_b200 <command>``.

Parity with the sub-commands of ``triune/cli.py:39-1618`` that concern the ML core and serving: ``serve``, ``chat``,
``infer``, ``scan``, ``transmute``, ``finetune``, ``adapter {list,merge,export}``, ``checkpoint {list,export}``,
``export``, ``models``, ``train``, ``bench``, ``gpucheck``, ``plan-memory``, ``cache`` (NVFP4 disk cache), ``native``
(build the extensions), ``profile``, ``tokenizer``, ``sandbox``; and of the product shell: ``desktop`` (launcher, also
through WSL 2 on a Windows host), ``package`` (launcher bundles), ``install`` / ``uninstall`` (``installer.py``).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path
from typing import Any, Dict, List, Optional


def _device(arg: Optional[str]):
    import torch

    return torch.device(arg or ("cuda:0" if torch.cuda.is_available() else "cpu"))


def _dtype(dev):
    import torch

    return torch.bfloat16 if dev.type == "cuda" else torch.float32


def _print(obj) -> None:
    print(json.dumps(obj, indent=2, default=str))


def _load_for_inference(args):
    from .serve.engine_state import EngineState

    st = EngineState(str(_device(args.device)))
    st.load_model(args.model, getattr(args, "tokenizer", None), getattr(args, "precision", None))
    return st


# ---------------------------------------------------------------------------------------------------- commands
def cmd_serve(a) -> int:
    from .serve import run_server

    if a.model:
        from .serve import get_state

        get_state().load_model(a.model, a.tokenizer, a.precision)
    run_server(a.host, a.port, a.static_dir)
    return 0


def cmd_chat(a) -> int:
    st = _load_for_inference(a)
    sid = "cli"
    print(f"loaded {st.config.get('model_id')} ({st.config.get('params', 0) / 1e6:.1f}M parameters) on {st.device}; empty line quits")
    while True:
        try:
            prompt = input("you> ").strip()
        except (EOFError, KeyboardInterrupt):
            break
        if not prompt:
            break
        sys.stdout.write("model> ")
        out = st.generate(prompt, session_id=sid, max_new_tokens=a.max_tokens, temperature=a.temperature, top_k=a.top_k,
                          decode_depth=a.depth, stream_callback=lambda s: (sys.stdout.write(s), sys.stdout.flush()),
                          speculative=a.speculative)
        t = out["telemetry"]
        print()
        from .cli_ui import render_telemetry_bar

        render_telemetry_bar(str(t.get("exit") or t.get("depth") or a.depth or "auto"), tok_sec=float(t.get("decode_tok_s", 0.0)),
                             ttft_ms=1e3 * float(t.get("ttft_s", 0.0)), tokens=int(t.get("new_tokens", 0)),
                             latency_ms=1e3 * float(t.get("total_s", 0.0) or 0.0))
    return 0


def cmd_infer(a) -> int:
    st = _load_for_inference(a)
    prompt = a.prompt if a.prompt is not None else sys.stdin.read()
    out = st.generate(prompt, max_new_tokens=a.max_tokens, temperature=a.temperature, top_k=a.top_k, decode_depth=a.depth,
                      template=not a.raw, speculative=a.speculative)
    if a.json:
        _print({"text": out["text"], "telemetry": out["telemetry"]})
    else:
        print(out["text"])
    return 0


def cmd_scan(a) -> int:
    from .runtime.model_scanner import scan_models

    _print(scan_models(a.paths or None, max_depth=a.depth))
    return 0


def cmd_transmute(a) -> int:
    import torch

    from .models.transmuter import transfer_weights_to_native_triune, transmute_hf_to_triune

    if a.mode == "exits":
        model, meta = transmute_hf_to_triune(a.source, reflex_ratio=a.reflex_ratio, rank=a.rank, use_jev=not a.no_jev,
                                             device=_device(a.device), local_files_only=not a.online)
    else:
        from transformers import AutoModelForCausalLM

        teacher = AutoModelForCausalLM.from_pretrained(a.source, local_files_only=not a.online)
        model, meta = transfer_weights_to_native_triune(teacher, num_experts=a.experts, top_k=a.top_k, target_layers=a.layers,
                                                        target_dim=a.dim, reflex_ratio=a.reflex_ratio)
    if a.output:
        Path(a.output).parent.mkdir(parents=True, exist_ok=True)
        torch.save({"model_state": model.state_dict(), "config": {}, "transmute": meta}, a.output)
        meta["saved_to"] = a.output
    _print(meta)
    return 0


def _read_records(path: str) -> List[Any]:
    p = Path(path)
    if p.suffix == ".jsonl":
        return [json.loads(l) for l in p.read_text(encoding="utf-8").splitlines() if l.strip()]
    if p.suffix == ".json":
        data = json.loads(p.read_text(encoding="utf-8"))
        return data if isinstance(data, list) else data.get("data", [])
    return [{"text": t} for t in p.read_text(encoding="utf-8").split("\n\n") if t.strip()]


def cmd_finetune(a) -> int:
    from .trainer.finetune import LoRAConfig, TriuneFineTuner

    st = _load_for_inference(a)
    ft = TriuneFineTuner(st.model, LoRAConfig(rank=a.rank, alpha=a.alpha, dropout=a.dropout, use_qlora=a.qlora), tokenizer=st.tokenizer,
                         model_name_or_path=a.model)
    res = ft.fit(_read_records(a.data), epochs=a.epochs, batch_size=a.batch_size, lr=a.lr, max_seq_len=a.seq_len, max_steps=a.max_steps,
                 callback=lambda r: print(f"step {r['step']:5d}  loss {r['loss']:.4f}  lr {r['lr']:.2e}  {r['tok_s']:.0f} tok/s"))
    out = ft.save_adapter(a.output)
    _print({k: v for k, v in res.items() if k != "history"} | {"adapter_dir": str(out)})
    return 0


def cmd_adapter(a) -> int:
    from .trainer.finetune import export_adapter, list_adapters, merge_adapter_checkpoint

    if a.action == "list":
        _print(list_adapters(a.dirs or None))
    elif a.action == "merge":
        import torch

        from .models.zoo import load_model

        model = merge_adapter_checkpoint(load_model(a.base), a.adapter, a.output)
        _print({"merged_into": a.base, "saved_to": a.output, "parameters": sum(p.numel() for p in model.parameters())})
    elif a.action == "export":
        _print({"path": str(export_adapter(a.adapter, a.output, a.format))})
    return 0


def cmd_checkpoint(a) -> int:
    if a.action == "list":
        d = Path(a.dir)
        rows = [{"name": p.name, "size_mb": round(p.stat().st_size / 2**20, 1), "modified": time.ctime(p.stat().st_mtime)}
                for p in sorted(d.glob("*.pt"))] if d.is_dir() else []
        _print(rows)
        return 0
    if a.action == "merge":
        from .trainer.sharded_checkpoint import merge_shards

        out = a.output if a.output != "exports/model.safetensors" else str(Path(a.dir) / "merged.pt")
        payload = merge_shards(a.dir, out)
        _print({"path": out, "tensors": len(payload["model_state"]), "shards": payload["merged_from"]["shards"],
                "step": payload["step"]})
        return 0
    return cmd_export(a)


def cmd_export(a) -> int:
    from .export import export_model
    from .models.zoo import load_model

    model = load_model(a.model)
    try:
        path = export_model(model, a.output, a.format)
    except NotImplementedError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    _print({"path": str(path), "format": a.format})
    return 0


def cmd_models(a) -> int:
    from .models.zoo import CANONICAL_MODEL_SPECS

    from .cli_ui import render_table

    rows = []
    for k, s in CANONICAL_MODEL_SPECS.items():
        total, active = s.compute_exact_params()
        rows.append([k, f"{total / 1e6:.1f}M", f"{active / 1e6:.1f}M", s.num_layers, s.hidden_dim, s.num_experts, s.tier])
    render_table("Model presets", [("preset", "left", "bold cyan"), ("parameters", "right", ""), ("active", "right", ""), ("layers", "right", ""),
                                   ("dim", "right", ""), ("experts", "right", ""), ("tier", "left", "dim")], rows)
    return 0


def _train_elastic(a) -> int:
    """Data-parallel training that survives lost ranks. Selected by the environment the elastic launcher sets
    (``TRIUNE_ELASTIC_STORE=host:port``, ``TRIUNE_ELASTIC_IDENT``, ``TRIUNE_ELASTIC_WORLD``). Gradients are reduced with
    library collectives here: a fused NVLink group is built over a fixed set of peers and cannot lose a member."""
    import torch

    from .config import build_config
    from .data import SyntheticTokenSource
    from .models.zoo import load_model
    from .optim import CentroidSteerOptimizer
    from .parallel.data_parallel import ShardedDataParallel
    from .parallel.dist import DistributedContext
    from .parallel.elastic import ElasticGroup, run_elastic
    from .trainer import Trainer
    from .utils import place_model

    host, _, port = os.environ["TRIUNE_ELASTIC_STORE"].rpartition(":")
    ident, world = int(os.environ["TRIUNE_ELASTIC_IDENT"]), int(os.environ["TRIUNE_ELASTIC_WORLD"])
    cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", ident))
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
    backend = "nccl" if cuda else "gloo"
    group = ElasticGroup(host or "127.0.0.1", int(port), ident, world, backend,
                         hb_timeout=float(os.environ.get("TRIUNE_ELASTIC_HB_TIMEOUT", "3.0")),
                         pg_timeout=float(os.environ.get("TRIUNE_ELASTIC_PG_TIMEOUT", "30.0")), device_id=dev if cuda else None)
    over = json.loads(a.overrides) if a.overrides else {}
    latest = os.path.join(a.checkpoint_dir, "latest.pt")
    state: Dict[str, Any] = {}

    def build() -> int:
        """(Re)build everything that depends on the membership, then load the last checkpoint if there is one."""
        state.pop("tr", None)
        ctx = DistributedContext(True, group.rank, local, group.world, backend, dev)
        torch.manual_seed(0)
        model = place_model(load_model(a.model, **over), dev, _dtype(dev))
        cfg = build_config({"batch_size": a.batch_size, "seq_len": a.seq_len, "lr": a.lr, "total_steps": a.steps, "depth_mode": a.depth_mode,
                            "grad_accum_steps": a.grad_accum, "checkpoint_dir": a.checkpoint_dir, "vocab_size": int(model.vocab_size),
                            "cuda_graph": False})
        dp = ShardedDataParallel(ctx, mode="nccl") if group.world > 1 else None
        opt = CentroidSteerOptimizer(model, lr=a.lr, grad_clip=1.0, storage_factory=dp.storage_factory if dp is not None else None)
        loader = SyntheticTokenSource(int(model.vocab_size), cfg["batch_size"], cfg["seq_len"], seed=group.ident)
        tr = Trainer(model, cfg, optimizer=opt, train_loader=loader, device=dev, dp=dp)
        resume_from = latest if os.path.exists(latest) else (a.resume if a.resume and os.path.exists(a.resume) else None)
        if resume_from:
            tr.resume(resume_from)
        state["tr"], state["cfg"] = tr, cfg
        return int(tr.engine.step)

    def step_fn(step, g):
        out = state["tr"].engine.step_once()
        if g.rank == 0 and state["tr"].engine.step % a.log_every == 0:
            print(f"step {state['tr'].engine.step:6d}  loss {float(out['loss']):.4f}  world {g.world}", flush=True)
        return float(out["loss"])

    res = run_elastic(group, step_fn, lambda step: state["tr"].save_latest(), build, total_steps=a.steps,
                      checkpoint_every=max(1, int(os.environ.get("TRIUNE_ELASTIC_CKPT_EVERY", "10"))))
    if group.rank == 0:
        _print({k: res[k] for k in ("steps", "world", "members", "generation", "failures")})
    group.shutdown()
    return 0


def cmd_train(a) -> int:
    if os.environ.get("TRIUNE_ELASTIC_STORE"):
        return _train_elastic(a)
    import torch

    from .config import build_config
    from .data import SyntheticTokenSource
    from .models.zoo import load_model
    from .optim import CentroidSteerOptimizer
    from .parallel import setup_distributed
    from .trainer import Trainer
    from .utils import place_model

    ctx = setup_distributed()
    dev = ctx.device
    over = json.loads(a.overrides) if a.overrides else {}
    model = place_model(load_model(a.model, **over), dev, _dtype(dev))
    cfg = build_config({"batch_size": a.batch_size, "seq_len": a.seq_len, "lr": a.lr, "total_steps": a.steps, "depth_mode": a.depth_mode,
                        "grad_accum_steps": a.grad_accum, "checkpoint_dir": a.checkpoint_dir, "vocab_size": int(model.vocab_size),
                        "cuda_graph": a.cuda_graph and dev.type == "cuda" and a.depth_mode == "cortex"})
    if a.plan or a.force or a.auto_fit:
        from .runtime.resource_manager import DynamicResourceManager

        plan = DynamicResourceManager.validate_and_allot({**cfg, **over, "num_layers": model.num_layers, "hidden_dim": model.hidden_dim},
                                                         device=dev, force=a.force, auto_fit=a.auto_fit, model=model)
        cfg["batch_size"], cfg["grad_accum_steps"] = plan.batch_size, plan.grad_accum_steps
    dp = None
    if ctx.world_size > 1:
        from .parallel.data_parallel import ShardedDataParallel

        dp = ShardedDataParallel(ctx, mode=a.dp_mode)
    opt = CentroidSteerOptimizer(model, lr=a.lr, grad_clip=1.0, storage_factory=dp.storage_factory if dp is not None else None)
    if a.data:
        from .data import build_dataloader, load_tokenizer

        tok = load_tokenizer(a.tokenizer)
        sep = tok.token_to_id("[SEP]") or 3
        loader = build_dataloader(tok, {**cfg, "dataset_name": a.data, "dataset_config": None}, sep, is_holdout=False, rank=ctx.rank,
                                  world_size=ctx.world_size)
    else:
        loader = SyntheticTokenSource(int(model.vocab_size), cfg["batch_size"], cfg["seq_len"], seed=ctx.rank)
    tr = Trainer(model, cfg, optimizer=opt, train_loader=loader, device=dev, dp=dp)
    if a.resume and os.path.exists(a.resume):
        tr.resume(a.resume)
    t0, toks = time.perf_counter(), 0
    for _ in range(a.steps):
        out = tr.engine.step_once()
        toks += cfg["batch_size"] * cfg["seq_len"] * ctx.world_size
        if ctx.rank == 0 and tr.engine.step % a.log_every == 0:
            print(f"step {tr.engine.step:6d}  loss {float(out['loss']):.4f}  {toks / (time.perf_counter() - t0):,.0f} tok/s", flush=True)
    if ctx.rank == 0 and a.save:
        print("saved", tr.save_latest())
    return 0


def cmd_bench(a) -> int:
    import subprocess

    root = Path(__file__).resolve().parent.parent
    if a.kernels:
        return subprocess.call([sys.executable, "-m", "triune_b200.bench_kernels", "--case", a.kernels])
    cmd = [sys.executable, str(root / "bench.py"), "--steps", str(a.steps), "--warmup", str(a.warmup)]
    if a.gpus > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", "29555", str(root / "bench.py"), "--gpus", str(a.gpus), "--steps", str(a.steps), "--warmup", str(a.warmup)]
    return subprocess.call(cmd)


def cmd_gpucheck(a) -> int:
    import torch

    from . import _ext
    from .runtime.capabilities import PrecisionCapabilities
    from .runtime.resource_manager import DynamicResourceManager

    info: Dict[str, Any] = {"torch": torch.__version__, "cuda_available": torch.cuda.is_available(), "extension_built": _ext.ext_available()}
    if torch.cuda.is_available():
        from dataclasses import asdict

        info["devices"] = [asdict(DynamicResourceManager.probe_hardware(f"cuda:{i}")) for i in range(torch.cuda.device_count())]
        info["capabilities"] = PrecisionCapabilities.detect("cuda:0").summary()
        info["cuda_runtime"] = torch.version.cuda
    _print(info)
    return 0


def cmd_doctor(a) -> int:
    """One report of everything an installation depends on; exit code 1 when something required is missing."""
    import importlib.util
    import platform

    import torch

    from . import _ext
    from .models.zoo import CANONICAL_MODEL_SPECS

    rep: Dict[str, Any] = {"python": platform.python_version(), "platform": platform.platform(), "torch": torch.__version__,
                           "cuda_available": torch.cuda.is_available(), "cuda_runtime": torch.version.cuda}
    problems: List[str] = []
    if torch.cuda.is_available():
        rep["gpus"] = []
        for i in range(torch.cuda.device_count()):
            pr = torch.cuda.get_device_properties(i)
            rep["gpus"].append({"index": i, "name": pr.name, "memory_gib": round(pr.total_memory / 2**30, 2), "capability": f"{pr.major}.{pr.minor}",
                                "sms": pr.multi_processor_count})
            if pr.major != 10:
                problems.append(f"GPU {i} ({pr.name}) is not compute capability 10.x: the sm_100a kernels cannot run on it")
    rep["cuda_extension"] = {"built": _ext.ext_available()}
    if torch.cuda.is_available() and not _ext.ext_available():
        problems.append("the CUDA extension is not built: run `python -m triune_b200 native`")
    try:
        from .ops import _c_bridge

        rep["native_host_library"] = _c_bridge.get_native_c_info()
    except Exception as e:
        rep["native_host_library"] = {"loaded": False, "error": f"{type(e).__name__}: {e}"}
    rep["model_zoo"] = {"presets": len(CANONICAL_MODEL_SPECS)}
    rep["optimizers"] = ["centroid_steer (subspace tier with triangular core)", "muon (Newton-Schulz)", "adamw"]
    rep["server_extras"] = {m: importlib.util.find_spec(m) is not None for m in ("fastapi", "uvicorn", "pydantic")}
    if not all(rep["server_extras"].values()):
        problems.append("the HTTP server needs fastapi, uvicorn and pydantic")
    rep["optional"] = {m: importlib.util.find_spec(m) is not None for m in ("tokenizers", "safetensors", "pyarrow", "transformers", "datasets")}
    studio = Path(__file__).resolve().parent / "studio" / "index.html"
    rep["studio_page"] = studio.is_file()
    try:
        from .runtime.model_scanner import query_ollama_running_tags

        tags = sorted(query_ollama_running_tags())
        rep["local_ollama"] = tags[:6] if tags else "not detected on 127.0.0.1:11434"
    except Exception:
        rep["local_ollama"] = "not probed"
    ck = Path("checkpoints_full")
    rep["checkpoints"] = sorted(p.name for p in ck.glob("*.pt"))[:8] if ck.is_dir() else []
    try:  # a forward pass of a tiny model is the one end-to-end proof that the install computes
        from .models.zoo import load_model

        m = load_model("default", vocab_size=64, hidden_dim=32, num_layers=4, num_heads=1, head_dim=32, num_experts=2, router_prefix_layers=1,
                       reflex_exit_layer=2, limbic_exit_layer=3)
        y = m(torch.randint(0, 64, (1, 8)), force_depth=2)[0]
        rep["tiny_forward"] = bool(torch.isfinite(y).all())
    except Exception as e:
        rep["tiny_forward"] = False
        problems.append(f"a tiny forward pass failed: {type(e).__name__}: {e}")
    rep["status"] = "healthy" if not problems else "problems"
    rep["problems"] = problems
    _print(rep)
    return 0 if not problems else 1


def cmd_agent(a) -> int:
    """A goal through the agent harness (persona, workspace tools, skills, persistent memory) on a locally loaded model."""
    from .agents.harness import AgentHarness

    goal = a.goal or a.goal_pos
    if not goal:
        print("a goal is required (positional or --goal)", file=sys.stderr)
        return 2
    st = _load_for_inference(a)

    def generate(prompt: str) -> str:
        return st.generate(prompt, max_new_tokens=a.max_tokens, temperature=0.7, template=False)["text"]

    h = AgentHarness(generate, a.store_dir, workspace=a.workspace, persona=a.persona, read_only=a.read_only, allow_shell=a.allow_shell,
                     auto_skill=not a.no_auto_skill, max_steps=a.max_steps)
    if a.team:
        _print(h.run_team(goal, [n.strip() for n in a.team.split(",") if n.strip()]))
    else:
        _print(h.run(goal))
    return 0


def cmd_plan_memory(a) -> int:
    from .config import get_model_config
    from .runtime.memory_planner import MemoryPlanner

    if a.hf_config:
        _print(MemoryPlanner.estimate_hf_model(json.loads(Path(a.hf_config).read_text()), a.batch_size, a.seq_len, a.training, a.vram_gb, a.quantization))
    else:
        cfg = {**get_model_config(a.model).to_dict(), "batch_size": a.batch_size, "seq_len": a.seq_len, "gradient_checkpointing": a.checkpointing}
        _print(MemoryPlanner.estimate_vram(cfg, available_vram_gb=a.vram_gb, training=a.training).to_dict())
    return 0


def cmd_cache(a) -> int:
    from .runtime.disk_streaming import build_nvfp4_disk_cache, describe_cache

    if a.action == "build":
        _print(build_nvfp4_disk_cache(a.source, a.cache_dir, hadamard=a.hadamard, device=str(_device(a.device))))
    else:
        _print(describe_cache(a.cache_dir))
    return 0


def cmd_native(a) -> int:
    from . import _build

    _build.build_all(force=a.force, verbose=a.verbose)
    print("built", _build.EXT_SO, _build.CORE_SO, _build.NOALLOC_SO)
    return 0


def cmd_profile(a) -> int:
    from .profiling import profile_model

    print(profile_model(checkpoint_path=a.checkpoint, preset=a.model, output_path=a.output, batch_size=a.batch_size, seq_len=a.seq_len,
                        warmup_steps=a.warmup, active_steps=a.steps))
    return 0


def cmd_tokenizer(a) -> int:
    from .data.tokenizer import build_tokenizer, load_tokenizer

    if a.action == "train":
        texts = None
        if a.corpus:
            texts = (l for f in a.corpus for l in Path(f).read_text(encoding="utf-8", errors="replace").splitlines() if l.strip())
        tok = build_tokenizer(a.output, texts=texts, vocab_size=a.vocab_size)
        _print({"saved_to": a.output, "vocab_size": tok.get_vocab_size()})
    else:
        tok = load_tokenizer(a.path)
        ids = tok.encode(a.text)
        ids = list(getattr(ids, "ids", ids))
        _print({"ids": ids, "count": len(ids), "decoded": tok.decode(ids)})
    return 0


def cmd_sandbox(a) -> int:
    from .runtime.sandbox import PythonSandbox

    code = Path(a.file).read_text() if a.file else sys.stdin.read()
    out = PythonSandbox(a.timeout, a.memory_mb).execute_code(code)
    _print(out)
    return 0 if out["success"] else 1


def cmd_rescue(a) -> int:
    """Continuation training that makes loss monotone in exit depth again; writes the repaired checkpoint and a report."""
    import torch

    from .trainer import checkpoint as ckpt
    from .trainer.rescue import load_documents, pack_blocks, rescue_checkpoint

    st = _load_for_inference(a)
    model, tok = st.model, st.tokenizer
    if not hasattr(model, "exit_losses"):
        print("rescue needs a model with early exits (the Triune transformer family)", file=sys.stderr)
        return 2
    sep = getattr(tok, "sep_token_id", None)
    val_docs = load_documents(a.data, tok, a.val_docs + (0 if a.train_data else a.train_docs))
    if a.train_data:
        train_docs = load_documents(a.train_data, tok, a.train_docs)
    else:  # one corpus: the first documents are held out, the rest train
        val_docs, train_docs = val_docs[: a.val_docs], val_docs[a.val_docs:]
    train, val = pack_blocks(train_docs, a.seq_len, sep), pack_blocks(val_docs, a.seq_len, sep)
    if len(val) == 0 or len(train) < a.batch_size:
        print(f"not enough data: {len(train)} training and {len(val)} validation blocks of {a.seq_len} tokens", file=sys.stderr)
        return 2
    model.float() if st.device.type == "cpu" else None
    rep = rescue_checkpoint(model, train, val, a.deepen_steps, a.align_steps, a.joint_steps, a.lr, a.batch_size, a.accum,
                            eval_every=a.eval_every, log=lambda m: print(f"[rescue] {m}", flush=True))
    cfg = model.cfg.to_dict() if hasattr(getattr(model, "cfg", None), "to_dict") else {}
    cfg.update(rep["config_update"])
    ckpt.save_checkpoint(a.out, model=model, step=int(st.config.get("step", 0)), loss=rep["after"]["cortex"]["loss"], config=cfg)
    if a.report:
        Path(a.report).parent.mkdir(parents=True, exist_ok=True)
        Path(a.report).write_text(json.dumps(rep, indent=2, default=str))
    _print({"checkpoint": a.out, "before": rep["before"], "after": rep["after"], "monotone": rep["after"]["monotone"]})
    return 0


def cmd_eval(a) -> int:
    from .evals import mqar

    argv = ["--seq", *[str(t) for t in a.seq], "--dim", str(a.dim), "--heads", str(a.heads), "--batch", str(a.batch)]
    if a.device:
        argv += ["--device", a.device]
    return mqar.main(argv)


def cmd_plugin(a) -> int:
    from .plugins.registry import PluginError, PluginRegistry, create_plugin, write_manifest

    try:
        if a.action == "create":
            _print({"created": str(create_plugin(a.dir, a.name, a.key))})
        elif a.action == "sign":
            _print(write_manifest(Path(a.dir) / a.name if a.name else a.dir, a.key))
        else:  # list / verify
            reg = PluginRegistry(a.key)
            found = reg.discover(a.dir)
            if a.action == "verify":
                for info in found:
                    reg.verify(info)
            _print({"plugins": reg.list(), "verified": a.action == "verify"})
    except PluginError as e:
        print(f"plugin error: {e}", file=sys.stderr)
        return 1
    return 0


def cmd_desktop(a) -> int:
    from .desktop import launch_desktop_app

    launch_desktop_app(a.port, use_browser=not a.no_browser, host=a.host, model=a.model, static_dir=a.static_dir,
                       precision=a.precision, allow_wsl=a.allow_wsl)
    return 0


def cmd_install(a) -> int:
    from . import installer

    if a.scripts:
        _print(installer.write_bootstrap_scripts(Path(a.scripts)))
        return 0
    out = installer.install(a.venv, a.find_links, a.offline, not a.no_build, not a.no_shortcuts, not a.no_extras, a.dry_run)
    if a.json:
        _print(out)
    return 0 if out["ok"] else 1


def cmd_uninstall(a) -> int:
    from . import installer

    _print(installer.uninstall(a.venv, a.dist, a.dry_run))
    return 0


def cmd_package(a) -> int:
    from .packaging import build_native_targets

    _print(build_native_targets(a.target, out_dir=Path(a.out) if a.out else None))
    return 0


# ---------------------------------------------------------------------------------------------------- parser
def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="triune_b200", description="Triune on B200: training, serving and model tools")
    sub = p.add_subparsers(dest="command", required=True)

    def model_args(sp, default="triune-base"):
        sp.add_argument("--model", default=default, help="preset, checkpoint path, JSON config or registered architecture")
        sp.add_argument("--tokenizer", default=None)
        sp.add_argument("--device", default=None)
        sp.add_argument("--precision", default=None, choices=[None, "bf16", "fp8", "fp4", "nvfp4"])

    def gen_args(sp):
        sp.add_argument("--max-tokens", type=int, default=256)
        sp.add_argument("--temperature", type=float, default=0.7)
        sp.add_argument("--top-k", type=int, default=50)
        sp.add_argument("--depth", type=int, default=2, choices=[0, 1, 2])
        sp.add_argument("--speculative", action="store_true")

    s = sub.add_parser("serve", help="start the HTTP API")
    model_args(s, default=None)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--static-dir", default=None)
    s.set_defaults(fn=cmd_serve)

    s = sub.add_parser("chat", help="interactive chat in the terminal")
    model_args(s)
    gen_args(s)
    s.set_defaults(fn=cmd_chat)

    s = sub.add_parser("infer", help="one-shot generation")
    model_args(s)
    gen_args(s)
    s.add_argument("--prompt", default=None)
    s.add_argument("--raw", action="store_true", help="do not wrap the prompt in the chat template")
    s.add_argument("--json", action="store_true")
    s.set_defaults(fn=cmd_infer)

    s = sub.add_parser("scan", help="find models on this machine (checkpoints, HF caches, GGUF, Ollama, adapters)")
    s.add_argument("paths", nargs="*")
    s.add_argument("--depth", type=int, default=4)
    s.set_defaults(fn=cmd_scan)

    s = sub.add_parser("transmute", help="convert a Hugging Face causal LM (attach exits, or build a native Triune student)")
    s.add_argument("source")
    s.add_argument("--mode", choices=["exits", "native"], default="exits")
    s.add_argument("--reflex-ratio", type=float, default=0.25)
    s.add_argument("--rank", type=int, default=64)
    s.add_argument("--no-jev", action="store_true")
    s.add_argument("--experts", type=int, default=8)
    s.add_argument("--top-k", type=int, default=2)
    s.add_argument("--layers", type=int, default=None)
    s.add_argument("--dim", type=int, default=None)
    s.add_argument("--online", action="store_true")
    s.add_argument("--device", default=None)
    s.add_argument("--output", default=None)
    s.set_defaults(fn=cmd_transmute)

    s = sub.add_parser("finetune", help="LoRA / QLoRA fine-tuning")
    model_args(s)
    s.add_argument("--data", required=True)
    s.add_argument("--output", default="adapters/latest")
    s.add_argument("--rank", type=int, default=16)
    s.add_argument("--alpha", type=float, default=32.0)
    s.add_argument("--dropout", type=float, default=0.05)
    s.add_argument("--qlora", action="store_true")
    s.add_argument("--epochs", type=int, default=1)
    s.add_argument("--batch-size", type=int, default=4)
    s.add_argument("--lr", type=float, default=2e-4)
    s.add_argument("--seq-len", type=int, default=512)
    s.add_argument("--max-steps", type=int, default=None)
    s.set_defaults(fn=cmd_finetune)

    s = sub.add_parser("adapter", help="manage LoRA adapters")
    s.add_argument("action", choices=["list", "merge", "export"])
    s.add_argument("--dirs", nargs="*")
    s.add_argument("--base", default="triune-base")
    s.add_argument("--adapter", default="adapters/latest")
    s.add_argument("--output", default=None)
    s.add_argument("--format", default="safetensors")
    s.set_defaults(fn=cmd_adapter)

    for name in ("checkpoint", "export"):
        s = sub.add_parser(name, help="list checkpoints / export a model" if name == "checkpoint" else "export a model")
        if name == "checkpoint":
            s.add_argument("action", choices=["list", "export", "merge"],
                           help="merge: assemble the rank-local shard files of --dir into one canonical checkpoint (--output)")
            s.add_argument("--dir", default="checkpoints_full")
        s.add_argument("--model", default="checkpoints_full/latest.pt")
        s.add_argument("--output", default="exports/model.safetensors")
        s.add_argument("--format", default="safetensors", choices=["safetensors", "hf", "huggingface", "onnx", "gguf", "pt", "lora"])
        s.set_defaults(fn=cmd_checkpoint if name == "checkpoint" else cmd_export)

    sub.add_parser("models", help="list the preset zoo").set_defaults(fn=cmd_models)

    s = sub.add_parser("train", help="pre-training loop (launch under torchrun for several GPUs)")
    s.add_argument("--model", default="triune-base")
    s.add_argument("--overrides", default=None, help="JSON dict of model overrides")
    s.add_argument("--data", default=None, help="local .jsonl/.parquet/.txt file or HF dataset name; synthetic tokens if omitted")
    s.add_argument("--tokenizer", default="triune_tokenizer.json")
    s.add_argument("--batch-size", type=int, default=16)
    s.add_argument("--seq-len", type=int, default=2048)
    s.add_argument("--steps", type=int, default=100)
    s.add_argument("--lr", type=float, default=3e-4)
    s.add_argument("--grad-accum", type=int, default=1)
    s.add_argument("--depth-mode", default="cortex", choices=["cortex", "joint", "dynamic"])
    s.add_argument("--dp-mode", default="fused", choices=["fused", "nccl"])
    s.add_argument("--no-cuda-graph", dest="cuda_graph", action="store_false")
    s.add_argument("--checkpoint-dir", default="checkpoints_full")
    s.add_argument("--resume", default=None)
    s.add_argument("--save", action="store_true")
    s.add_argument("--log-every", type=int, default=10)
    s.add_argument("--plan", action="store_true", help="check the memory budget before starting")
    s.add_argument("--force", action="store_true")
    s.add_argument("--auto_fit", "--auto-fit", dest="auto_fit", action="store_true")
    s.set_defaults(fn=cmd_train)

    s = sub.add_parser("bench", aliases=["benchmark"], help="run the headline benchmark or a kernel micro-benchmark")
    s.add_argument("--gpus", type=int, default=1)
    s.add_argument("--steps", type=int, default=10)
    s.add_argument("--warmup", type=int, default=3)
    s.add_argument("--kernels", default=None, help="bench_kernels case: gemm | wgrad | gla | rmsnorm | ce | fp8 | nvfp4 | all")
    s.set_defaults(fn=cmd_bench)

    sub.add_parser("gpucheck", help="device, driver and kernel diagnostics").set_defaults(fn=cmd_gpucheck)
    sub.add_parser("doctor", aliases=["info"], help="health of the whole installation: runtime, devices, kernels, zoo, server extras, local state").set_defaults(fn=cmd_doctor)

    s = sub.add_parser("agent", help="run a goal through the tool-using agent loop on a local model")
    model_args(s, default="triune-nano")
    s.add_argument("goal_pos", nargs="?", default=None, help="the goal (or use --goal)")
    s.add_argument("-g", "--goal", default=None)
    s.add_argument("--persona", default="auto", help="auto (by the goal), architect, engineer, researcher, debugger, optimizer, tutor, sentinel, "
                   "or 'name=system prompt' for one defined on the spot")
    s.add_argument("--workspace", default=".", help="directory the file tools are confined to")
    s.add_argument("--allow-shell", action="store_true", help="offer a shell tool inside the workspace")
    s.add_argument("--no-auto-skill", action="store_true", help="do not write successful tool sequences down as skills")
    s.add_argument("--team", default=None, help="comma-separated personas that take the goal in turn, each seeing the previous answer")
    s.add_argument("--max-steps", type=int, default=3, help="tool rounds per goal")
    s.add_argument("--max-tokens", type=int, default=128)
    s.add_argument("--read-only", action="store_true", help="leave out the tools that write files")
    s.add_argument("--store-dir", default="checkpoints/agent_harness", help="persistent memory and skills")
    s.set_defaults(fn=cmd_agent)

    s = sub.add_parser("plan-memory", help="estimate the memory budget of a run")
    s.add_argument("--model", default="triune-base")
    s.add_argument("--hf-config", default=None)
    s.add_argument("--batch-size", type=int, default=16)
    s.add_argument("--seq-len", type=int, default=2048)
    s.add_argument("--vram-gb", type=float, default=None)
    s.add_argument("--inference", dest="training", action="store_false")
    s.add_argument("--checkpointing", action="store_true")
    s.add_argument("--quantization", default=None)
    s.set_defaults(fn=cmd_plan_memory)

    s = sub.add_parser("cache", aliases=["cache-nvfp4"], help="NVFP4 disk cache of a Hugging Face checkpoint")
    s.add_argument("action", choices=["build", "info"])
    s.add_argument("--source", default=None)
    s.add_argument("--cache-dir", required=True)
    s.add_argument("--hadamard", action="store_true")
    s.add_argument("--device", default=None)
    s.set_defaults(fn=cmd_cache)

    s = sub.add_parser("native", help="build the CUDA extension and the C libraries in tree")
    s.add_argument("--force", action="store_true")
    s.add_argument("-v", "--verbose", action="store_true")
    s.set_defaults(fn=cmd_native)

    s = sub.add_parser("profile", help="profile training steps")
    s.add_argument("--model", default="triune-base")
    s.add_argument("--checkpoint", default="checkpoints_full/latest.pt")
    s.add_argument("--output", default="profiler_output.txt")
    s.add_argument("--batch-size", type=int, default=4)
    s.add_argument("--seq-len", type=int, default=256)
    s.add_argument("--warmup", type=int, default=5)
    s.add_argument("--steps", type=int, default=10)
    s.set_defaults(fn=cmd_profile)

    s = sub.add_parser("tokenizer", help="train a BPE tokenizer or tokenise text")
    s.add_argument("action", choices=["train", "encode"])
    s.add_argument("--corpus", nargs="*")
    s.add_argument("--output", default="triune_tokenizer.json")
    s.add_argument("--vocab-size", type=int, default=32000)
    s.add_argument("--path", default="triune_tokenizer.json")
    s.add_argument("--text", default="")
    s.set_defaults(fn=cmd_tokenizer)

    s = sub.add_parser("sandbox", help="run Python in the restricted sandbox")
    s.add_argument("--file", default=None)
    s.add_argument("--timeout", type=int, default=10)
    s.add_argument("--memory-mb", type=int, default=256)
    s.set_defaults(fn=cmd_sandbox)

    s = sub.add_parser("rescue", help="continuation training that repairs a starved deep exit (deepen, align, joint)")
    model_args(s)
    s.add_argument("--data", required=True, help=".jsonl (text field) or plain text; validation comes from here")
    s.add_argument("--train-data", default=None, help="separate training corpus (default: the rest of --data)")
    s.add_argument("--out", required=True, help="where to write the repaired checkpoint")
    s.add_argument("--report", default=None, help="optional JSON report path")
    s.add_argument("--train-docs", type=int, default=7500)
    s.add_argument("--val-docs", type=int, default=500)
    s.add_argument("--seq-len", type=int, default=512)
    s.add_argument("--batch-size", type=int, default=8)
    s.add_argument("--accum", type=int, default=1)
    s.add_argument("--deepen-steps", type=int, default=3500)
    s.add_argument("--align-steps", type=int, default=300)
    s.add_argument("--joint-steps", type=int, default=500)
    s.add_argument("--lr", type=float, default=1e-4)
    s.add_argument("--eval-every", type=int, default=0)
    s.set_defaults(fn=cmd_rescue)

    s = sub.add_parser("eval", help="task evaluations of the sequence mixers (associative recall)")
    s.add_argument("task", choices=["mqar"])
    s.add_argument("--seq", type=int, nargs="+", default=[256, 512, 1024, 2048])
    s.add_argument("--dim", type=int, default=256)
    s.add_argument("--heads", type=int, default=4)
    s.add_argument("--batch", type=int, default=8)
    s.add_argument("--device", default=None)
    s.set_defaults(fn=cmd_eval)

    s = sub.add_parser("plugin", help="scaffold, sign, list or verify DAG plugins")
    s.add_argument("action", choices=["create", "sign", "list", "verify"])
    s.add_argument("--dir", default="plugins", help="directory that holds the plugin directories")
    s.add_argument("--name", default=None, help="plugin name (create / sign)")
    s.add_argument("--key", default=None, help="signing key (default: TRIUNE_PLUGIN_KEY)")
    s.set_defaults(fn=cmd_plugin)

    s = sub.add_parser("desktop", aliases=["studio"], help="start (or reuse) the local server and open its page in the browser")
    model_args(s, default=None)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--static-dir", default=None)
    s.add_argument("--no-browser", action="store_true", help="do not open a browser; print the address only")
    s.add_argument("--allow-wsl", action="store_true", help="on a Windows host without a CUDA PyTorch, run the server inside WSL 2")
    s.set_defaults(fn=cmd_desktop)

    s = sub.add_parser("install", help="set the framework up on this machine (virtual environment, dependencies, kernels, launcher)")
    s.add_argument("--venv", default=None, help="virtual environment to create or reuse (default: the current interpreter)")
    s.add_argument("--find-links", default=None, help="directory of wheels to install from")
    s.add_argument("--offline", action="store_true", help="never contact a package index")
    s.add_argument("--no-build", action="store_true", help="do not compile the CUDA extensions")
    s.add_argument("--no-shortcuts", action="store_true", help="do not generate the launcher bundle")
    s.add_argument("--no-extras", action="store_true", help="skip the optional packages (tokenizers, safetensors, pyarrow, transformers)")
    s.add_argument("--dry-run", action="store_true", help="print the plan and change nothing")
    s.add_argument("--json", action="store_true", help="print the record of the run as JSON")
    s.add_argument("--scripts", default=None, help="only write install.sh / install.bat into this directory")
    s.set_defaults(fn=cmd_install)

    s = sub.add_parser("uninstall", help="remove the virtual environment and the generated launcher bundles")
    s.add_argument("--venv", required=True)
    s.add_argument("--dist", default=None)
    s.add_argument("--dry-run", action="store_true")
    s.set_defaults(fn=cmd_uninstall)

    s = sub.add_parser("package", aliases=["build-native"], help="generate launcher bundles (Linux AppDir, macOS .app, Windows .cmd)")
    s.add_argument("--target", default="all", help="linux, macos, windows or all")
    s.add_argument("--out", default=None, help="output directory (default: dist/ in the source tree)")
    s.set_defaults(fn=cmd_package)
    return p


build_cli_parser = build_parser  # the reference's name (``triune/cli.py``)


def main(argv: Optional[List[str]] = None) -> int:
    from . import cli_ui

    cli_ui.ensure_utf8_stdio()
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv in (["-h"], ["--help"], ["help"]):  # the grouped overview; each command's -h lists its options
        cli_ui.render_help_overview()
        return 0
    args = build_parser().parse_args(argv)
    return int(args.fn(args) or 0)


if __name__ == "__main__":
    sys.exit(main())
