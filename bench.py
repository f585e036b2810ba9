"""Flagship benchmark: training tokens/s of the 90.8M-class MoE-GLA TriuneTransformer, bf16, data parallel.

Contract: ``python bench.py --gpus N --steps K --warmup W`` (under torchrun for N > 1) prints ONE JSON line from
rank 0. ``value`` is the whole-job tokens/s from a device-timed loop (CUDA events, max over ranks); ``e2e`` is
the same metric through the public ``Trainer.train_step`` API including the pinned host->device copy of every
batch and the device->host read of every loss. ``prefill`` is the serving half of the metric: tokens/s of a 4 x 16384 prefill through the public
forward, as N independent replicas for N > 1. ``wait_status`` is the status word of the fused data-parallel kernels
(0 = every bounded wait completed). ``--impl reference`` runs the unmodified reference project (installed under
``baseline/_ref``) on the same config.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
BASELINE_TOK_S = 9560.0  # reference's published pre-training number (RTX 5070 Laptop, B=4, T=256)
BATCH, SEQ, VOCAB = 16, 2048, 32000
PREFILL_BATCH, PREFILL_SEQ = 4, 16384  # the serving half of the metric: prefill tok/s at T = 16K


def timed_prefill(fn, iters: int = 5, warmup: int = 3) -> float:
    """Milliseconds per call of ``fn`` (CUDA events on the current stream, after warm-up, synchronised on both sides).
    The 4 x 16384 inputs and their activations are far larger than the 126 MB L2, so no explicit flush."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []
        self._nvml = None      # (module, handle) when the NVML binding is importable: 20 ms sampling from a thread
        self._samples = []
        self._stop = threading.Event()

    def _nvml_loop(self):
        nv, h = self._nvml
        while not self._stop.is_set():
            try:
                self._samples.append((nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                                      int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))))
            except Exception:
                break
            self._stop.wait(0.02)

    def start(self):
        try:  # read-only NVML queries; a short timed region still gets several samples
            import pynvml as nv

            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.idx)
            self._max = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            self._nvml = (nv, h)
            self.thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self._nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self._nvml is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            sm = [c for c, _ in self._samples]
            bits = 0
            for _, r in self._samples:
                bits |= r
            names = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(self._max), "sm_min_mhz": min(sm) if sm else None,
                    "reasons": sorted(n for n, b in names if bits & b), "samples": len(sm), "source": "nvml, 20 ms"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def barrier_sync():
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()


def run_ours(args):
    from triune_b200 import ops
    from triune_b200.config import get_model_config
    from triune_b200.data import SyntheticTokenSource
    from triune_b200.models import TriuneTransformer
    from triune_b200.optim import CentroidSteerOptimizer
    from triune_b200.parallel import max_over_ranks, setup_distributed
    from triune_b200.parallel.data_parallel import ShardedDataParallel
    from triune_b200.trainer import Trainer
    from triune_b200.utils import place_model

    ctx = setup_distributed()
    dev = ctx.device
    torch.manual_seed(0)
    cfg = get_model_config("bench-90m")
    model = place_model(TriuneTransformer.from_config(cfg), dev, torch.bfloat16)
    # constant learning rate 3e-4, as the reference arm uses, so the two final losses are comparable
    run_cfg = {"lr": 3e-4, "min_lr": 3e-4, "warmup_steps": 0, "total_steps": 100000, "depth_mode": "cortex",
               "grad_accum_steps": 1, "grad_clip": 1.0, "vocab_size": VOCAB, "ns_steps": 5,
               "cuda_graph": (not args.no_graph) and (ctx.world_size == 1 or args.dp_mode == "fused")}
    dp, opt = None, None
    if ctx.world_size > 1:
        try:
            dp = ShardedDataParallel(ctx, mode=args.dp_mode)
            opt = CentroidSteerOptimizer(model, lr=3e-4, muon_ns_steps=5, grad_clip=1.0, storage_factory=dp.storage_factory)
        except Exception as e:  # no peer-mapped memory on this box: fall back to the NCCL all-reduce path, eagerly
            if args.dp_mode != "fused":
                raise
            print(f"[bench] fused NVLink DP unavailable ({type(e).__name__}: {e}); using --dp-mode nccl", file=sys.stderr, flush=True)
            args.dp_mode, run_cfg["cuda_graph"] = "nccl", False
            dp = ShardedDataParallel(ctx, mode="nccl")
            opt = None
    if opt is None:
        opt = CentroidSteerOptimizer(model, lr=3e-4, muon_ns_steps=5, grad_clip=1.0)
    trainer = Trainer(model, run_cfg, optimizer=opt, device=dev, dp=dp)
    src = SyntheticTokenSource(VOCAB, BATCH, SEQ, seed=1234 + ctx.rank, pin=True, pool=4)
    tokens_per_step = BATCH * SEQ * ctx.world_size

    # ---- device-timed loop: batches resident on the device, no host reads inside ----
    dev_batches = [tuple(t.to(dev) for t in next(src)) for _ in range(4)]

    def dev_step(i):
        x, y = dev_batches[i % len(dev_batches)]
        return trainer.step_on_device(x, y, x.numel())

    # W warm-up steps, plus (graph mode) enough extra untimed steps for every step kind to have been captured:
    # the CentroidSteer tier refreshes its steering axis every 10th step and that kind has its own graph.
    priming = 0
    for i in range(args.warmup):
        dev_step(i)
    if run_cfg["cuda_graph"]:
        while priming < 24 and (trainer.graph_engine.captures < 2 or opt.step_kind() != "plain"):
            dev_step(args.warmup + priming)
            priming += 1
    barrier_sync()
    sampler = ClockSampler(ctx.local_rank)
    if ctx.rank == 0:
        sampler.start()
    ops.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = None
    for i in range(args.steps):
        last = dev_step(i)
    e1.record()
    barrier_sync()
    ms = max_over_ranks(e0.elapsed_time(e1), dev) / args.steps
    launches = ops.launch_count()
    clocks = sampler.stop() if ctx.rank == 0 else None
    final_loss = float(last)

    # ---- end-to-end loop through the public API: pinned H2D each step + loss D2H each step ----
    for _ in range(2):
        x, y = next(src)
        trainer.train_step(x, y)
    barrier_sync()
    h0, d0 = trainer.h2d_bytes, trainer.d2h_bytes
    t0 = time.perf_counter()
    for _ in range(args.steps):
        x, y = next(src)
        loss = trainer.train_step(x, y)
    barrier_sync()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, dev) / args.steps
    h2d = (trainer.h2d_bytes - h0) // args.steps
    d2h = (trainer.d2h_bytes - d0) // args.steps

    # ---- status word of the fused data-parallel kernels: a bounded wait that expired would have skipped a reduction
    # (and shortened the step), so a non-zero word invalidates the run. One device->host read, outside the timed loops.
    wait_status = 0
    fused = getattr(dp, "_fused", None) if dp is not None else None
    if fused is not None:
        wait_status = int(fused.check())
    wait_status = int(max_over_ranks(float(wait_status), dev))

    # ---- prefill tok/s at T = 16K through the public forward (recurrent cache, last-token logits); N > 1 runs N
    # independent replicas and reports the whole-job rate from the slowest rank ----
    prefill = None
    if not args.no_prefill:
        del dev_batches
        torch.cuda.empty_cache()
        model.eval()
        pg = torch.Generator(device=dev).manual_seed(99 + ctx.rank)
        pids = torch.randint(0, VOCAB, (PREFILL_BATCH, PREFILL_SEQ), device=dev, generator=pg)

        @torch.no_grad()
        def prefill_once():
            return model(pids, force_depth=2, cache=model.init_cache(PREFILL_BATCH), last_token_only=True)

        ops.reset_launch_count()
        prefill_once()
        p_launches = ops.launch_count()
        barrier_sync()
        p_ms = max_over_ranks(timed_prefill(prefill_once), dev)
        prefill = {"tok_s": PREFILL_BATCH * PREFILL_SEQ * ctx.world_size / (p_ms / 1e3), "ms": p_ms,
                   "batch": PREFILL_BATCH, "seq": PREFILL_SEQ, "dtype": "bf16", "variant": "bf16",
                   "layout": f"{ctx.world_size} independent replica(s)", "gpu_launches": p_launches}

    if ctx.rank == 0:
        value = tokens_per_step / (ms / 1e3)
        out = {
            "metric": "train tok/s (device-timed, max over ranks)", "value": value, "unit": "tok/s",
            "n_gpus": ctx.world_size, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": value / BASELINE_TOK_S, "dtype": "bf16",
            "data": "synthetic uniform-random token ids, random-init N(0,0.02) weights",
            "config": {"model": f"TriuneTransformer 90.8M-class MoE-GLA ({model.num_parameters()} params: 8L d384 6x64 "
                                "GLA heads, E=8 top-2 + shared, hidden 1536, exits 2/5/8)",
                       "global_batch": BATCH * ctx.world_size, "seq_len": SEQ,
                       "parallelism": f"dp{ctx.world_size}" + (f" ({args.dp_mode})" if ctx.world_size > 1 else ""),
                       "optimizer": "CentroidSteer (Muon NS 5 iters + triangular core + AdamW)",
                       "cuda_graph": bool(run_cfg["cuda_graph"]), "graph_priming_steps": priming,
                       "l2": "per-step working set (GBs of activations) far exceeds the 126 MB L2; no explicit flush"},
            "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tok/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "prefill": prefill, "wait_status": wait_status,
            "final_loss": final_loss, "impl": "triune_b200",
        }
        print(json.dumps(out), flush=True)
    from triune_b200.parallel import cleanup_distributed

    cleanup_distributed()


def run_reference(args):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "triune")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}))
        return
    try:
        sys.path.insert(0, ref_dir)
        import triune.model.config as rc  # the reference's module constants are its configuration surface

        rc.TOP_K_EXPERTS = 2
        rc.EXPERT_HIDDEN_MULTIPLIER = 4
        from triune.kernels.fast_cross_entropy import fast_cross_entropy
        from triune.model.transformer import TriuneTransformer as RefModel
        from triune.optim.centroid import CentroidSteerOptimizer as RefOpt
        import triune.model.moe as rmoe
        import triune.model.attention as ratt

        # the named config: expert hidden 1536 = 4 * d, top-2 (module-level constants of the reference)
        rmoe.EXPERT_HIDDEN_MULTIPLIER = 4
        rmoe.TOP_K_EXPERTS = 2
    except Exception as e:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"[:300]}))
        return
    import torch.distributed as dist

    rank, local, world = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    model = RefModel(vocab_size=VOCAB, hidden_dim=384, num_layers=8, num_heads=6, head_dim=64, num_experts=8,
                     router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=5).to(device=dev, dtype=torch.bfloat16)
    for m in model.modules():
        if isinstance(m, rmoe.MoE_FFN):
            m.top_k = 2
    nparams = sum(p.numel() for p in {id(p): p for p in model.parameters()}.values())
    opt = RefOpt(model, lr=3e-4, muon_ns_steps=5)
    train_model = model
    if world > 1:
        from triune.trainer.distributed import wrap_distributed_model, setup_distributed as ref_setup

        train_model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], find_unused_parameters=True,
                                                                broadcast_buffers=False)
    g = torch.Generator().manual_seed(1234 + rank)
    pool = []
    for _ in range(4):
        ids = torch.randint(0, VOCAB, (BATCH, SEQ + 1), generator=g)
        pool.append((ids[:, :-1].contiguous().pin_memory(), ids[:, 1:].contiguous().pin_memory()))
    dev_pool = [(x.to(dev), y.to(dev)) for x, y in pool]
    moes = [m for m in model.modules() if isinstance(m, rmoe.MoE_FFN)]

    def step(x, y):
        train_model.train()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits, _ = train_model(x, force_depth=2)
            loss = fast_cross_entropy(logits.reshape(-1, logits.shape[-1]), y.reshape(-1))
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        for m in moes:
            m.step_bias()
        return loss

    try:
        for i in range(args.warmup):
            step(*dev_pool[i % 4])
        barrier_sync()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            loss = step(*dev_pool[i % 4])
        e1.record()
        barrier_sync()
        ms = e0.elapsed_time(e1) / args.steps
        clocks = sampler.stop() if rank == 0 else None
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        t0 = time.perf_counter()
        for i in range(args.steps):
            x, y = pool[i % 4]
            lv = float(step(x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)).item())
        barrier_sync()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    except Exception as e:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"run failed: {type(e).__name__}: {e}"[:300]}))
        return
    # The same step through the reference's own Trainer / TrainingEngine.step_once in cortex mode (its data prefetcher,
    # its sub-batch slicing, its loss bookkeeping). The faster of the two loops is the reference's number.
    engine_ms, engine_note = None, None
    # With "both" the engine loop is only taken on one GPU: it is nine times slower than the hand-written loop there
    # (eight 4096-token sub-batches per step), so it cannot be the faster one, and under DDP every sub-batch backward
    # is one more gradient all-reduce.
    if args.ref_loop == "engine" or (args.ref_loop == "both" and world == 1):
        try:
            engine_ms = _reference_engine_loop(args, train_model, opt, pool, dev, rank, world)
        except Exception as e:
            engine_note = f"{type(e).__name__}: {e}"[:200]
    loops = {"manual": ms, "engine": engine_ms}
    ref_loop = "manual"
    if engine_ms is not None and (args.ref_loop == "engine" or engine_ms < ms):
        ref_loop = "engine"
        ms = engine_ms
        e2e_ms = min(e2e_ms, engine_ms) if args.ref_loop == "both" else engine_ms  # the engine loop is end to end by construction
    prefill = None
    if not args.no_prefill:
        try:  # the reference's own forward: recurrent cache, last-token logits, bf16 autocast as its scripts use
            del dev_pool
            opt.zero_grad(set_to_none=True)
            torch.cuda.empty_cache()
            model.eval()
            pg = torch.Generator(device=dev).manual_seed(99 + rank)
            pids = torch.randint(0, VOCAB, (PREFILL_BATCH, PREFILL_SEQ), device=dev, generator=pg)

            @torch.no_grad()
            def prefill_once():
                cache = model.init_cache(PREFILL_BATCH)
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    return model(pids, force_depth=2, cache=cache, last_token_only=True)

            barrier_sync()
            p_ms = timed_prefill(prefill_once)
            t = torch.tensor([p_ms], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            p_ms = float(t.item())
            prefill = {"tok_s": PREFILL_BATCH * PREFILL_SEQ * world / (p_ms / 1e3), "ms": p_ms, "batch": PREFILL_BATCH,
                       "seq": PREFILL_SEQ, "dtype": "bf16", "variant": "bf16",
                       "layout": f"{world} independent replica(s)"}
        except Exception as e:
            prefill = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    if rank == 0:
        tps = BATCH * SEQ * world
        value = tps / (ms / 1e3)
        print(json.dumps({
            "metric": "train tok/s (device-timed, max over ranks)", "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / BASELINE_TOK_S, "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
            "config": {"model": f"reference TriuneTransformer ({nparams} params; 8L d384 6x64 heads E=8 top-2 hidden 1536)",
                       "global_batch": BATCH * world, "seq_len": SEQ, "parallelism": f"dp{world} (DDP/NCCL)",
                       "has_fla": bool(getattr(ratt, "HAS_FLA", False)), "lr": "constant 3e-4", "ref_loop": ref_loop,
                       "ref_loop_ms": loops, "ref_engine_note": engine_note},
            "clocks": clocks, "e2e": {"value": tps / (e2e_ms / 1e3), "unit": "tok/s", "ms_per_step": e2e_ms,
                                      "h2d_bytes_per_step": BATCH * SEQ * 16, "d2h_bytes_per_step": 4},
            "prefill": prefill, "final_loss": lv, "impl": "reference"}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _reference_engine_loop(args, train_model, opt, pool, dev, rank, world):
    """ms per step of ``TrainingEngine.step_once`` (the reference's public training step) over the same batches."""
    import torch.distributed as dist
    from triune.trainer.trainer import Trainer as RefTrainer

    class _Tok:
        def get_vocab_size(self):
            return VOCAB

        def token_to_id(self, t):
            return {"[PAD]": 0, "[SEP]": 1}.get(t)

    cfg = {"vocab_size": VOCAB, "grad_accum_steps": 1, "target_depth_dist": [0.2, 0.3, 0.5], "exploration": "none",
           "exploration_steps": 0, "eval_batches": 1, "cuda_graph": False, "lr": 3e-4, "min_lr": 3e-4, "warmup_steps": 0,
           "total_steps": 100000, "depth_mode": "cortex", "grad_clip": 1.0, "balance_coef": 0.3}
    tr = RefTrainer(model=train_model, optimizer=opt, train_loader=list(pool), eval_loader=list(pool[:1]), tokenizer=_Tok(),
                    config=cfg, device=dev)
    for _ in range(args.warmup):
        tr.engine.step_once(advance_step=True)
    barrier_sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        tr.engine.step_once(advance_step=True)
    e1.record()
    barrier_sync()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="run every step eagerly (no CUDA-graph replay)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill (T = 16K) measurement after the training loops")
    ap.add_argument("--dp-mode", default=os.environ.get("TRIUNE_DP_MODE", "fused"), choices=["nccl", "fused"])
    ap.add_argument("--ref-loop", default="both", choices=["manual", "engine", "both"],
                    help="reference arm: hand-written full-batch step, the reference's TrainingEngine.step_once, or both "
                         "(the faster one is reported)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return
    if args.impl == "reference":
        run_reference(args)
        return
    try:
        run_ours(args)
    except Exception as e:  # a failed graph capture must not cost the measurement: rerun eagerly in a fresh process
        if args.no_graph or int(os.environ.get("WORLD_SIZE", "1")) > 1:
            raise
        print(f"[bench] graph path failed ({type(e).__name__}: {e}); re-running with --no-graph", file=sys.stderr, flush=True)
        os.execv(sys.executable, [sys.executable] + sys.argv + ["--no-graph"])


if __name__ == "__main__":
    main()
