"""Latency of the three exits and throughput with the depth router in charge.

For one batch shape: the forward pass forced to each exit (Reflex, Limbic, Cortex), then the same batch with the
router deciding per sequence (``force_depth=None``), with the distribution of depths it chose; optionally with the
confidence policy (``exit_policy="calm"``) at a threshold. Device-timed with CUDA events on a GPU (median after
warm-up, L2 flushed between calls), wall clock on the CPU. Same measurement as the reference's
``scripts/benchmark_dynamic_exits.py`` (published on its laptop GPU at V=4096, B=4, T=512: Reflex 7.29 ms,
Cortex 26.76 ms, dynamic 299,506 tok/s).

    python -m triune_b200.evals.dynamic_exits --model bench-90m --vocab 4096 --batch 4 --seq 512
"""

from __future__ import annotations

import argparse
import json
import statistics
import time

import torch


def _timer(device: torch.device, iters: int, warmup: int = 3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if device.type == "cuda" else None

    def timed(fn) -> float:
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(iters):
            if flush is not None:
                flush.fill_(1)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b))
            else:
                t0 = time.perf_counter()
                fn()
                ts.append((time.perf_counter() - t0) * 1e3)
        return statistics.median(ts)

    return timed


@torch.no_grad()
def measure(model, ids: torch.Tensor, iters: int = 10, calm_tau: float = 0.0) -> dict:
    dev = ids.device
    timed = _timer(dev, iters)
    tokens = ids.numel()
    was = model.training
    model.eval()
    out = {"exits": {}}
    try:
        for depth, name in enumerate(("reflex", "limbic", "cortex")):
            ms = timed(lambda: model(ids, force_depth=depth, last_token_only=True))
            out["exits"][name] = {"ms": ms, "tok_s": tokens / ms * 1e3}
        full = out["exits"]["cortex"]["ms"]
        for name in ("reflex", "limbic"):
            out["exits"][name]["speedup_over_cortex"] = full / out["exits"][name]["ms"]
        ms = timed(lambda: model(ids, last_token_only=True))
        choice = getattr(model, "last_depth_choice", None)
        hist = torch.bincount(choice.reshape(-1).long().cpu(), minlength=3).tolist() if choice is not None else None
        out["router"] = {"ms": ms, "tok_s": tokens / ms * 1e3, "sequences_per_depth": hist}
        if calm_tau > 0:
            ms = timed(lambda: model(ids, exit_policy="calm", confidence_threshold=calm_tau))
            out["calm"] = {"tau": calm_tau, "ms": ms, "tok_s": tokens / ms * 1e3, "where_tokens_left": dict(model.last_calm_compaction_stats or {})}
    finally:
        model.train(was)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="exit latencies and router-driven throughput")
    ap.add_argument("--model", default="bench-90m")
    ap.add_argument("--vocab", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--calm-tau", type=float, default=0.0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    from ..config import MODEL_PRESETS, get_model_config
    from ..models import TriuneTransformer
    from ..models.zoo import load_model
    from ..utils import place_model

    dev = torch.device(a.device)
    torch.manual_seed(0)
    if a.model in MODEL_PRESETS:
        cfg = get_model_config(a.model)
        cfg.vocab_size = a.vocab
        model = TriuneTransformer.from_config(cfg)
    else:
        model = load_model(a.model, vocab_size=a.vocab)
    model = place_model(model, dev, torch.bfloat16 if dev.type == "cuda" else torch.float32)
    ids = torch.randint(0, a.vocab, (a.batch, a.seq), device=dev)
    res = measure(model, ids, a.iters, a.calm_tau)
    print(json.dumps({"eval": "dynamic exits", "model": a.model, "vocab": a.vocab, "batch": a.batch, "seq_len": a.seq, "device": str(dev),
                      "parameters": sum(p.numel() for p in model.parameters()), **res}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
