"""Calibration of the confidence exits: choose the margin threshold on one split, check it on another.

The ``calm`` exit policy lets a token leave at the Reflex or Limbic exit when the gap between its two most likely
next tokens there is at least a threshold tau. This evaluation answers what tau buys: for each early exit it collects,
per position, the margin at that exit and whether its arg-max agrees with the full-depth (Cortex) arg-max; on a
*calibration* split it picks the smallest tau on a grid whose agreement among the positions it lets go (by the Wilson
lower bound, so that a handful of lucky positions cannot pass) reaches a target; on a disjoint *held-out* split it
reports what that tau delivers: coverage (share of positions that leave), agreement among them, the share of layer
evaluations saved, the expected calibration error of the margin as a confidence score, its AUROC as a detector of
agreement, and the latency of a forward pass with the policy against the full-depth pass.

Same experiment as the reference's ``benchmarks/calm_calibration.py:119-337`` (collect / calibrate / evaluate / Pareto
sweep / live speed); token sequences come from a local text file through a tokenizer, or are synthetic (a Markov
language, so that early exits of a briefly trained model have something to agree on) when no corpus is given.

    python -m triune_b200.evals.calm --model triune-nano --train-steps 60
    python -m triune_b200.evals.calm --checkpoint ck.pt --corpus data.jsonl --tokenizer tok.json
"""

from __future__ import annotations

import argparse
import json
import math
import time
from typing import Dict, List, Optional

import torch

GRID = [round(0.05 * k, 2) for k in range(1, 20)]
EXITS = ("reflex", "limbic")


def wilson_lower(hits: int, n: int, z: float = 1.96) -> float:
    """Lower end of the Wilson score interval of a proportion: what agreement can be claimed from ``n`` positions."""
    if n == 0:
        return 0.0
    p = hits / n
    den = 1.0 + z * z / n
    centre = p + z * z / (2 * n)
    spread = z * math.sqrt(p * (1 - p) / n + z * z / (4 * n * n))
    return (centre - spread) / den


def auroc(scores: torch.Tensor, labels: torch.Tensor) -> Optional[float]:
    """Probability that a position whose exit agrees has a larger margin than one that does not (ties count half)."""
    pos, neg = int(labels.sum()), int((~labels).sum())
    if pos == 0 or neg == 0:
        return None
    order = torch.argsort(scores)
    s = scores[order]
    ranks = torch.arange(1, len(s) + 1, dtype=torch.float64)
    # average ranks over ties
    uniq, inv, counts = torch.unique_consecutive(s, return_inverse=True, return_counts=True)
    ends = torch.cumsum(counts, 0).double()
    mean_rank = ends - (counts.double() - 1) / 2
    ranks = mean_rank[inv]
    r_pos = ranks[labels[order]].sum()
    return float((r_pos - pos * (pos + 1) / 2) / (pos * neg))


def reliability(scores: torch.Tensor, agree: torch.Tensor, bins: int = 10) -> Dict:
    """Expected calibration error of the margin read as a confidence, with the per-bin table."""
    edges = torch.linspace(0, 1, bins + 1)
    table, ece, n = [], 0.0, len(scores)
    for b in range(bins):
        m = (scores >= edges[b]) & ((scores < edges[b + 1]) if b < bins - 1 else (scores <= edges[b + 1]))
        c = int(m.sum())
        if c == 0:
            continue
        conf, acc = float(scores[m].mean()), float(agree[m].float().mean())
        ece += c / n * abs(conf - acc)
        table.append({"lo": float(edges[b]), "hi": float(edges[b + 1]), "count": c, "confidence": conf, "agreement": acc})
    return {"ece": ece, "bins": table}


@torch.no_grad()
def collect(model, batches: List[torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Per position: margins at the two early exits, agreement of their arg-max with the Cortex arg-max, and whether
    each exit predicts the actual next token."""
    out = {f"{e}_{k}": [] for e in EXITS for k in ("margin", "agree")}
    out.update({f"{e}_correct": [] for e in EXITS + ("cortex",)})
    was = model.training
    model.eval()
    try:
        for ids in batches:
            x, y = ids[:, :-1], ids[:, 1:]
            lr, ll, lc, _ = model.forward_all_exits(x)
            top_c = lc.float().argmax(-1)
            for name, lg in zip(EXITS, (lr, ll)):
                out[f"{name}_margin"].append(model._margin(lg).reshape(-1).cpu())
                top = lg.float().argmax(-1)
                out[f"{name}_agree"].append((top == top_c).reshape(-1).cpu())
                out[f"{name}_correct"].append((top == y).reshape(-1).cpu())
            out["cortex_correct"].append((top_c == y).reshape(-1).cpu())
    finally:
        model.train(was)
    return {k: torch.cat(v) for k, v in out.items()}


def curve(margin: torch.Tensor, agree: torch.Tensor) -> List[Dict]:
    rows = []
    for tau in GRID:
        m = margin >= tau
        n = int(m.sum())
        hits = int(agree[m].sum()) if n else 0
        rows.append({"tau": tau, "positions": n, "coverage": n / max(1, len(margin)), "agreement": hits / n if n else None,
                     "agreement_lower": wilson_lower(hits, n)})
    return rows


def calibrate(margin: torch.Tensor, agree: torch.Tensor, target: float, min_positions: int = 50) -> Optional[float]:
    """Smallest tau of the grid whose released positions agree with the full depth at ``target`` or better (Wilson lower
    bound), with at least ``min_positions`` of them; None when no tau qualifies."""
    for row in curve(margin, agree):
        if row["positions"] >= min_positions and row["agreement_lower"] >= target:
            return row["tau"]
    return None


def layers_saved(model, released_reflex: float, released_limbic: float) -> float:
    """Share of block evaluations that are not run when those shares of positions leave at the two early exits."""
    L = model.num_layers
    after_reflex = L - (model.reflex_exit_layer + 1)
    after_limbic = L - (model.limbic_exit_layer + 1)
    return (released_reflex * after_reflex + released_limbic * after_limbic) / L


@torch.no_grad()
def policy_latency(model, ids: torch.Tensor, tau: float, iters: int = 5) -> Dict:
    """Milliseconds of one forward pass: full depth against the confidence policy at ``tau`` (which also reports where the
    tokens left)."""
    def run(**kw):
        def once():
            return model(ids, **kw)
        once()
        if ids.is_cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            once()
        if ids.is_cuda:
            torch.cuda.synchronize()
        return (time.perf_counter() - t0) / iters * 1e3

    was = model.training
    model.eval()
    try:
        full = run(force_depth=2)
        calm = run(exit_policy="calm", confidence_threshold=float(tau))
        stats = dict(model.last_calm_compaction_stats or {})
    finally:
        model.train(was)
    return {"full_depth_ms": full, "calm_ms": calm, "speedup": full / calm if calm > 0 else None, "where_tokens_left": stats}


def evaluate(model, cal: Dict[str, torch.Tensor], held: Dict[str, torch.Tensor], targets=(0.90, 0.95), min_positions: int = 50) -> Dict:
    res: Dict = {"positions": {"calibration": int(len(cal["reflex_margin"])), "held_out": int(len(held["reflex_margin"]))},
                 "accuracy_held_out": {e: float(held[f"{e}_correct"].float().mean()) for e in EXITS + ("cortex",)}, "exits": {}}
    for e in EXITS:
        hm, ha = held[f"{e}_margin"], held[f"{e}_agree"]
        entry = {"agreement_all_positions": float(ha.float().mean()), "auroc": auroc(hm, ha), **reliability(hm, ha), "targets": {},
                 "held_out_curve": curve(hm, ha)}
        for t in targets:
            tau = calibrate(cal[f"{e}_margin"], cal[f"{e}_agree"], t, min_positions)
            if tau is None:
                entry["targets"][str(t)] = {"tau": None, "note": "no threshold of the grid reaches this agreement on the calibration split"}
                continue
            m = hm >= tau
            n = int(m.sum())
            cov = n / max(1, len(hm))
            entry["targets"][str(t)] = {
                "tau": tau, "coverage": cov, "agreement": float(ha[m].float().mean()) if n else None,
                "agreement_lower": wilson_lower(int(ha[m].sum()), n) if n else 0.0,
                "layer_evaluations_saved": layers_saved(model, cov, 0.0) if e == "reflex" else layers_saved(model, 0.0, cov)}
        res["exits"][e] = entry
    return res


def synthetic_batches(vocab: int, n: int, batch: int, seq: int, seed: int, order_seed: int = 7) -> List[torch.Tensor]:
    """Sequences of a fixed random first-order Markov language with peaked transitions (something to learn and agree on)."""
    g = torch.Generator().manual_seed(order_seed)
    logits = torch.randn(vocab, vocab, generator=g) * 3.0
    P = torch.softmax(logits, dim=-1)
    g2 = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.empty(batch, seq + 1, dtype=torch.long)
        ids[:, 0] = torch.randint(0, vocab, (batch,), generator=g2)
        for t in range(seq):
            ids[:, t + 1] = torch.multinomial(P[ids[:, t]], 1, generator=g2).squeeze(1)
        out.append(ids)
    return out


def corpus_batches(path: str, tokenizer, n: int, batch: int, seq: int, skip: int = 0) -> List[torch.Tensor]:
    from ..data.dataset import TEXT_KEYS, iter_local_texts

    stream: List[int] = []
    need = (skip + n) * batch * (seq + 1)
    for row in iter_local_texts(path):
        text = next((row[k] for k in TEXT_KEYS if isinstance(row.get(k), str)), None) if isinstance(row, dict) else row
        if not text:
            continue
        enc = tokenizer.encode(text)
        stream.extend(getattr(enc, "ids", enc))
        if len(stream) >= need:
            break
    t = torch.tensor(stream[: (len(stream) // (batch * (seq + 1))) * batch * (seq + 1)], dtype=torch.long).view(-1, batch, seq + 1)
    return list(t[skip: skip + n])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="threshold calibration of the confidence exits")
    ap.add_argument("--model", default="triune-nano")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--corpus", default=None, help=".txt / .jsonl / .parquet file; synthetic Markov sequences when absent")
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--train-steps", type=int, default=0, help="joint-exit training steps on the synthetic language before calibrating")
    ap.add_argument("--batches", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--targets", type=float, nargs="+", default=[0.90, 0.95])
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    from ..models.zoo import load_model
    from ..utils import place_model

    dev = torch.device(a.device)
    over = {} if a.checkpoint or a.corpus else {"vocab_size": 256}
    model = place_model(load_model(a.checkpoint or a.model, **over), dev, torch.bfloat16 if dev.type == "cuda" else torch.float32)
    vocab = int(model.vocab_size)
    if a.corpus:
        from ..data.tokenizer import load_tokenizer
        from ..serve.engine_state import ByteTokenizer

        tok = load_tokenizer(a.tokenizer) if a.tokenizer else ByteTokenizer(min(256, vocab))
        cal = corpus_batches(a.corpus, tok, a.batches, a.batch, a.seq, 0)
        held = corpus_batches(a.corpus, tok, a.batches, a.batch, a.seq, a.batches)
    else:
        cal = synthetic_batches(vocab, a.batches, a.batch, a.seq, seed=1)
        held = synthetic_batches(vocab, a.batches, a.batch, a.seq, seed=2)
        if a.train_steps:
            opt = torch.optim.AdamW(model.parameters(), lr=2e-3)
            model.train()
            for k, ids in enumerate(synthetic_batches(vocab, a.train_steps, a.batch, a.seq, seed=3)):
                ids = ids.to(dev)
                losses, _ = model.exit_losses(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
                opt.zero_grad()
                (0.3 * losses[0] + 0.5 * losses[1] + losses[2]).backward()
                opt.step()
    cal, held = [b.to(dev) for b in cal], [b.to(dev) for b in held]
    if not cal or not held:
        print(json.dumps({"error": "the corpus is too short for two disjoint splits"}))
        return 1
    res = evaluate(model, collect(model, cal), collect(model, held), tuple(a.targets))
    tau = next((v["tau"] for v in res["exits"]["reflex"]["targets"].values() if v.get("tau") is not None), 0.5)
    res["latency"] = policy_latency(model, held[0][:, :-1], tau)
    res["config"] = {"model": a.checkpoint or a.model, "device": str(dev), "data": a.corpus or "synthetic Markov language", "train_steps": a.train_steps,
                     "latency_tau": tau}
    for e in EXITS:
        res["exits"][e].pop("held_out_curve")
        res["exits"][e].pop("bins")
    print(json.dumps({"eval": "calm calibration", **res}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
