"""Multi-query associative recall, solved analytically by the three sequence mixers.

A sequence holds ``pairs`` (key token, value token) pairs at random even offsets among filler tokens and ends with one
of the keys as a query; the answer is the value last bound to that key. In the *overwrite* variant half of the keys
are first bound to a stale value and re-bound later, and the query asks for one of those.

No weights are trained. Operands are written down directly, the way a one-layer induction circuit would produce them:
every token has a fixed random unit code per head (keys) and over the model width (values); at a value position the
mixer *writes* ``k = code(previous token)``, ``v = code(this token)``; at a key position it *reads* with
``q = code(this token)``. The prediction is the value token whose code is closest to the mixer's output at the last
position. What this separates:

* softmax attention averages over every matching write, stale or fresh;
* gated linear attention adds both bindings into the state, so a re-bound key returns a superposition;
* the delta rule subtracts what the state currently returns for the key before writing, so the stale value is erased.

Reported per mixer: latency of the operator (device-timed on CUDA, wall clock on CPU) and recall on the standard and
the overwrite task. Same experiment as the reference's ``scripts/benchmark_associative_recall.py:26-207``; the linear
mixers run through this package's operators (the GLA tcgen05 kernels and the Gated DeltaNet recurrence kernel on CUDA).

    python -m triune_b200.evals.mqar --seq 256 512 1024 2048
"""

from __future__ import annotations

import argparse
import json
import time
from typing import Dict, List, Tuple

import torch
import torch.nn.functional as F

from .. import ops

FILLER = (1200, 2000)     # token ranges: filler, keys, fresh values, stale values
KEYS = (10, 510)
VALUES = (2200, 3200)
STALE = (3200, 4000)
VOCAB = 4096
MIXERS = ("softmax", "gla", "gated_deltanet")


def make_task(batch: int, seq_len: int, pairs: int, overwrite: bool = False, seed: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> tokens ``[batch, seq_len]`` (the last one is the query key) and the expected value token ``[batch]``."""
    gen = torch.Generator().manual_seed(seed * 7919 + seq_len)
    tokens = torch.randint(FILLER[0], FILLER[1], (batch, seq_len), generator=gen)
    answers = torch.empty(batch, dtype=torch.long)
    n_stale = pairs // 2 if overwrite else 0
    slots_total = (seq_len - 2) // 2
    if pairs + n_stale > slots_total:
        raise ValueError(f"{pairs} pairs (+{n_stale} stale) do not fit into {seq_len} tokens")
    for b in range(batch):
        keys = torch.randperm(KEYS[1] - KEYS[0], generator=gen)[:pairs] + KEYS[0]
        vals = torch.randperm(VALUES[1] - VALUES[0], generator=gen)[:pairs] + VALUES[0]
        stale = torch.randperm(STALE[1] - STALE[0], generator=gen)[:max(1, n_stale)] + STALE[0]
        # stale bindings come first in time, then every key's final binding
        events = [(int(keys[i]), int(stale[i])) for i in range(n_stale)] + [(int(keys[i]), int(vals[i])) for i in range(pairs)]
        slots = torch.randperm(slots_total, generator=gen)[: len(events)].sort().values
        for (kt, vt), s in zip(events, slots.tolist()):
            tokens[b, 2 * s], tokens[b, 2 * s + 1] = kt, vt
        ask = int(torch.randint(0, n_stale, (1,), generator=gen)) if n_stale else int(torch.randint(0, pairs, (1,), generator=gen))
        tokens[b, -1] = keys[ask]
        answers[b] = vals[ask]
    return tokens, answers


def make_operands(tokens: torch.Tensor, dim: int, heads: int, device, dtype) -> Dict[str, torch.Tensor]:
    """q, k, v ``[B, T, H, D]``, the log decay ``g`` (almost none), the write strength ``beta`` ``[B, T, H]`` and the
    value code book ``[VOCAB, dim]``."""
    hd = dim // heads
    gen = torch.Generator().manual_seed(4242)
    key_codes = F.normalize(torch.randn(VOCAB, heads, hd, generator=gen), dim=-1)
    val_codes = F.normalize(torch.randn(VOCAB, dim, generator=gen), dim=-1)
    B, T = tokens.shape
    prev = torch.zeros_like(tokens)
    prev[:, 1:] = tokens[:, :-1]
    is_key = (tokens >= KEYS[0]) & (tokens < KEYS[1])
    write = ((tokens >= VALUES[0]) & (prev >= KEYS[0]) & (prev < KEYS[1])).float()
    q = key_codes[tokens] * is_key[..., None, None]
    k = key_codes[prev] * write[..., None, None]
    v = (val_codes[tokens] * write[..., None]).view(B, T, heads, hd)
    g = torch.full((B, T, heads, hd), -1e-4)
    beta = write[..., None].expand(B, T, heads).contiguous()
    to = lambda t: t.to(device=device, dtype=dtype).contiguous()  # noqa: E731
    return {"q": to(q), "k": to(k), "v": to(v), "g": to(g), "beta": beta.to(device=device, dtype=torch.float32),
            "codes": val_codes.to(device)}


@torch.no_grad()
def recall(mixer: str, x: Dict[str, torch.Tensor]) -> torch.Tensor:
    """Predicted value token ``[B]`` at the last position."""
    q, k, v = x["q"], x["k"], x["v"]
    B, T, H, D = q.shape
    if mixer == "softmax":
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, scale=2.0 * D ** 0.5)
        o = o.transpose(1, 2)
    elif mixer == "gla":
        o, _ = ops.gla(q, k, v, x["g"])
    elif mixer == "gated_deltanet":
        o, _ = ops.gated_deltanet(q, k, v, x["g"], beta=x["beta"])
    else:
        raise ValueError(f"unknown mixer {mixer!r}")
    last = F.normalize(o[:, -1].reshape(B, H * D).float(), dim=-1)
    lo, hi = VALUES[0], STALE[1]                      # only value tokens (fresh or stale) are candidates
    return (last @ x["codes"][lo:hi].float().t()).argmax(-1).cpu() + lo


def _time(fn, reps: int, warmup: int, device) -> float:
    for _ in range(warmup):
        fn()
    if device.type == "cuda":
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    return (time.perf_counter() - t0) * 1e3 / reps


def evaluate(mixer: str, seq_len: int, pairs: int, dim: int = 256, heads: int = 4, batch: int = 8, device=None, dtype=None,
             reps: int = 15, warmup: int = 3) -> Dict[str, float]:
    device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dtype = dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
    out: Dict[str, float] = {"mixer": mixer, "seq_len": seq_len, "pairs": pairs, "dim": dim, "heads": heads, "batch": batch,
                             "dtype": str(dtype).split(".")[-1], "timer": "cuda events" if device.type == "cuda" else "wall clock"}
    for name, over in (("recall", False), ("overwrite_recall", True)):
        tokens, answers = make_task(batch, seq_len, pairs, overwrite=over)
        x = make_operands(tokens, dim, heads, device, dtype)
        out[name] = float((recall(mixer, x) == answers).float().mean())
        if not over:
            out["latency_ms"] = round(_time(lambda: recall(mixer, x), reps, warmup, device), 4)
    return out


def main(argv: List[str] = None) -> int:
    ap = argparse.ArgumentParser(description="multi-query associative recall: softmax, GLA, Gated DeltaNet")
    ap.add_argument("--seq", type=int, nargs="+", default=[256, 512, 1024, 2048])
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--reps", type=int, default=15)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    for T in a.seq:
        for mixer in MIXERS:
            print(json.dumps(evaluate(mixer, T, max(2, T // 32), a.dim, a.heads, a.batch, a.device, reps=a.reps)), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
