"""Short convergence runs: the same small model and data under each optimizer, loss curve and step time side by side.

The data is a learnable synthetic language: a fixed random first-order Markov chain over the vocabulary with a few
likely successors per token, so the achievable loss is known (the chain's conditional entropy) and 100 steps are enough
to see whether an optimizer is moving towards it. Reports, per optimizer: loss at the start, at every quarter and at
the end, the entropy floor, milliseconds per step and the bytes of optimizer state.

Counterpart of the reference's ``scripts/benchmark_convergence_100_steps.py``, ``benchmark_moe_convergence_100_steps.py``
and the optimizer comparison in ``scripts/benchmark_optimizer_suite.py``.

    python -m triune_b200.evals.convergence --steps 100 --family moe
"""

from __future__ import annotations

import argparse
import json
import math
import time
from typing import Dict, List

import torch

OPTIMIZERS = ("centroid_steer", "muon", "adamw")


def markov_language(vocab: int, branching: int = 4, seed: int = 0):
    """Transition table ``[vocab, branching]`` of successors, their probabilities, and the conditional entropy (nats)."""
    gen = torch.Generator().manual_seed(seed)
    succ = torch.stack([torch.randperm(vocab, generator=gen)[:branching] for _ in range(vocab)])
    probs = torch.softmax(torch.randn(vocab, branching, generator=gen) * 1.5, dim=-1)
    entropy = float(-(probs * probs.log()).sum(-1).mean())
    return succ, probs, entropy


def sample_batch(succ, probs, batch: int, seq_len: int, gen: torch.Generator) -> torch.Tensor:
    x = torch.empty(batch, seq_len + 1, dtype=torch.long)
    x[:, 0] = torch.randint(0, succ.shape[0], (batch,), generator=gen)
    for t in range(seq_len):
        choice = torch.multinomial(probs[x[:, t]], 1, generator=gen).squeeze(1)
        x[:, t + 1] = succ[x[:, t], choice]
    return x


def build_model(family: str, vocab: int, width: int, layers: int, device, dtype):
    from ..config import ModelConfig
    from ..models import TriuneTransformer
    from ..models.universal import UniversalDenseTransformer
    from ..utils import place_model

    heads, hd = max(1, width // 64), min(64, width)
    if family == "moe":
        reflex = max(2, layers // 4)
        cfg = ModelConfig(vocab_size=vocab, hidden_dim=width, num_layers=layers, num_heads=heads, head_dim=hd, num_experts=4, top_k=2,
                          router_prefix_layers=1, reflex_exit_layer=reflex, limbic_exit_layer=max(reflex + 1, layers // 2))
        model = TriuneTransformer.from_config(cfg)
    else:
        cfg = ModelConfig(family="universal", vocab_size=vocab, hidden_dim=width, num_layers=layers, num_heads=heads, head_dim=hd,
                          mixer="gla", ffn="swiglu", tie_embeddings=False)
        model = UniversalDenseTransformer.from_config(cfg)
    return place_model(model, device, dtype)


def optimizer_state_bytes(opt) -> int:
    """Bytes of distinct tensor storage reachable from the optimizer's ``state_dict()["state"]``."""
    seen, total = set(), 0

    def visit(x):
        nonlocal total
        if torch.is_tensor(x):
            key = (x.untyped_storage().data_ptr(), x.untyped_storage().nbytes())
            if key not in seen:
                seen.add(key)
                total += x.untyped_storage().nbytes()
        elif isinstance(x, dict):
            for v in x.values():
                visit(v)
        elif isinstance(x, (list, tuple)):
            for v in x:
                visit(v)

    sd = opt.state_dict()
    visit(sd["state"] if "state" in sd else sd)  # torch optimizers keep tensors under "state"; ours keeps flat buffers at the top
    return total


def run(optimizer: str, family: str = "dense", steps: int = 100, vocab: int = 256, width: int = 128, layers: int = 4, batch: int = 8,
        seq_len: int = 64, lr: float = 3e-3, device=None, seed: int = 0) -> Dict[str, object]:
    from ..optim import build_optimizer

    device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    torch.manual_seed(seed)
    model = build_model(family, vocab, width, layers, device, dtype)
    opt = build_optimizer(model, {"optimizer": optimizer, "lr": lr, "grad_clip": 1.0, "weight_decay": 0.01})
    succ, probs, floor = markov_language(vocab, seed=seed)
    gen = torch.Generator().manual_seed(seed + 1)
    losses: List[float] = []
    model.train()
    t0 = None
    for step in range(steps):
        if step == min(3, steps - 1):  # the first steps pay for allocations and caches
            if device.type == "cuda":
                torch.cuda.synchronize()
            t0, timed_from = time.perf_counter(), step
        x = sample_batch(succ, probs, batch, seq_len, gen).to(device)
        opt.zero_grad()
        loss = model.forward_loss(x[:, :-1], x[:, 1:], force_depth=2)
        loss.backward()
        if optimizer == "adamw":
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        losses.append(float(loss.detach()))
    if device.type == "cuda":
        torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / max(1, steps - timed_from)
    q = lambda f: losses[min(steps - 1, max(0, int(round(f * steps)) - 1))]  # noqa: E731
    return {"optimizer": optimizer, "family": family, "steps": steps, "loss_start": losses[0], "loss_25": q(0.25), "loss_50": q(0.5),
            "loss_75": q(0.75), "loss_end": sum(losses[-5:]) / len(losses[-5:]), "entropy_floor": floor, "uniform_loss": math.log(vocab),
            "ms_per_step": round(ms, 3), "optimizer_state_bytes": optimizer_state_bytes(opt),
            "params": sum(p.numel() for p in model.parameters()), "device": str(device), "dtype": str(dtype).split(".")[-1]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="100-step convergence of the optimizers on a learnable synthetic language")
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--family", default="dense", choices=["dense", "moe"])
    ap.add_argument("--optimizers", nargs="+", default=list(OPTIMIZERS))
    ap.add_argument("--vocab", type=int, default=256)
    ap.add_argument("--width", type=int, default=128)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--lr", type=float, default=3e-3)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    for o in a.optimizers:
        print(json.dumps(run(o, a.family, a.steps, a.vocab, a.width, a.layers, a.batch, a.seq, a.lr, a.device)), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
