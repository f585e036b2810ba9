"""Run every benchmark of the repository in one go and gather their JSON lines into one file.

    python bench_all.py --out results.jsonl                 # everything that fits the visible GPUs
    python bench_all.py --only A,C --out results.jsonl      # headline training + kernels
    python bench_all.py --list                              # show the commands without running them

Categories (the reference groups its suite the same way, `scripts/run_all_benchmarks.py`, categories A-F):

    A  headline training step (bench.py, ours and the reference arm)         1 GPU
    B  serving: prefill 4 x 16384, decode, FP8 / NVFP4 (bench_serving.py)    1 GPU
    C  kernels one at a time (triune_b200.bench_kernels, all cases) and the
       reference's published micro-benchmarks with both arms (bench_micro.py)  1 GPU
    D  associative recall of the mixers, 100-step optimizer convergence,
       confidence-exit calibration, QR residuals, exit latencies              1 GPU (or CPU)
    E  multi-GPU: data parallel scaling, expert / tensor / pipeline parallel  2+ GPUs, skipped when there are fewer
    F  layer-streamed training from host memory (bench_streaming.py)         1 GPU

Each command runs as a child process with its own time limit; its stdout lines that parse as JSON objects are copied
to `--out` with the category and the command attached, and a failure or a timeout is recorded as a line of its own
instead of stopping the run.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from typing import List, Tuple

ROOT = os.path.dirname(os.path.abspath(__file__))
PY = sys.executable


def torchrun(n: int, port: int, script: str, *args: str) -> List[str]:
    return [PY, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
            "--master-port", str(port), os.path.join(ROOT, script), *args]


def plan(gpus: int, quick: bool) -> List[Tuple[str, int, int, List[str]]]:
    """(category, GPUs needed, time limit in seconds, command)."""
    steps, warm = ("3", "3") if quick else ("10", "3")
    p: List[Tuple[str, int, int, List[str]]] = [
        ("A", 1, 900, [PY, os.path.join(ROOT, "bench.py"), "--steps", steps, "--warmup", warm]),
        ("A", 1, 900, [PY, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", steps, "--warmup", warm]),
        ("B", 1, 1200, [PY, os.path.join(ROOT, "bench_serving.py")]),
        ("B", 1, 900, [PY, os.path.join(ROOT, "bench_serving.py"), "--impl", "reference"]),
        ("C", 1, 900, [PY, "-m", "triune_b200.bench_kernels", "--case", "all"]),
    ]
    for case in ("mlp", "moe_route", "fp8", "nvfp4", "ce"):
        p.append(("C", 1, 600, [PY, "-m", "triune_b200.bench_kernels", "--case", case]))
    p += [
        ("C", 1, 600, [PY, "-m", "triune_b200.bench_kernels", "--case", "gdn"]),
        ("C", 1, 900, [PY, "-m", "triune_b200.bench_kernels", "--case", "gdn", "--batch", "4", "--seq", "8192", "--heads", "16",
                       "--head-dim", "128", "--iters", "4"]),
        ("D", 0, 900, [PY, "-m", "triune_b200.evals.mqar"]),
        ("D", 0, 900, [PY, "-m", "triune_b200.evals.convergence", "--family", "dense"]),
        ("D", 0, 900, [PY, "-m", "triune_b200.evals.convergence", "--family", "moe"]),
        ("D", 0, 900, [PY, "-m", "triune_b200.evals.calm", "--train-steps", "60"]),
        ("D", 0, 900, [PY, "-m", "triune_b200.evals.qr_residuals", "--train-steps", "30"]),
        ("D", 1, 600, [PY, "-m", "triune_b200.evals.dynamic_exits", "--calm-tau", "0.2"]),
        ("C", 1, 1500, [PY, os.path.join(ROOT, "bench_micro.py")]),
    ]
    for n in (2, 4, 8):
        p.append(("E", n, 900, torchrun(n, 29500 + n, "bench.py", "--gpus", str(n), "--steps", steps, "--warmup", warm)))
    p += [
        ("E", 8, 1800, torchrun(8, 29540, "bench_ep.py", "--steps", "5", "--warmup", "3")),
        ("E", 8, 900, torchrun(8, 29541, "bench_dp.py", "--params", "1.5e9", "--iters", "5")),
        ("E", 8, 900, torchrun(8, 29542, "bench_dp.py", "--params", "1.5e9", "--iters", "5", "--mode", "nccl")),
        ("E", 8, 1200, torchrun(8, 29543, "bench_serving.py", "--new-tokens", "0", "--layout", "replicas")),
        ("E", 8, 1200, torchrun(8, 29544, "bench_serving.py", "--new-tokens", "0", "--layout", "ep")),
        ("E", 2, 1800, torchrun(2, 29560, "bench_tp.py", "--steps", "5", "--warmup", "3")),
        ("E", 2, 1800, torchrun(2, 29561, "bench_tp.py", "--steps", "5", "--warmup", "3", "--mixer", "gla")),
        ("E", 8, 1800, torchrun(8, 29562, "bench_tp.py", "--tp", "2", "--batch", "4", "--seq", "8192", "--steps", "3", "--warmup", "2")),
        ("E", 8, 1800, torchrun(8, 29563, "bench_tp.py", "--tp", "2", "--batch", "4", "--seq", "8192", "--steps", "3", "--warmup", "2",
                                "--tp-mode", "nccl", "--dp-mode", "nccl")),
        ("E", 4, 1800, torchrun(4, 29570, "bench_pp.py", "--steps", "5", "--warmup", "3")),
        ("F", 1, 1800, [PY, os.path.join(ROOT, "bench_streaming.py")]),
        ("F", 1, 1800, [PY, os.path.join(ROOT, "bench_streaming.py"), "--shape", "1536", "13", "--vocab", "4096", "--batch", "2",
                        "--seq", "512"]),
    ]
    return [c for c in p if c[1] <= gpus or c[1] == 0]


def run_one(cat: str, limit: int, cmd: List[str], out) -> bool:
    shown = " ".join("python" if c == PY else os.path.relpath(c, ROOT) if c.startswith(ROOT) else c for c in cmd)
    t0 = time.time()
    env = dict(os.environ, PYTHONPATH=ROOT + (os.pathsep + os.environ["PYTHONPATH"] if os.environ.get("PYTHONPATH") else ""))
    try:
        r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=limit)
        code, text, err = r.returncode, r.stdout, r.stderr
    except subprocess.TimeoutExpired as e:
        code, text, err = -1, (e.stdout or b"").decode() if isinstance(e.stdout, bytes) else (e.stdout or ""), f"timed out after {limit} s"
    n = 0
    for line in text.splitlines():
        line = line.strip()
        if line.startswith("{"):
            try:
                rec = json.loads(line)
            except ValueError:
                continue
            out.write(json.dumps({"category": cat, "command": shown, **rec}) + "\n")
            n += 1
    if code != 0 or n == 0:
        out.write(json.dumps({"category": cat, "command": shown, "failed": True, "exit_code": code,
                              "stderr_tail": (err or "")[-1500:]}) + "\n")
    out.flush()
    print(f"[{cat}] {'ok ' if code == 0 and n else 'FAIL'} {time.time() - t0:6.1f}s {n:3d} records  {shown}", flush=True)
    return code == 0 and n > 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="bench_results.jsonl")
    ap.add_argument("--only", default="", help="comma-separated categories, e.g. A,C (default: all)")
    ap.add_argument("--gpus", type=int, default=-1, help="how many GPUs may be used (default: all visible)")
    ap.add_argument("--quick", action="store_true", help="fewer timed steps for the training benchmarks")
    ap.add_argument("--list", action="store_true", help="print the commands and exit")
    a = ap.parse_args()
    gpus = a.gpus
    if gpus < 0:
        try:
            import torch

            gpus = torch.cuda.device_count()
        except Exception:
            gpus = 0
    want = {c.strip().upper() for c in a.only.split(",") if c.strip()}
    todo = [c for c in plan(gpus, a.quick) if not want or c[0] in want]
    if a.list:
        for cat, n, limit, cmd in todo:
            print(cat, f"gpus={n}", f"limit={limit}s", " ".join(cmd))
        return 0
    ok = 0
    with open(a.out, "a") as out:
        out.write(json.dumps({"category": "meta", "started": time.strftime("%Y-%m-%d %H:%M:%S"), "gpus": gpus,
                              "commands": len(todo)}) + "\n")
        for cat, _, limit, cmd in todo:
            ok += run_one(cat, limit, cmd, out)
    print(f"{ok}/{len(todo)} commands produced results -> {a.out}")
    return 0 if ok == len(todo) else 1


if __name__ == "__main__":
    sys.exit(main())
