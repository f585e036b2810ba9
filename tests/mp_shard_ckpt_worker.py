"""Worker for the sharded-checkpoint test (gloo, two ranks): a tensor-parallel dense model and an expert-parallel MoE
model each save rank-local shard files; rank 0 then merges them with the command-line tool, loads the merged file into
the unsharded model and compares logits; every rank also resumes its own shard into a re-initialised sharded model."""

import json
import os
import subprocess
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from triune_b200.config import ModelConfig  # noqa: E402
from triune_b200.models import TriuneTransformer  # noqa: E402
from triune_b200.models.universal import UniversalDenseTransformer  # noqa: E402
from triune_b200.parallel.expert_parallel import EPContext, shard_experts  # noqa: E402
from triune_b200.parallel.tensor_parallel import TPContext  # noqa: E402
from triune_b200.parallel.tp_model import TensorParallelDense  # noqa: E402
from triune_b200.trainer.checkpoint import load_checkpoint  # noqa: E402
from triune_b200.trainer.sharded_checkpoint import collect_pieces, load_sharded, save_sharded  # noqa: E402


def main():
    dist.init_process_group("gloo")
    r, w = dist.get_rank(), dist.get_world_size()
    out_dir = sys.argv[1]
    out = {"rank": r}
    ids = torch.randint(0, 256, (2, 24), generator=torch.Generator().manual_seed(3))

    # ---- tensor parallel, both block kinds
    for mixer, ffn in (("gla", "swiglu"), ("gated_deltanet", "gelu")):
        key = f"tp_{mixer}_{ffn}"
        torch.manual_seed(11)
        cfg = ModelConfig(family="universal", vocab_size=256, hidden_dim=64, num_layers=2, num_heads=4, head_dim=16,
                          mixer=mixer, ffn=ffn, dense_hidden=128, num_experts=1, top_k=1, tie_embeddings=False)
        full = UniversalDenseTransformer.from_config(cfg)
        with torch.no_grad():
            for p in full.parameters():
                p.mul_(1.5)  # "trained" weights, identical on both ranks
        full.eval()
        want = full(ids)
        want = (want[0] if isinstance(want, tuple) else want).detach()
        model = TensorParallelDense(full, TPContext(device="cpu", mode="nccl"))
        d = os.path.join(out_dir, key)
        save_sharded(d, model, step=7, loss=1.25, config={"vocab_size": 256})
        dist.barrier()
        if r == 0:
            p = subprocess.run([sys.executable, "-m", "triune_b200", "checkpoint", "merge", "--dir", d, "--output",
                                os.path.join(d, "merged.pt")], capture_output=True, text=True, cwd=ROOT)
            assert p.returncode == 0, p.stdout + p.stderr
            torch.manual_seed(99)
            fresh = UniversalDenseTransformer.from_config(cfg).eval()
            ck = load_checkpoint(os.path.join(d, "merged.pt"), fresh, strict=True)
            got = fresh(ids)
            got = (got[0] if isinstance(got, tuple) else got).detach()
            out[key + "_merged_logits"] = float((got - want).abs().max())
            out[key + "_step"] = ck["step"]
        # resume: a differently initialised sharded model takes this rank's shard back
        torch.manual_seed(5)
        other = TensorParallelDense(UniversalDenseTransformer.from_config(cfg), TPContext(device="cpu", mode="nccl"))
        meta = load_sharded(d, other)
        a, _ = collect_pieces(model)
        b, _ = collect_pieces(other)
        out[key + "_resume"] = max(float((x[5] - y[5]).abs().max()) for x, y in zip(a, b))
        out[key + "_resume_step"] = meta["step"]
        dist.barrier()

    # ---- expert parallel
    torch.manual_seed(13)
    arch = dict(vocab_size=256, hidden_dim=64, num_layers=4, num_heads=2, head_dim=32, num_experts=4,
                router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3)
    full = TriuneTransformer(**arch).eval()
    want = full(ids, force_depth=2)[0].detach()
    canonical = {k: v.detach().clone() for k, v in full.state_dict().items()}
    n = shard_experts(full, EPContext(4, device="cpu", mode="nccl"))
    assert n >= 1
    d = os.path.join(out_dir, "ep")
    save_sharded(d, full, step=3)
    dist.barrier()
    if r == 0:
        p = subprocess.run([sys.executable, "-m", "triune_b200", "checkpoint", "merge", "--dir", d, "--output",
                            os.path.join(d, "merged.pt")], capture_output=True, text=True, cwd=ROOT)
        assert p.returncode == 0, p.stdout + p.stderr
        torch.manual_seed(77)
        fresh = TriuneTransformer(**arch).eval()
        load_checkpoint(os.path.join(d, "merged.pt"), fresh, strict=True)
        out["ep_merged_logits"] = float((fresh(ids, force_depth=2)[0].detach() - want).abs().max())
        merged = torch.load(os.path.join(d, "merged.pt"), weights_only=True)["model_state"]
        out["ep_keys_equal"] = int(sorted(merged) == sorted(canonical))
        out["ep_has_per_expert_keys"] = int(any(".experts.3.2.weight" in k for k in merged))
    dist.barrier()
    print("RESULT " + json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
