"""Worker of the elastic data-parallel test: a tiny regression trained with gradient all-reduce on gloo. One rank
(VICTIM) leaves without notice, either between two steps or after the others have already entered the step's
collective; the survivors must notice, re-form, reload the last checkpoint and finish with identical weights."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from triune_b200.parallel.elastic import ElasticGroup, run_elastic

    port, ident, world = int(os.environ["EL_PORT"]), int(os.environ["EL_IDENT"]), int(os.environ["EL_WORLD"])
    victim, die_at, mode = int(os.environ["EL_VICTIM"]), int(os.environ["EL_DIE_AT"]), os.environ["EL_MODE"]
    ckpt = os.environ["EL_CKPT"]
    total = int(os.environ.get("EL_STEPS", "8"))
    on_gpu = os.environ.get("EL_DEVICE", "cpu") == "cuda"
    strict = os.environ.get("EL_STRICT", "1" if on_gpu else "0") == "1"
    dev = torch.device("cpu")
    if on_gpu:
        # GPU form of the test: NCCL over plain peer transport (no NVLS), members meet on the store before every step,
        # and a rank only ever leaves between two steps with its own work drained
        torch.cuda.set_device(ident)
        dev = torch.device("cuda", ident)
    group = ElasticGroup("127.0.0.1", port, ident, world, backend="nccl" if on_gpu else "gloo", hb_interval=0.1, hb_timeout=1.0,
                         pg_timeout=20.0 if on_gpu else 4.0, device_id=dev if on_gpu else None, strict_steps=strict)
    torch.manual_seed(0)
    w = torch.zeros(4, dtype=torch.float64, device=dev)
    target = torch.tensor([1.0, -2.0, 0.5, 3.0], dtype=torch.float64, device=dev)

    def save(step):
        tmp = ckpt + ".tmp"
        torch.save({"w": w.clone(), "step": step}, tmp)
        os.replace(tmp, ckpt)

    def load():
        if not os.path.exists(ckpt):
            return 0
        ck = torch.load(ckpt, map_location="cpu")
        w.copy_(ck["w"])
        return int(ck["step"])

    def step_fn(step, g):
        if ident == victim and step == die_at and mode == "between" and not on_gpu:
            os._exit(17)  # gone between two steps, nothing in flight
        gen = torch.Generator().manual_seed(1000 * step + g.rank)  # data sharded by the CURRENT rank
        x = torch.randn(16, 4, generator=gen, dtype=torch.float64).to(dev)
        err = x @ w - x @ target
        grad = x.t() @ err / len(x)
        if ident == victim and step == die_at and mode == "midstep" and not on_gpu:
            os._exit(17)  # the others are already on their way into the all-reduce
        dist.all_reduce(grad)
        w.sub_(0.1 * grad / g.world)
        loss = float((err ** 2).mean())
        if on_gpu and ident == victim and step + 1 == die_at:
            # leave BEFORE the next step's meeting: this rank's step is complete and drained, it says so on the store,
            # and the others learn of it on the host before they launch anything
            torch.cuda.synchronize()
            g.leave()
            os._exit(17)
        return loss

    out = run_elastic(group, step_fn, save, load, total_steps=total, checkpoint_every=2)
    out["ident"] = ident
    out["w"] = [round(float(v), 12) for v in w]
    print("RESULT " + json.dumps(out), flush=True)
    group.shutdown()


if __name__ == "__main__":
    main()
