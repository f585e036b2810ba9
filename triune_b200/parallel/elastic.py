"""Rank-failure detection and elastic data parallelism: heartbeats in a key-value store, a detector every rank polls
before it launches the next step, and re-forming the process group over the survivors.

How a failure is seen. Every rank runs a :class:`Heartbeat` thread that bumps a counter under its own key a few times
per second. A :class:`FailureDetector` remembers when it last saw each counter move; a rank whose counter stands still
for longer than ``timeout`` is dead. Ranks consult the detector on the host *between* steps
(:meth:`ElasticGroup.guard`), so a peer that is gone is noticed before anything is launched towards it. If a peer dies
after the check, the next collective ends with the process group's own (short) timeout; that error is treated the same
way. Device-side waits of this package's fused kernels are bounded and report through a status word; a non-zero word
becomes :class:`CollectiveTimeout` (:func:`raise_on_status`) and enters the same path. Nothing here needs, causes or
simulates a GPU fault.

How the group re-forms. The survivors meet under a new generation prefix of the store: each writes a join key; the
lowest surviving original rank waits for the joins of everyone its detector still believes alive, publishes the member
list, and all of them initialise a fresh process group of that size with ranks in the order of their original ids.
:func:`run_elastic` wraps a training loop around this: check, step, periodic checkpoint; on a failure re-form, reload
the last checkpoint, go on with fewer ranks (data parallelism only: the surviving replicas hold complete models).

The reference has none of this (no heartbeat, no rank-failure handling; it checkpoints on exceptions and signals only:
``triune/trainer/engine.py:505-507``, ``triune/trainer/callbacks.py:9-26``).
"""

from __future__ import annotations

import datetime
import json
import threading
import time
from typing import Callable, Dict, List, Optional, Sequence

import torch.distributed as dist


class RankFailure(RuntimeError):
    """One or more peers stopped answering. ``dead`` holds their original rank ids."""

    def __init__(self, dead: Sequence[int], why: str = ""):
        self.dead = sorted(int(d) for d in dead)
        super().__init__(f"ranks {self.dead} stopped answering" + (f" ({why})" if why else ""))


class CollectiveTimeout(RuntimeError):
    """A bounded device-side wait of a fused communication kernel ran out; the context is still usable."""

    def __init__(self, status: int, where: str = ""):
        self.status = int(status)
        super().__init__(f"device-side wait expired{' in ' + where if where else ''}: status word {self.status:#x}")


def raise_on_status(status: int, where: str = "") -> None:
    """Turn the status word a fused kernel left behind (0 = fine) into an exception on the host."""
    if int(status) != 0:
        raise CollectiveTimeout(int(status), where)


class Heartbeat:
    """Background thread that bumps ``<prefix>/<rank>`` in the store every ``interval`` seconds."""

    def __init__(self, store, rank: int, interval: float = 0.2, prefix: str = "hb"):
        self.store, self.key, self.interval = store, f"{prefix}/{rank}", float(interval)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.beats = 0

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                self.beats += 1
                self.store.set(self.key, str(self.beats))
            except Exception:
                return  # the store is gone: nobody can read heartbeats any more
            self._stop.wait(self.interval)

    def start(self) -> "Heartbeat":
        self.store.set(self.key, "0")
        self._thread = threading.Thread(target=self._run, name="triune-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1.0)


class FailureDetector:
    """Declares a rank dead when its heartbeat counter has not moved for ``timeout`` seconds (this process's clock)."""

    def __init__(self, store, ranks: Sequence[int], timeout: float = 2.0, prefix: str = "hb", clock: Callable[[], float] = time.monotonic):
        self.store, self.prefix, self.timeout, self.clock = store, prefix, float(timeout), clock
        now = clock()
        self.seen: Dict[int, tuple] = {int(r): (None, now) for r in ranks}

    def _read(self, rank: int) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([f"{self.prefix}/{rank}"]):
                return None
            return self.store.get(f"{self.prefix}/{rank}").decode()
        except Exception:
            return None

    def poll(self) -> List[int]:
        """Refresh every rank's last-seen time; return the ranks that are overdue."""
        now, dead = self.clock(), []
        for r, (value, when) in list(self.seen.items()):
            cur = self._read(r)
            if cur is not None and cur != value:
                self.seen[r] = (cur, now)
            elif now - when > self.timeout:
                dead.append(r)
        return sorted(dead)

    def forget(self, ranks: Sequence[int]) -> None:
        for r in ranks:
            self.seen.pop(int(r), None)

    def wait_for_verdict(self, settle: Optional[float] = None) -> List[int]:
        """After an error whose cause is unknown: keep polling for a little more than the timeout, so that a peer that
        died just now has time to become overdue; return the dead ranks (possibly none)."""
        end = self.clock() + (settle if settle is not None else self.timeout * 1.5 + 0.5)
        dead: List[int] = []
        while self.clock() < end:
            dead = self.poll()
            if dead:
                return dead
            time.sleep(min(0.1, self.timeout / 4))
        return dead


def connect_store(host: str, port: int, is_master: bool = False, timeout_s: float = 60.0):
    """A TCP key-value store client (or the server itself when ``is_master``). A store hosted by a training rank dies
    with that rank; for a store that outlives any rank run :func:`serve_store` in a process of its own."""
    return dist.TCPStore(host, port, None, is_master, timeout=datetime.timedelta(seconds=timeout_s), wait_for_workers=False)


def serve_store(port: int, host: str = "127.0.0.1") -> None:
    """Host the store and sleep until interrupted (``python -m triune_b200.parallel.elastic --serve-store PORT``)."""
    store = connect_store(host, port, is_master=True)
    store.set("store/up", "1")
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        pass


class ElasticGroup:
    """Membership of one rank in a data-parallel job that shrinks when peers fail.

    ``ident`` is this rank's original id (stable for the whole job); :attr:`rank` / :attr:`world` describe the current
    process group and change with every :meth:`reform`. ``pg_timeout`` is the process group's own limit for one
    collective: keep it short (seconds), it is what ends a collective whose peer died after the last check.
    """

    def __init__(self, host: str, port: int, ident: int, world: int, backend: str = "gloo", hb_interval: float = 0.2,
                 hb_timeout: float = 2.0, pg_timeout: float = 10.0, host_store: bool = False, device_id=None,
                 strict_steps: bool = False):
        """``strict_steps``: before every step all members meet on the store (``step_rendezvous``), so that no rank
        launches a collective, or a fused kernel that waits for a peer, while a member is missing. This is the mode
        for GPUs: a kernel that waits for a rank that is gone only ends through a timeout."""
        self.strict_steps = bool(strict_steps)
        self.host, self.port, self.ident, self.backend = host, int(port), int(ident), backend
        self.hb_timeout, self.pg_timeout, self.device_id = float(hb_timeout), float(pg_timeout), device_id
        self.store = connect_store(host, port, is_master=host_store)
        self._hb_store = connect_store(host, port)  # the heartbeat thread talks over its own connection
        self.members: List[int] = list(range(world))
        self.generation = 0
        self.heartbeat = Heartbeat(self._hb_store, self.ident, hb_interval).start()
        self.detector = FailureDetector(self.store, [m for m in self.members if m != self.ident], hb_timeout)
        self.failures: List[List[int]] = []
        self._init_pg()

    # ------------------------------------------------------------------ process group
    @property
    def rank(self) -> int:
        return self.members.index(self.ident)

    @property
    def world(self) -> int:
        return len(self.members)

    def _init_pg(self) -> None:
        kw = {}
        if self.backend == "nccl" and self.device_id is not None:
            kw["device_id"] = self.device_id
        dist.init_process_group(self.backend, store=dist.PrefixStore(f"pg{self.generation}", self.store), rank=self.rank,
                                world_size=self.world, timeout=datetime.timedelta(seconds=self.pg_timeout), **kw)

    def _drop_pg(self) -> None:
        if not dist.is_initialized():
            return
        if self.backend == "nccl":
            # a communicator with a dead peer must be aborted, not drained: destroy would wait for work that never ends
            abort = getattr(dist.distributed_c10d, "_abort_process_group", None)
            if abort is not None:
                try:
                    abort()
                    return
                except Exception:
                    pass
        dist.destroy_process_group()

    # ------------------------------------------------------------------ detection
    def guard(self) -> None:
        """Call on the host before launching a step: raises :class:`RankFailure` if a peer is overdue or has left."""
        dead = sorted(set(self.detector.poll()) | set(self._left()))
        if dead:
            raise RankFailure(dead, "heartbeat overdue or rank left")

    def _left(self) -> List[int]:
        return [m for m in self.members if m != self.ident and self.store.check([f"left/{m}"])]

    def leave(self) -> None:
        """Announce on the store that this rank is going (between two steps, with nothing of its own in flight) and stop
        its heartbeat. The others see the announcement at their next :meth:`guard` / :meth:`step_rendezvous`."""
        self.store.set(f"left/{self.ident}", "1")
        self.heartbeat.stop()

    def step_rendezvous(self, step: int, poll_s: float = 0.002) -> None:
        """Host-side meeting before step ``step``: returns once every member has arrived; raises :class:`RankFailure`
        as soon as a member is known to have left or its heartbeat is overdue. Nothing is launched before it returns."""
        prefix = f"ready/{self.generation}/{step}"
        self.store.set(f"{prefix}/{self.ident}", "1")
        others = [m for m in self.members if m != self.ident]
        while True:
            gone = sorted(set(self._left()) | set(self.detector.poll()))
            if gone:
                raise RankFailure(gone, "member missing at the step rendezvous")
            if all(self.store.check([f"{prefix}/{m}"]) for m in others):
                return
            time.sleep(poll_s)

    def diagnose(self, error: BaseException) -> RankFailure:
        """An error came out of a step: find out whether a peer died (waits up to about 1.5 heartbeat timeouts)."""
        if isinstance(error, RankFailure):
            return error
        dead = self.detector.wait_for_verdict()
        if not dead:
            raise error  # everybody is alive: this is not a membership problem
        return RankFailure(dead, f"{type(error).__name__}: {str(error)[:120]}")

    # ------------------------------------------------------------------ re-forming
    def reform(self, dead: Sequence[int], join_timeout: float = 30.0) -> List[int]:
        """Build the next generation's group over the survivors; returns the new member list (original ids)."""
        self._drop_pg()
        gen = self.generation + 1
        prefix = f"gen{gen}"
        self.store.set(f"{prefix}/join/{self.ident}", "1")
        believed = [m for m in self.members if m not in set(dead)]
        if not believed or self.ident not in believed:
            raise RuntimeError("this rank is not among the survivors")
        leader = min(believed)
        if self.ident == leader:
            end = time.monotonic() + join_timeout
            joined = [self.ident]
            while time.monotonic() < end:
                joined = [m for m in believed if self.store.check([f"{prefix}/join/{m}"])]
                late_dead = set(self.detector.poll())
                if set(joined) >= set(believed) - late_dead:
                    break
                time.sleep(0.05)
            self.store.set(f"{prefix}/members", json.dumps(sorted(joined)))
        self.store.wait([f"{prefix}/members"], datetime.timedelta(seconds=join_timeout + 5.0))
        members = json.loads(self.store.get(f"{prefix}/members").decode())
        if self.ident not in members:
            raise RuntimeError("this rank joined too late and was left out of the new group")
        self.failures.append(sorted(set(self.members) - set(members)))
        self.detector.forget([m for m in self.members if m not in members])
        self.members, self.generation = members, gen
        self._init_pg()
        return members

    def shutdown(self) -> None:
        self.heartbeat.stop()
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_elastic(group: ElasticGroup, step_fn: Callable[[int, ElasticGroup], float], save_fn: Callable[[int], None],
                load_fn: Callable[[], int], total_steps: int, checkpoint_every: int = 1, max_reforms: int = 8,
                on_reform: Optional[Callable[[ElasticGroup], None]] = None) -> Dict[str, object]:
    """Training loop that survives the loss of data-parallel peers.

    ``step_fn(step, group)`` runs one step (its collectives use the default process group) and returns the loss;
    ``save_fn(step)`` writes a checkpoint after ``step`` steps (the lowest-ranked member is asked to; make it atomic);
    ``load_fn()`` restores the last checkpoint and returns the number of steps it contains. ``on_reform(group)`` lets the
    caller rebuild whatever depends on the world size (gradient buckets, data sharding).
    """
    step, reforms, losses = load_fn(), 0, []
    while step < total_steps:
        try:
            if group.strict_steps:
                group.step_rendezvous(step)
            else:
                group.guard()
            loss = step_fn(step, group)
            step += 1
            losses.append(float(loss))
            if step % checkpoint_every == 0:
                if group.rank == 0:
                    save_fn(step)
                dist.barrier()
        except Exception as e:  # includes RankFailure, CollectiveTimeout and the process group's own timeout
            failure = group.diagnose(e)
            reforms += 1
            if reforms > max_reforms:
                raise
            group.reform(failure.dead)
            if on_reform is not None:
                on_reform(group)
            step = load_fn()
    return {"steps": step, "world": group.world, "members": list(group.members), "generation": group.generation,
            "failures": list(group.failures), "losses": losses}


def launch(n: int, command: Sequence[str], host: str = "127.0.0.1", port: int = 0) -> int:
    """Host the store in this process and start ``n`` copies of ``command`` with the elastic environment set
    (``TRIUNE_ELASTIC_STORE`` / ``_IDENT`` / ``_WORLD``, ``LOCAL_RANK``). Unlike a rendezvous launcher this one leaves the
    other children alone when one of them dies. Returns 0 when at least one child finished with exit code 0."""
    import os
    import socket
    import subprocess

    if port == 0:
        with socket.socket() as s:
            s.bind((host, 0))
            port = s.getsockname()[1]
    store = connect_store(host, port, is_master=True)  # noqa: F841  (the store lives as long as this process)
    procs = []
    for i in range(n):
        env = dict(os.environ, TRIUNE_ELASTIC_STORE=f"{host}:{port}", TRIUNE_ELASTIC_IDENT=str(i), TRIUNE_ELASTIC_WORLD=str(n),
                   LOCAL_RANK=str(i))
        procs.append(subprocess.Popen(list(command), env=env))
    codes = [p.wait() for p in procs]
    print(f"[elastic] children exited with {codes}", flush=True)
    return 0 if any(c == 0 for c in codes) else 1


if __name__ == "__main__":
    import argparse
    import sys

    ap = argparse.ArgumentParser(description="elastic jobs: a stand-alone store, or a launcher of N elastic ranks")
    ap.add_argument("--serve-store", type=int, default=None, metavar="PORT", help="only host the key-value store")
    ap.add_argument("--launch", type=int, default=None, metavar="N", help="start N ranks of the command after '--'")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("command", nargs=argparse.REMAINDER)
    a = ap.parse_args()
    if a.launch:
        cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
        if not cmd:
            ap.error("give the command to run after '--'")
        sys.exit(launch(a.launch, cmd, a.host, a.port))
    if a.serve_store is None:
        ap.error("one of --serve-store PORT or --launch N -- command")
    serve_store(a.serve_store, a.host)
