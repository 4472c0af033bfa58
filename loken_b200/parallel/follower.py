"""Serving under tensor parallelism: rank 0 owns the HTTP side, every rank owns an engine, and
all engines take the same steps.

Each rank's scheduler is deterministic, so it is enough that every rank sees the same requests in
the same order before every step: rank 0 records what was admitted or aborted since the last
step and broadcasts that list (a few hundred bytes over a gloo control group); then every rank
runs `engine.step()`, whose kernels meet in the tensor-parallel collectives.  Seeds are fixed on
rank 0 before the broadcast so all ranks draw the same uniforms.  Every other call that runs a
forward or changes the allocator (`embed`, `layer_perf`, `import_prefix`, `reset_prefix_cache`,
attaching or detaching a drafter) is broadcast as a ("call", name, args) message and executed by
all ranks at the same point between two steps; anything not on the read-only allow-list raises
instead of silently running on rank 0 alone.

Failure detection: rank 0 sends a keep-alive through the same group while the server idles, so a
follower's receive has a finite timeout; every rank beats in the job's key-value store
(`watchdog.RankWatchdog`) and rank 0 looks at the beats before each step.  A rank that left or
went silent makes rank 0's next step raise `RankLeft` (the worker's three-strikes rule then marks
the deployment unhealthy) and makes the followers' receive run out, after which they return.
Nothing here touches a GPU: a rank leaves between steps only.

The reference runs tensor parallelism inside one process over several cards
(`src/inference/generic_transformer/tensor_parallel.rs`); one process per GPU needs this
hand-shake instead.  Its failure handling is the worker's three strikes
(`src/inference/serve/continuous_serve.rs:1647-1675`) and the phi-accrual detector between nodes
(`src/distributed/membership.rs:78-160`).
"""
from __future__ import annotations

import dataclasses
import datetime
import random
import threading
import time
from typing import List, Optional

import torch.distributed as dist

# engine attributes rank 0's callers may read through the wrapper; none of them runs a forward
# or changes state the followers would have to mirror
READ_ONLY = frozenset({
    "cfg", "device", "max_ctx", "eos", "stats", "seqs", "rngs", "alloc", "runner", "sched", "spec", "weights",
    "cancelled", "has_work", "grammar_factory", "next_id",
})
# engine methods that every rank has to execute at the same point between two steps
MIRRORED = frozenset({"embed", "layer_perf", "import_prefix", "reset_prefix_cache", "detach_speculator",
                      "context_shift"})


class RankLeft(RuntimeError):
    """A tensor-parallel rank left or stopped beating; its collectives would never complete."""


def control_group(timeout_s: float = 60.0):
    """A gloo group for the step hand-shake.  The timeout bounds a follower's wait for rank 0's
    next message; rank 0 sends a keep-alive well inside it while the server idles."""
    return dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))


class LockstepEngine:
    """Rank 0's view: the engine the worker thread drives, with every mutation recorded and sent
    to the other ranks ahead of the step that uses it."""

    def __init__(self, engine, group=None, watchdog=None, keepalive_s: float = 10.0):
        self._e = engine
        self._group = group
        self._ops: List[tuple] = []
        self._watchdog = watchdog
        self._lock = threading.Lock()          # one broadcast at a time (worker thread, keep-alive thread)
        self._last_send = time.monotonic()
        self._closed = False
        self._beat = None
        if keepalive_s and keepalive_s > 0:
            self._beat = threading.Thread(target=self._keepalive, args=(keepalive_s,), daemon=True)
            self._beat.start()

    def __getattr__(self, name):
        if name in READ_ONLY:
            return getattr(self._e, name)
        if name in MIRRORED:
            return lambda *a, **kw: self._call(name, *a, **kw)
        raise AttributeError(f"'{name}' is not available under tensor parallelism: only calls that every rank "
                             f"mirrors ({', '.join(sorted(MIRRORED))}) or read-only attributes pass the wrapper")

    # ---- messages ----
    def _send(self, msg: tuple):
        with self._lock:
            if self._closed:
                raise RankLeft("the tensor-parallel group was shut down")
            box = [msg]
            try:
                dist.broadcast_object_list(box, src=0, group=self._group)
            except Exception as e:
                # a member left between the watchdog's last look and this send: the group is broken for good
                self._closed = True
                dead = []
                if self._watchdog is not None:
                    time.sleep(self._watchdog.interval * 2)
                    dead = self._watchdog.check()
                raise RankLeft(f"tensor-parallel rank(s) {dead or '?'} left or stopped beating "
                               f"({type(e).__name__} on the control group)") from e
            self._last_send = time.monotonic()

    def _keepalive(self, period: float):
        while not self._closed:
            time.sleep(min(period / 4, 1.0))
            if self._closed:
                return
            if time.monotonic() - self._last_send >= period:
                try:
                    self._send(("idle",))
                except Exception:
                    return

    def _check_peers(self):
        if self._watchdog is not None:
            dead = self._watchdog.check()
            if dead:
                self._closed = True
                raise RankLeft(f"tensor-parallel rank(s) {dead} left or stopped beating")

    def _call(self, name: str, *args, **kw):
        self._check_peers()
        self._send(("call", name, args, kw))
        return getattr(self._e, name)(*args, **kw)

    # ---- engine surface ----
    def add_request(self, prompt, params=None, salt: int = 0) -> int:
        if params is not None and params.seed is None:
            params = dataclasses.replace(params, seed=random.SystemRandom().getrandbits(62))
        embeds = getattr(prompt, "embeds", None)
        sid = self._e.add_request(prompt, params, salt, **({"embeds": embeds} if embeds is not None else {}))
        self._ops.append(("add", list(prompt), params, salt, embeds))
        return sid

    def abort(self, seq_id: int):
        self._e.abort(seq_id)
        self._ops.append(("abort", seq_id))

    def attach_speculator(self, spec):
        raise RuntimeError("under tensor parallelism a drafter is attached on every rank before serving starts "
                           "(`attach_draft` before the engines are wrapped)")

    def export_prefix(self, prompt, salt: int = 0):
        raise ValueError("a tensor-parallel model holds one cache shard per rank; hand-over is per engine")

    def step(self):
        self._check_peers()
        ops, self._ops = self._ops, []
        self._send(("step", ops))
        return self._e.step()

    def shutdown(self):
        try:
            self._send(("stop",))
        finally:
            self._closed = True


def follow(llm_or_engine, group=None, watchdog=None) -> int:
    """Ranks other than 0: apply what rank 0 admitted, take the step, repeat until told to stop.
    Returns 0 after an orderly stop, 3 when rank 0 (or the group) went away."""
    eng = getattr(llm_or_engine, "engine", llm_or_engine)
    worker = getattr(llm_or_engine, "worker", None)
    if worker is not None:
        worker.shutdown()            # this rank's engine is driven from here, not by a worker thread
        worker.join(timeout=5)
    while True:
        box = [None]
        try:
            dist.broadcast_object_list(box, src=0, group=group)
        except Exception:
            # the receive ran out (rank 0 sends keep-alives, so it is gone) or the group broke
            if watchdog is not None:
                watchdog.leave()
            return 3
        msg = box[0]
        kind = msg[0]
        if kind == "stop":
            return 0
        if kind == "idle":
            continue
        if kind == "call":
            _, name, args, kw = msg
            try:
                getattr(eng, name)(*args, **kw)
            except Exception:
                pass                 # rank 0 raised the same error to its caller; the ranks stay in step
            continue
        for op in msg[1]:
            if op[0] == "add":
                try:
                    eng.add_request(op[1], op[2], salt=op[3],
                                    **({"embeds": op[4]} if len(op) > 4 and op[4] is not None else {}))
                except ValueError:
                    pass             # refused on rank 0 too (same allocator state): no sequence anywhere
            elif op[0] == "abort":
                eng.abort(op[1])
        try:
            eng.step()
        except Exception:
            pass                     # rank 0's worker counts the strike; the plan's sequences ended on every rank
        # finished sequences are dropped as rank 0's worker drops them
        for sid in [sid for sid, s in eng.seqs.items() if s.state == "finished"]:
            eng.seqs.pop(sid, None)
            eng.rngs.pop(sid, None)
