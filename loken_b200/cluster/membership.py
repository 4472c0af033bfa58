"""Who is in the cluster and who has stopped answering.

`PhiAccrual` is the phi-accrual failure detector over heartbeat inter-arrival times
(`src/distributed/membership.rs:78-160`): phi = -log10(P(no heartbeat for this long)) under a
normal model of the observed intervals; a peer is suspected above `threshold`.  Time is injected
so tests never sleep.  `Membership` keeps the peer table gossip updates, and excludes a peer that
failed a hand-over for ten gossip intervals (`docs/CLUSTER.md:96-100`).  There is no consensus:
routing to a node that has just died costs one retry.
"""
from __future__ import annotations

import math
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


class PhiAccrual:
    def __init__(self, threshold: float = 8.0, window: int = 100, min_std_s: float = 0.05,
                 first_interval_s: float = 0.5, clock: Callable[[], float] = time.monotonic):
        self.threshold = threshold
        self.intervals: deque = deque(maxlen=window)
        self.min_std = min_std_s
        self.first = first_interval_s
        self.clock = clock
        self.last: Optional[float] = None

    def heartbeat(self, now: Optional[float] = None):
        now = self.clock() if now is None else now
        if self.last is not None:
            self.intervals.append(now - self.last)
        self.last = now

    def phi(self, now: Optional[float] = None) -> float:
        if self.last is None:
            return 0.0
        now = self.clock() if now is None else now
        if self.intervals:
            mean = sum(self.intervals) / len(self.intervals)
            var = sum((x - mean) ** 2 for x in self.intervals) / len(self.intervals)
        else:
            mean, var = self.first, (self.first / 4) ** 2
        std = max(math.sqrt(var), self.min_std)
        y = (now - self.last - mean) / std
        # logistic approximation of the normal tail (the one Akka / Cassandra use)
        e = math.exp(-y * (1.5976 + 0.070566 * y * y))
        p_later = e / (1.0 + e) if now - self.last > mean else 1.0 - 1.0 / (1.0 + e)
        return -math.log10(max(p_later, 1e-300))

    def available(self, now: Optional[float] = None) -> bool:
        return self.phi(now) < self.threshold


@dataclass
class Peer:
    node_id: str
    addr: str
    models: List[str] = field(default_factory=list)
    load: float = 0.0                  # running + queued requests
    tok_per_s: float = 0.0             # measured decode rate
    prefill_tok_per_s: float = 0.0     # measured prompt-reading rate
    free_kv_blocks: int = 0
    incarnation: int = 0
    detector: PhiAccrual = None
    excluded_until_round: int = -1
    rtt_ms: Optional[float] = None     # round trip of this node's gossip call to the peer (smoothed)
    layer_cost: Dict[str, dict] = field(default_factory=dict)   # model -> {card_ms, host_ms, card_bytes} as the peer measured it
    card_bytes_free: int = 0           # device memory the peer could give to weights


class Membership:
    def __init__(self, self_id: str, clock: Callable[[], float] = time.monotonic, suspect_phi: float = 8.0):
        self.self_id = self_id
        self.clock = clock
        self.suspect_phi = suspect_phi
        self.peers: Dict[str, Peer] = {}
        self.round = 0

    def observe(self, node_id: str, addr: str, *, models=None, load=None, tok_per_s=None, free_kv_blocks=None,
                incarnation: int = 0, layer_cost=None, card_bytes_free=None, prefill_tok_per_s=None):
        """A heartbeat / gossip entry about `node_id` arrived."""
        if node_id == self.self_id:
            return
        p = self.peers.get(node_id)
        if p is None or incarnation > p.incarnation:
            p = Peer(node_id, addr, incarnation=incarnation,
                     detector=PhiAccrual(self.suspect_phi, clock=self.clock))
            self.peers[node_id] = p
        p.addr = addr
        if models is not None:
            p.models = list(models)
        if load is not None:
            p.load = float(load)
        if tok_per_s is not None:
            p.tok_per_s = float(tok_per_s)
        if free_kv_blocks is not None:
            p.free_kv_blocks = int(free_kv_blocks)
        if isinstance(layer_cost, dict):
            p.layer_cost = {str(k): dict(v) for k, v in layer_cost.items() if isinstance(v, dict)}
        if card_bytes_free is not None:
            p.card_bytes_free = int(card_bytes_free)
        if prefill_tok_per_s is not None:
            p.prefill_tok_per_s = float(prefill_tok_per_s)
        p.detector.heartbeat()

    def timed(self, node_id: str, rtt_ms: float, alpha: float = 0.3):
        """A call to `node_id` took this long: the smoothed figure prices links (`cluster/cut_plan.py`)."""
        p = self.peers.get(node_id)
        if p is not None and rtt_ms >= 0:
            p.rtt_ms = rtt_ms if p.rtt_ms is None else p.rtt_ms + alpha * (rtt_ms - p.rtt_ms)

    def tick(self):
        """One gossip round passed."""
        self.round += 1

    def exclude(self, node_id: str, rounds: int = 10):
        if node_id in self.peers:
            self.peers[node_id].excluded_until_round = self.round + rounds

    def alive(self) -> List[Peer]:
        return [p for p in self.peers.values()
                if p.detector.available() and p.excluded_until_round < self.round]

    def state(self) -> dict:
        return {"self": self.self_id, "round": self.round, "peers": [
            {"id": p.node_id, "addr": p.addr, "models": p.models, "load": p.load, "tok_per_s": p.tok_per_s,
             "prefill_tok_per_s": p.prefill_tok_per_s,
             "phi": round(p.detector.phi(), 3), "alive": p.detector.available(), "rtt_ms": p.rtt_ms,
             "layer_cost": p.layer_cost, "card_bytes_free": p.card_bytes_free,
             "excluded": p.excluded_until_round >= self.round} for p in self.peers.values()]}

    def gossip_payload(self, self_addr: str, models, load, tok_per_s, free_kv_blocks, layer_cost=None,
                       card_bytes_free: int = 0, prefill_tok_per_s: float = 0.0) -> dict:
        return {"id": self.self_id, "addr": self_addr, "models": list(models), "load": load, "tok_per_s": tok_per_s,
                "prefill_tok_per_s": prefill_tok_per_s,
                "free_kv_blocks": free_kv_blocks, "layer_cost": layer_cost or {}, "card_bytes_free": int(card_bytes_free),
                "known": [{"id": p.node_id, "addr": p.addr, "incarnation": p.incarnation} for p in self.alive()]}
