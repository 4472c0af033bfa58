"""Where a request runs: here, or on a peer that holds the model and would finish it sooner.

`choose` restates the reference's routing rule (`src/distributed/routing.rs:244`): among the nodes
that serve the model and are believed alive, estimate time-to-finish = (queue ahead + this
request's expected tokens) / measured decode rate, prefer the node that already holds the
request's prefix (sticky conversations reuse their KV), and stay local unless a peer wins by a
margin that pays for the hop.  `RateMeter` is the EWMA of observed tokens per second
(`rate_meter.rs`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

from .membership import Membership


class RateMeter:
    def __init__(self, alpha: float = 0.2, initial: float = 0.0):
        self.alpha, self.rate, self.n = alpha, initial, 0

    def observe(self, tokens: int, seconds: float):
        if seconds <= 0 or tokens <= 0:
            return
        r = tokens / seconds
        self.rate = r if self.n == 0 else self.rate + self.alpha * (r - self.rate)
        self.n += 1


@dataclass
class Candidate:
    node_id: str
    addr: Optional[str]         # None = this node
    eta_s: float
    has_prefix: bool


class Router:
    def __init__(self, membership: Membership, hop_margin: float = 0.15, hop_cost_s: float = 0.02):
        self.m = membership
        self.hop_margin = hop_margin
        self.hop_cost_s = hop_cost_s
        self.sticky: Dict[str, str] = {}        # conversation key -> node id that served it last

    def choose(self, model: str, expected_tokens: int, local_load: float, local_rate: float,
               local_serves: bool = True, conversation: Optional[str] = None, *, prompt_tokens: int = 0,
               local_cached: int = 0, local_prefill_rate: float = 0.0,
               peer_cached: Optional[Dict[str, int]] = None) -> Candidate:
        """`prompt_tokens`, the tokens of it each node already holds (`local_cached`, `peer_cached`: what the peers
        answered on `/api/cluster/prefix`) and the measured prompt-reading rates put the prefix cache into the same
        arithmetic as everything else: a node that holds the prompt reads less of it, which is a smaller predicted
        completion (`src/distributed/routing.rs:13-16` of the reference)."""
        peer_cached = peer_cached or {}

        def read_s(cached: int, rate: float) -> float:
            left = max(0, prompt_tokens - cached)
            return left / rate if rate > 0 and left > 0 else 0.0

        cands: List[Candidate] = []
        if local_serves:
            rate = max(local_rate, 1e-6)
            eta = (local_load * expected_tokens + expected_tokens) / rate + read_s(local_cached, local_prefill_rate)
            cands.append(Candidate(self.m.self_id, None, eta,
                                   conversation is not None and self.sticky.get(conversation) == self.m.self_id))
        for p in self.m.alive():
            if model not in p.models or p.tok_per_s <= 0:
                continue
            eta = ((p.load * expected_tokens + expected_tokens) / p.tok_per_s + self.hop_cost_s
                   + read_s(peer_cached.get(p.node_id, 0), getattr(p, "prefill_tok_per_s", 0.0) or local_prefill_rate))
            cands.append(Candidate(p.node_id, p.addr, eta,
                                   conversation is not None and self.sticky.get(conversation) == p.node_id))
        if not cands:
            raise LookupError(f"no live node serves {model}")
        # a node holding the prefix skips most of the prefill: count that as a head start
        best = min(cands, key=lambda c: c.eta_s * (0.5 if c.has_prefix else 1.0))
        local = next((c for c in cands if c.addr is None), None)
        if local is not None and best is not local:
            if best.eta_s * (0.5 if best.has_prefix else 1.0) > local.eta_s * (1.0 - self.hop_margin):
                best = local
        if conversation is not None:
            self.sticky[conversation] = best.node_id
        return best

    def failed(self, node_id: str):
        """The chosen peer did not answer: exclude it for a while; the caller retries once."""
        self.m.exclude(node_id)
        for k in [k for k, v in self.sticky.items() if v == node_id]:
            del self.sticky[k]
