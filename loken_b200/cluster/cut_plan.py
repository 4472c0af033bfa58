"""Where to cut a layer stack across the nodes of a cluster.

A pipeline over nodes is a chain: every node takes one contiguous run of layers, and every token pays each
boundary's crossing for as long as the model stays loaded.  Filling nodes until they are full puts cuts
wherever memory happens to end, a narrow link included; since the structure is a chain the best placement
can be computed instead (reference: `src/distributed/cut_plan.rs:1-24`, `:139`, `:382`, `:457`, `:517`).

Two rules are kept from there.  Capacity is a hard constraint: a run that does not fit its node has
infinite cost and can never appear in a plan.  And no answer beats a wrong one: when nothing fits the
planner returns None, it never hands back its least bad overflow.

The search here is one dynamic programme over (set of nodes used so far, last node, layers covered), the
inner minimum over the previous boundary done as one numpy reduction, so node subset, node order and cut
points are chosen together and exactly for up to `EXACT_NODES` nodes (the reference enumerates orderings
and runs a chain DP under each).  Beyond that the nodes are tried in one fixed order, and the plan says so
(`exact=False`).

    costs = LinkCosts.from_gbps([("a", "b", 10.0)], activation_bytes=2 * 8192).with_base_ms(0.2)
    plan  = plan_by_capacity(layer_bytes, [Node("a", 48 << 30), Node("b", 24 << 30)], costs)
    plan.segments   # [Segment("a", 0, 54), Segment("b", 54, 80)]

Three objectives share the search: `plan_by_capacity` (least crossing time among the placements that fit),
`plan_dense_by_time` (least predicted time per token of a dense stack: each layer at its node's measured
card or host time) and `plan_moe_by_time` (a mixture stack: the room a node has left after the always-read
weights holds experts, the rest of a token's experts miss to the host at the node's own price).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

EXACT_NODES = 8
INF = float("inf")


@dataclass(frozen=True)
class Node:
    id: str
    bytes: int                    # weights it can hold on its cards
    layer_ms: float = 0.0         # one layer on the cards (with the experts that are resident)
    host_ms: float = 0.0          # dense: one layer on the host; mixture: one missed expert on the host cores


class LinkCosts:
    """Milliseconds per token for an activation to cross from one node to another.  Pairs are ordered (an
    uplink may be slower than the downlink); a pair that was never given is unreachable, not free."""

    def __init__(self, ms: Optional[Dict[Tuple[str, str], float]] = None, base_ms: float = 0.0):
        self.ms = dict(ms or {})
        self.base_ms = float(base_ms)

    @classmethod
    def from_gbps(cls, pairs: Iterable[Tuple[str, str, float]], activation_bytes: int, symmetric: bool = True) -> "LinkCosts":
        """`pairs`: (a, b, GB/s).  The cost is the activation's transfer time."""
        ms = {}
        for a, b, gbps in pairs:
            t = INF if gbps <= 0 else activation_bytes / 1e9 / gbps * 1e3
            ms[(a, b)] = t
            if symmetric:
                ms.setdefault((b, a), t)
        return cls(ms)

    @classmethod
    def from_rtt_ms(cls, pairs: Iterable[Tuple[str, str, float]]) -> "LinkCosts":
        """Crossings priced from the round-trip times the membership layer already measures."""
        ms = {}
        for a, b, t in pairs:
            ms[(a, b)] = float(t)
            ms.setdefault((b, a), float(t))
        return cls(ms)

    def with_base_ms(self, base_ms: float) -> "LinkCosts":
        """A fixed cost on every crossing (latency, the receiver's per-token set-up): what makes many short
        hops dearer than their bytes."""
        return LinkCosts(self.ms, base_ms)

    def cost(self, a: str, b: str) -> float:
        if a == b:
            return 0.0
        t = self.ms.get((a, b))
        return INF if t is None else self.base_ms + t


@dataclass(frozen=True)
class Segment:
    node: str
    lo: int
    hi: int

    def __len__(self) -> int:
        return self.hi - self.lo


@dataclass
class CutPlan:
    segments: List[Segment]
    crossing_ms: float            # per token, all boundaries
    total_ms: float               # objective value: crossings, plus compute under the time models
    exact: bool = True

    def covers(self, layers: int) -> bool:
        """Every layer once, in order, no empty run: what a caller may assume before loading."""
        nxt = 0
        for s in self.segments:
            if s.lo != nxt or s.hi <= s.lo:
                return False
            nxt = s.hi
        return nxt == layers

    def node_of(self, layer: int) -> Optional[str]:
        for s in self.segments:
            if s.lo <= layer < s.hi:
                return s.node
        return None

    def to_json(self) -> dict:
        return {"segments": [{"node": s.node, "from": s.lo, "to": s.hi} for s in self.segments],
                "crossing_ms": self.crossing_ms, "total_ms": self.total_ms, "exact": self.exact}


# ---- the search ---------------------------------------------------------------------------------------------
def _search(L: int, nodes: Sequence[Node], costs: LinkCosts, run_cost: Callable[[int], np.ndarray],
            clean: Optional[Callable[[int], bool]] = None, first: Optional[int] = None) -> Optional[CutPlan]:
    """Least sum of run costs and crossings.  `run_cost(j)` is an (L+1, L+1) array: entry [k, i] is the cost of
    node j running layers [k, i) (inf where it cannot; entries with k >= i are ignored)."""
    n = len(nodes)
    if L <= 0 or n == 0:
        return None
    upper = np.triu(np.ones((L + 1, L + 1), dtype=bool), 1)                   # k < i
    C = []
    for j in range(n):
        c = np.where(upper, np.asarray(run_cost(j), dtype=np.float64), INF)
        if clean is not None:
            for k in range(1, L):
                if not clean(k):
                    c[k, :] = INF          # no run may start ...
                    c[:, k] = INF          # ... or end at a boundary that is not clean
        C.append(c)
    X = np.array([[costs.cost(a.id, b.id) for b in nodes] for a in nodes])
    if n > EXACT_NODES:
        return _search_fixed_order(L, nodes, X, C, first)

    # dp[(mask, last)] = vector over i: least cost of covering [0, i) with the nodes of `mask`, `last` holding the end
    dp: Dict[Tuple[int, int], np.ndarray] = {}
    back: Dict[Tuple[int, int], Tuple[np.ndarray, np.ndarray]] = {}
    for j in range(n):
        if first is not None and j != first:
            continue
        v = C[j][0, :].copy()
        v[0] = INF
        dp[(1 << j, j)] = v
    best: Tuple[float, Optional[Tuple[int, int]]] = (INF, None)
    for mask in range(1, 1 << n):
        for last in range(n):
            v = dp.get((mask, last))
            if v is None:
                continue
            if v[L] < best[0]:
                best = (float(v[L]), (mask, last))
            if not np.isfinite(v).any():
                continue
            for nx in range(n):
                if mask >> nx & 1 or not math.isfinite(X[last, nx]):
                    continue
                cand = v[:, None] + X[last, nx] + C[nx]                       # [k, i]
                ks = cand.argmin(0)
                nv = cand[ks, np.arange(L + 1)]
                key = (mask | 1 << nx, nx)
                old = dp.get(key)
                if old is None:
                    dp[key] = nv
                    back[key] = (np.full(L + 1, last), ks)
                else:
                    better = nv < old
                    if better.any():
                        old[better] = nv[better]
                        bl, bk = back[key]
                        bl[better] = last
                        bk[better] = ks[better]
    if best[1] is None or not math.isfinite(best[0]):
        return None
    segs, crossing = [], 0.0
    (mask, last), i = best[1], L
    while True:
        key = (mask, last)
        if key in back and mask != 1 << last:
            prev, k = int(back[key][0][i]), int(back[key][1][i])
            segs.append(Segment(nodes[last].id, k, i))
            crossing += float(X[prev, last])
            mask, last, i = mask & ~(1 << last), prev, k
        else:
            segs.append(Segment(nodes[last].id, 0, i))
            break
    segs.reverse()
    return CutPlan(segs, crossing, best[0], exact=True)


def _search_fixed_order(L, nodes, X, C, first) -> Optional[CutPlan]:
    """Chain DP under one ordering (largest node first, `first` in front): a node may be skipped."""
    order = sorted(range(len(nodes)), key=lambda j: -nodes[j].bytes)
    if first is not None:
        order.remove(first)
        order.insert(0, first)
    # state: (position in order of the last used node) -> vector over i
    vecs: List[Optional[np.ndarray]] = [None] * len(order)
    backs: List[Optional[Tuple[np.ndarray, np.ndarray]]] = [None] * len(order)
    best = (INF, -1)
    for p, j in enumerate(order):
        if first is None or p == 0:
            v = C[j][0, :].copy()
            v[0] = INF
            vecs[p], backs[p] = v, (np.full(L + 1, -1), np.zeros(L + 1, dtype=np.int64))
        for q in range(p):
            if vecs[q] is None or not math.isfinite(X[order[q], j]):
                continue
            cand = vecs[q][:, None] + X[order[q], j] + C[j]
            ks = cand.argmin(0)
            nv = cand[ks, np.arange(L + 1)]
            if vecs[p] is None:
                vecs[p], backs[p] = nv, (np.full(L + 1, q), ks)
            else:
                better = nv < vecs[p]
                vecs[p][better] = nv[better]
                backs[p][0][better] = q
                backs[p][1][better] = ks[better]
        if vecs[p] is not None and vecs[p][L] < best[0]:
            best = (float(vecs[p][L]), p)
    if best[1] < 0 or not math.isfinite(best[0]):
        return None
    segs, crossing, p, i = [], 0.0, best[1], L
    while p >= 0:
        q, k = int(backs[p][0][i]), int(backs[p][1][i])
        segs.append(Segment(nodes[order[p]].id, k if q >= 0 else 0, i))
        if q >= 0:
            crossing += float(X[order[q], order[p]])
        p, i = q, k
    segs.reverse()
    return CutPlan(segs, crossing, best[0], exact=False)


def _prefix(values: Sequence[int]) -> np.ndarray:
    p = np.zeros(len(values) + 1, dtype=np.float64)
    p[1:] = np.cumsum(np.asarray(values, dtype=np.float64))
    return p


# ---- the three objectives -----------------------------------------------------------------------------------
def plan_by_capacity(layer_bytes: Sequence[int], nodes: Sequence[Node], costs: LinkCosts) -> Optional[CutPlan]:
    """The placement that fits every node and spends the least time per token on crossings; None when none fits."""
    L = len(layer_bytes)
    pre = _prefix(layer_bytes)
    size = pre[None, :] - pre[:, None]                                        # [k, i] bytes of layers [k, i)

    def run(j):
        return np.where(size <= nodes[j].bytes, 0.0, INF)

    return _search(L, nodes, costs, run)


def plan_dense_by_time(layer_bytes: Sequence[int], head_bytes: int, nodes: Sequence[Node], first: int,
                       costs: LinkCosts) -> Optional[CutPlan]:
    """Least predicted time per token for a dense stack that starts on `nodes[first]` (the node holding the
    request).  A node's run fills its cards in order at `layer_ms` each (the output head's bytes set aside on
    the node that ends the stack); what does not fit runs on its host at `host_ms`, which a node that
    measured no host path reports as zero and so cannot take."""
    L = len(layer_bytes)
    if L == 0 or not 0 <= first < len(nodes):
        return None
    pre = _prefix(layer_bytes)

    def run(j):
        nd = nodes[j]
        c = np.full((L + 1, L + 1), INF)
        for k in range(L):
            for tail in (False, True):
                room = nd.bytes - (head_bytes if tail else 0)
                fit = 0                    # layers of the run that stay on the cards: its longest prefix that fits
                if nd.layer_ms > 0 and room >= 0:
                    fit = max(0, int(np.searchsorted(pre, pre[k] + room, side="right")) - 1 - k)
                cols = [L] if tail else range(k + 1, L)
                for i in cols:
                    on_card = min(fit, i - k)
                    on_host = i - k - on_card
                    if on_host and nd.host_ms <= 0:
                        continue
                    c[k, i] = on_card * nd.layer_ms + on_host * nd.host_ms
        return c

    return _search(L, nodes, costs, run, first=first)


def resident_experts(resident_bytes: Sequence[int], room: int, expert_bytes: int, working_set: int) -> int:
    """Experts a run of layers keeps on the cards: the room left after the always-read weights, never more
    than the run routes over (`working_set` per layer)."""
    if not len(resident_bytes) or expert_bytes <= 0:
        return 0
    left = max(0, room - int(sum(resident_bytes)))
    return min(left // expert_bytes, working_set * len(resident_bytes))


def moe_run_ms(resident_bytes: Sequence[int], node: Node, expert_bytes: int, working_set: int, activated: int) -> float:
    """Predicted time per token of a node running these layers of a mixture stack.  Coverage = the resident
    share of the working set (a floor: routing is concentrated); the covered experts ride in `layer_ms`, the
    rest miss to the cores at `host_ms` each.  Card and core time add: a cut is never rewarded for an overlap
    it may not get."""
    n = len(resident_bytes)
    if n == 0 or working_set == 0:
        return 0.0
    if int(sum(resident_bytes)) > node.bytes:
        return INF                                                            # the always-read weights alone do not fit
    held = resident_experts(resident_bytes, node.bytes, expert_bytes, working_set)
    coverage = min(1.0, held / n / working_set)
    misses = activated * n * (1.0 - coverage)
    if misses > 0 and node.host_ms <= 0:
        return INF                                                            # no host path was measured on this node
    return n * node.layer_ms + misses * node.host_ms


def plan_moe_by_time(resident_per_layer: Sequence[int], expert_bytes: int, working_set: int, activated: int,
                     nodes: Sequence[Node], costs: LinkCosts, clean: Optional[Callable[[int], bool]] = None) -> Optional[CutPlan]:
    """Subset, order and cuts of a mixture stack together; a node that would only slow the chain is left out,
    and one node alone is among the candidates (`len(plan.segments) == 1`)."""
    L = len(resident_per_layer)
    if L == 0 or expert_bytes <= 0 or not nodes:
        return None

    def run(j):
        c = np.full((L + 1, L + 1), INF)
        for k in range(L):
            for i in range(k + 1, L + 1):
                c[k, i] = moe_run_ms(resident_per_layer[k:i], nodes[j], expert_bytes, working_set, activated)
        return c

    return _search(L, nodes, costs, run, clean=clean)


def residency_cut(resident_per_layer: Sequence[int], expert_bytes: int, working_set: int, node_bytes: Tuple[int, int],
                  clean: Optional[Callable[[int], bool]] = None) -> Optional[int]:
    """Two nodes, no timings yet: the clean boundary that keeps the most experts resident over both nodes; on
    a tie the longer head, so the tail (the smaller node, by convention) runs fewer layers.  Returns the
    head's layer count."""
    n = len(resident_per_layer)
    if n == 0 or expert_bytes <= 0:
        return None
    best = None
    for cut in range(1, n):
        if clean is not None and not clean(cut):
            continue
        held = (resident_experts(resident_per_layer[:cut], node_bytes[0], expert_bytes, working_set)
                + resident_experts(resident_per_layer[cut:], node_bytes[1], expert_bytes, working_set))
        if best is None or (held, cut) > best:
            best = (held, cut)
    return None if best is None else best[1]


# ---- from what a cluster knows --------------------------------------------------------------------------------
def layer_bytes_of(cfg, weight_bits: float = 16.0, kv_tokens: int = 0, kv_bytes_per_value: float = 1.0625) -> List[int]:
    """Bytes of each layer of a decoder described by `cfg` (weights at `weight_bits` per value, plus the cache
    of `kv_tokens` positions), for planning before any file is read."""
    hd = cfg.head_dim
    attn = cfg.hidden * (cfg.n_q + 2 * cfg.n_kv) * hd + cfg.n_q * hd * cfg.hidden
    if cfg.n_experts > 0:
        ffn = cfg.n_experts * 3 * cfg.hidden * cfg.expert_intermediate + cfg.hidden * cfg.n_experts
    else:
        ffn = 3 * cfg.hidden * cfg.intermediate
    w = int((attn + ffn) * weight_bits / 8) + 2 * cfg.hidden * 2
    kv = int(2 * cfg.n_kv * hd * kv_tokens * kv_bytes_per_value)
    return [w + kv] * cfg.n_layers


def costs_from_peers(self_id: str, peers: Iterable, activation_bytes: int, base_ms: float = 0.0) -> LinkCosts:
    """Link prices from the membership table: each peer's measured round trip to this node (`rtt_ms`) and,
    where known, its link rate (`link_gbps`).  Links between two other nodes are priced by the slower of
    their two links to this one (traffic between them crosses both unless they report otherwise)."""
    mine: Dict[str, float] = {}
    for p in peers:
        rtt = getattr(p, "rtt_ms", None)
        gbps = getattr(p, "link_gbps", None)
        t = 0.0
        if gbps:
            t += activation_bytes / 1e9 / gbps * 1e3
        if rtt:
            t += rtt / 2.0
        if gbps or rtt:
            mine[p.node_id] = t
    ms: Dict[Tuple[str, str], float] = {}
    for a, ta in mine.items():
        ms[(self_id, a)] = ms[(a, self_id)] = ta
        for b, tb in mine.items():
            if a != b:
                ms[(a, b)] = max(ta, tb)
    return LinkCosts(ms, base_ms)


def _size(v) -> int:
    """42, "48G", "512M": bytes."""
    if isinstance(v, (int, float)):
        return int(v)
    s = str(v).strip().upper().rstrip("B").rstrip("I")
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30, "T": 1 << 40}.get(s[-1:], 1)
    return int(float(s[:-1] if mult > 1 else s) * mult)


def plan_from_request(body: dict) -> Optional[CutPlan]:
    """The planner behind `POST /api/cluster/plan` and `loken plan-cut`:

        {"layers": 80, "layer_bytes": "850M" | [..], "head_bytes": "2G",
         "nodes": [{"id": "a", "bytes": "48G", "layer_ms": 0.4, "host_ms": 3.0}, ...],
         "links": [{"from": "a", "to": "b", "gbps": 10} | {"from": "a", "to": "b", "ms": 0.8}],
         "activation_bytes": 16384, "base_ms": 0.2,
         "objective": "capacity" | "time", "first": "a",
         "experts": {"bytes": "25M", "working_set": 32, "activated": 4}}        # a mixture stack, objective "time"

    Raises ValueError on a body that names no nodes or layers."""
    nodes = [Node(str(n["id"]), _size(n.get("bytes", 0)), float(n.get("layer_ms", 0.0)), float(n.get("host_ms", 0.0)))
             for n in body.get("nodes", [])]
    if not nodes:
        raise ValueError("a plan needs nodes: [{id, bytes, ...}]")
    if len({n.id for n in nodes}) != len(nodes):
        raise ValueError("node ids must differ")
    lb = body.get("layer_bytes")
    if isinstance(lb, list):
        layer_bytes = [_size(x) for x in lb]
    elif lb is not None and body.get("layers"):
        layer_bytes = [_size(lb)] * int(body["layers"])
    else:
        raise ValueError("a plan needs layer_bytes (a list, or one size with layers)")
    act = int(body.get("activation_bytes", 0))
    ms: Dict[Tuple[str, str], float] = {}
    for ln in body.get("links", []):
        a, b = str(ln["from"]), str(ln["to"])
        if "ms" in ln:
            t = float(ln["ms"])
        else:
            g = float(ln.get("gbps", 0.0))
            t = INF if g <= 0 else act / 1e9 / g * 1e3
        ms[(a, b)] = t
        if not ln.get("one_way"):
            ms.setdefault((b, a), t)
    costs = LinkCosts(ms, float(body.get("base_ms", 0.0)))
    objective = body.get("objective", "capacity")
    if objective == "capacity":
        return plan_by_capacity(layer_bytes, nodes, costs)
    if objective != "time":
        raise ValueError("objective is capacity or time")
    ex = body.get("experts")
    if ex:
        return plan_moe_by_time(layer_bytes, _size(ex["bytes"]), int(ex["working_set"]), int(ex["activated"]), nodes, costs)
    ids = [n.id for n in nodes]
    first = ids.index(str(body["first"])) if body.get("first") is not None else 0
    return plan_dense_by_time(layer_bytes, _size(body.get("head_bytes", 0)), nodes, first, costs)
