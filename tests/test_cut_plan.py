"""The pipeline cut planner against brute force and against the properties it promises: capacity is hard,
"nothing fits" is an answer, narrow links are avoided, slow nodes are dropped."""
import itertools
import random

import pytest

from loken_b200.cluster.cut_plan import (INF, LinkCosts, Node, costs_from_peers, layer_bytes_of, moe_run_ms, plan_by_capacity,
                                         plan_dense_by_time, plan_moe_by_time, residency_cut, resident_experts)


def brute_capacity(layer_bytes, nodes, costs):
    """Every subset, order and cut list; returns the least crossing cost or None."""
    L, best = len(layer_bytes), None
    for r in range(1, len(nodes) + 1):
        for order in itertools.permutations(range(len(nodes)), r):
            for cuts in itertools.combinations(range(1, L), r - 1):
                bounds = (0,) + cuts + (L,)
                ok, cost = True, 0.0
                for s, j in enumerate(order):
                    if sum(layer_bytes[bounds[s]:bounds[s + 1]]) > nodes[j].bytes:
                        ok = False
                        break
                    if s:
                        cost += costs.cost(nodes[order[s - 1]].id, nodes[j].id)
                if ok and cost < INF and (best is None or cost < best):
                    best = cost
    return best


def test_capacity_plan_equals_brute_force_on_random_cases():
    rng = random.Random(7)
    for case in range(40):
        L = rng.randint(2, 7)
        layers = [rng.randint(1, 9) for _ in range(L)]
        n = rng.randint(1, 4)
        nodes = [Node(f"n{j}", rng.randint(3, 20)) for j in range(n)]
        pairs = [(f"n{a}", f"n{b}", rng.choice([0.5, 1.0, 3.0, 9.0])) for a in range(n) for b in range(a + 1, n) if rng.random() < 0.85]
        costs = LinkCosts.from_rtt_ms(pairs).with_base_ms(rng.choice([0.0, 0.25]))
        want = brute_capacity(layers, nodes, costs)
        got = plan_by_capacity(layers, nodes, costs)
        if want is None:
            assert got is None, (case, layers, nodes)
            continue
        assert got is not None and got.covers(L)
        assert got.crossing_ms == pytest.approx(want), (case, layers, nodes, got)
        byid = {nd.id: nd for nd in nodes}
        for s in got.segments:
            assert sum(layers[s.lo:s.hi]) <= byid[s.node].bytes            # never an overflow
        assert len({s.node for s in got.segments}) == len(got.segments)     # a node holds one run


def test_nothing_fits_is_none_and_one_node_needs_no_link():
    costs = LinkCosts()
    assert plan_by_capacity([5, 5, 5], [Node("a", 9), Node("b", 4)], LinkCosts.from_rtt_ms([("a", "b", 1.0)])) is None
    p = plan_by_capacity([5, 5], [Node("a", 10)], costs)
    assert p.segments[0].node == "a" and p.crossing_ms == 0 and p.covers(2)
    assert plan_by_capacity([5, 5], [Node("a", 6), Node("b", 6)], costs) is None          # no link between them: unreachable
    assert plan_by_capacity([], [Node("a", 6)], costs) is None


def test_the_narrow_link_is_not_cut():
    # three nodes in a row; b-c is the slow link.  A greedy fill would use a, b, c; the plan avoids crossing b-c
    layers = [10] * 12
    nodes = [Node("a", 60), Node("b", 60), Node("c", 60)]
    costs = LinkCosts.from_gbps([("a", "b", 10.0), ("b", "c", 0.1), ("a", "c", 10.0)], activation_bytes=16384)
    p = plan_by_capacity(layers, nodes, costs)
    assert p.covers(12) and len(p.segments) == 2
    used = [s.node for s in p.segments]
    assert not ({"b", "c"} <= set(used))
    # asymmetric fabric: only a -> b is cheap
    costs = LinkCosts({("a", "b"): 0.1, ("b", "a"): 5.0})
    p = plan_by_capacity([10] * 8, [Node("b", 50), Node("a", 50)], costs)
    assert [s.node for s in p.segments] == ["a", "b"]


def test_many_nodes_fall_back_to_a_fixed_order_and_say_so():
    n = 11
    nodes = [Node(f"n{j}", 30 + j) for j in range(n)]
    pairs = [(f"n{a}", f"n{b}", 1.0) for a in range(n) for b in range(a + 1, n)]
    p = plan_by_capacity([10] * 20, nodes, LinkCosts.from_rtt_ms(pairs))
    assert p is not None and not p.exact and p.covers(20)
    byid = {nd.id: nd.bytes for nd in nodes}
    assert all(10 * len(s) <= byid[s.node] for s in p.segments)
    assert len(p.segments) >= 5                                          # 200 bytes over nodes of at most 40


def test_dense_time_plan_drops_a_slow_node_and_keeps_the_first():
    layers = [100] * 10
    fast, slow = Node("fast", 2000, layer_ms=1.0), Node("slow", 2000, layer_ms=5.0)
    costs = LinkCosts.from_rtt_ms([("fast", "slow", 0.5)])
    p = plan_dense_by_time(layers, 50, [fast, slow], 0, costs)
    assert [s.node for s in p.segments] == ["fast"] and p.total_ms == pytest.approx(10.0)
    # the request sits on the slow node: it must start the chain, hands over after one layer
    p = plan_dense_by_time(layers, 50, [fast, slow], 1, costs)
    assert [(s.node, s.lo, s.hi) for s in p.segments] == [("slow", 0, 1), ("fast", 1, 10)]
    assert p.total_ms == pytest.approx(5.0 + 0.5 + 9.0)
    # memory forces a split: the head's 50 bytes count on the node that ends the stack
    small = Node("fast", 600, layer_ms=1.0)
    p = plan_dense_by_time(layers, 50, [small, slow], 0, costs)
    assert p.covers(10) and p.segments[0].node == "fast" and len(p.segments[0]) == 6
    # a host path lets one node keep everything when the link is dear
    hosty = Node("fast", 600, layer_ms=1.0, host_ms=2.0)
    p = plan_dense_by_time(layers, 50, [hosty, slow], 0, LinkCosts.from_rtt_ms([("fast", "slow", 50.0)]))
    assert [s.node for s in p.segments] == ["fast"] and p.total_ms == pytest.approx(5 * 1.0 + 5 * 2.0)
    assert plan_dense_by_time(layers, 50, [small], 0, costs) is None


def test_moe_time_model_and_plans():
    res = [10] * 8
    assert resident_experts(res[:4], 100, 5, 4) == 12                       # 60 bytes of room / 5, under the cap of 16
    assert resident_experts(res[:4], 1000, 5, 4) == 16                      # never more than the run routes over
    strong = Node("s", 10_000, layer_ms=1.0, host_ms=3.0)
    weak = Node("w", 120, layer_ms=1.0, host_ms=20.0)
    assert moe_run_ms(res, strong, 5, 4, 2) == pytest.approx(8.0)           # everything resident: no misses
    assert moe_run_ms(res, weak, 5, 4, 2) == pytest.approx(8 * 1.0 + 2 * 8 * (1 - 8 / 8 / 4) * 20.0)
    assert moe_run_ms(res, Node("x", 50), 5, 4, 2) == INF                   # the always-read weights do not fit
    costs = LinkCosts.from_rtt_ms([("s", "w", 0.3)])
    p = plan_moe_by_time(res, 5, 4, 2, [strong, weak], costs)
    assert [s.node for s in p.segments] == ["s"]                            # splitting only adds a crossing
    # two equal nodes that each cover half the experts: splitting doubles coverage
    a, b = Node("a", 40 + 5 * 16, layer_ms=1.0, host_ms=4.0), Node("b", 40 + 5 * 16, layer_ms=1.0, host_ms=4.0)
    p = plan_moe_by_time(res, 5, 4, 2, [a, b], LinkCosts.from_rtt_ms([("a", "b", 0.3)]))
    assert len(p.segments) == 2 and p.segments[0].hi == 4
    # only clean boundaries may be cut
    p = plan_moe_by_time(res, 5, 4, 2, [a, b], LinkCosts.from_rtt_ms([("a", "b", 0.3)]), clean=lambda k: k in (2, 6))
    assert len(p.segments) == 2 and p.segments[0].hi in (2, 6)


def test_residency_cut():
    res = [10] * 6
    assert residency_cut(res, 5, 4, (200, 60)) == 5                         # the big node takes all but one layer
    assert residency_cut(res, 5, 4, (200, 200)) == 5                        # tie between cuts: the longer head
    assert residency_cut(res, 5, 4, (200, 200), clean=lambda k: k == 2) == 2
    assert residency_cut(res, 5, 4, (200, 200), clean=lambda k: False) is None
    assert residency_cut([], 5, 4, (1, 1)) is None


def test_inputs_from_the_cluster():
    from types import SimpleNamespace as NS

    from loken_b200.models.config import get_config

    cfg = get_config("llama-3.1-8b")
    lb = layer_bytes_of(cfg, weight_bits=4.5, kv_tokens=4096)
    assert len(lb) == 32 and 100e6 < lb[0] < 200e6
    peers = [NS(node_id="p1", rtt_ms=0.4, link_gbps=12.5), NS(node_id="p2", rtt_ms=2.0, link_gbps=1.0), NS(node_id="p3", rtt_ms=None, link_gbps=None)]
    c = costs_from_peers("me", peers, activation_bytes=8192)
    assert c.cost("me", "p1") < c.cost("me", "p2") and c.cost("p1", "p2") == c.cost("me", "p2")
    assert c.cost("me", "p3") == INF and c.cost("me", "me") == 0.0


def test_request_form_cli_and_route(tmp_path):
    import io
    import json

    from loken_b200.cli import loken
    from loken_b200.cluster.cut_plan import plan_from_request

    spec = {"layers": 10, "layer_bytes": "1G", "nodes": [{"id": "a", "bytes": "6G"}, {"id": "b", "bytes": "6G"}, {"id": "c", "bytes": "6G"}],
            "links": [{"from": "a", "to": "b", "gbps": 10}, {"from": "b", "to": "c", "gbps": 0.05}, {"from": "a", "to": "c", "gbps": 10}],
            "activation_bytes": 16384, "base_ms": 0.1}
    plan = plan_from_request(spec)
    assert plan.covers(10) and len(plan.segments) == 2 and not {"b", "c"} <= {s.node for s in plan.segments}
    f = tmp_path / "spec.json"
    f.write_text(json.dumps(spec))
    out = io.StringIO()
    assert loken.main(["plan-cut", str(f)], out=out) == 0
    assert "layers   0 .." in out.getvalue() and "crossings" in out.getvalue()
    spec["nodes"] = spec["nodes"][:1]
    f.write_text(json.dumps(spec))
    assert loken.main(["plan-cut", str(f)], out=io.StringIO()) == 1                   # nothing fits
    with pytest.raises(ValueError):
        plan_from_request({"nodes": []})
    timed = {"layer_bytes": [100] * 10, "head_bytes": 50, "objective": "time", "first": "slow",
             "nodes": [{"id": "fast", "bytes": 2000, "layer_ms": 1.0}, {"id": "slow", "bytes": 2000, "layer_ms": 5.0}],
             "links": [{"from": "fast", "to": "slow", "ms": 0.5}]}
    assert [s.node for s in plan_from_request(timed).segments] == ["slow", "fast"]
    moe = dict(timed, experts={"bytes": 5, "working_set": 4, "activated": 2}, layer_bytes=[10] * 8)
    moe["nodes"] = [{"id": "s", "bytes": 10000, "layer_ms": 1.0, "host_ms": 3.0}, {"id": "w", "bytes": 120, "layer_ms": 1.0, "host_ms": 20.0}]
    moe["links"] = [{"from": "s", "to": "w", "ms": 0.3}]
    assert [s.node for s in plan_from_request(moe).segments] == ["s"]
