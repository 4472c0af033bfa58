"""Requests answered by a peer and taken back when it leaves; sampling keyed by (seed, position).
Two servers live in this process; the "network" is a function, and failures are raised by it."""
import json
import random

import pytest
from fastapi.testclient import TestClient

from fakes import fake_llm
from loken_b200.api.common import ModelRegistry
from loken_b200.api.context import ServerSettings
from loken_b200.api.server import create_app
from loken_b200.cluster.forward import PeerFailed, params_from_wire, params_to_wire
from loken_b200.cluster.membership import Membership
from loken_b200.engine.llm import GenerationParams
from loken_b200.serve.replay import PositionRng, ResumePoint, path_fingerprint, uniform_at

REPLY = "The quick brown fox jumps over the lazy dog."


# ---- randomness by position ---------------------------------------------------------------------------------
def test_uniforms_depend_on_seed_and_position_only():
    seed = 0x5EED1234ABCD0001
    whole = [PositionRng(seed).random() for _ in range(1)]
    g = PositionRng(seed)
    whole = [g.random() for _ in range(200)]
    assert all(0.0 <= u < 1.0 for u in whole)
    for cut in (1, 7, 63, 128, 199):
        a = PositionRng(seed)
        head = [a.random() for _ in range(cut)]
        b = PositionRng(seed, cut)                         # a resumed request starts at the position it stopped on
        assert head + [b.random() for _ in range(200 - cut)] == whole
    # speculative verification draws for every row, then keeps the draws of the committed ones
    g = PositionRng(seed)
    st = g.getstate()
    drawn = [g.random() for _ in range(5)]
    g.setstate(st)
    for _ in range(2):
        g.random()
    assert g.random() == whole[2] and drawn == whole[:5]
    # two requests never share a stream, shifted or not (what seed + position gets wrong)
    a = [uniform_at(1000, p) for p in range(64)]
    b = [uniform_at(1001, p) for p in range(65)]
    assert a != b[:64] and a != b[1:] and len(set(a) & set(b)) == 0
    assert uniform_at(7, 3, draw=0) != uniform_at(7, 3, draw=1)
    assert abs(sum(whole) / len(whole) - 0.5) < 0.08


def test_request_generators_and_resume_points(tmp_path):
    p = GenerationParams(seed=11)
    a, b = p.rng(0), GenerationParams(seed=11, resume_position=3).rng(0)
    first = [a.random() for _ in range(6)]
    assert [b.random() for _ in range(3)] == first[3:]
    assert p.rng(1).random() != p.rng(0).random()
    with pytest.raises(ValueError):
        GenerationParams(resume_position=-1).validate()
    rp = ResumePoint(11, [1, 2, 3], [4, 5], "sha256:ab12")
    assert rp.tokens == [1, 2, 3, 4, 5] and rp.position == 2
    assert rp.may_resume_on("sha256:ab12") and not rp.may_resume_on("sha256:ab13")
    assert not ResumePoint(11, [1], [2], "").may_resume_on("")
    assert not ResumePoint(11, [1], [2], "sha256:0000").may_resume_on("sha256:0000")       # a placeholder names nothing
    assert ResumePoint.from_json(json.loads(json.dumps(rp.to_json()))) == rp
    f1, f2 = tmp_path / "a.gguf", tmp_path / "b.gguf"
    body = random.Random(0).randbytes(6 << 20)
    f1.write_bytes(body)
    f2.write_bytes(body[:3 << 20] + bytes([body[3 << 20] ^ 1]) + body[(3 << 20) + 1:])   # one byte in the middle
    assert path_fingerprint(str(f1)).startswith("fp256:") and path_fingerprint(str(f1)) == path_fingerprint(str(f1))
    assert path_fingerprint(str(f1), probes=4096, probe_bytes=1 << 10) != path_fingerprint(str(f2), probes=4096, probe_bytes=1 << 10)
    wire = params_to_wire(GenerationParams(temperature=0.3, seed=5, logit_bias={7: -1.5}, max_tokens=9, resume_position=2))
    back = params_from_wire(json.loads(json.dumps(wire)))
    assert (back.temperature, back.seed, back.logit_bias, back.max_tokens, back.resume_position) == (0.3, 5, {7: -1.5}, 9, 2)


# ---- two nodes ----------------------------------------------------------------------------------------------------
class Net:
    """B's /api/cluster/generate reached through its test client; `fail_after` lines the link breaks."""

    def __init__(self, peer_client, fail_after=None, refuse=False):
        self.peer, self.fail_after, self.refuse = peer_client, fail_after, refuse
        self.closed = 0
        self.bodies = []

    def __call__(self, addr, body, timeout_s):
        if self.refuse:
            raise ConnectionError("connection refused")
        self.bodies.append(body)
        r = self.peer.post("/api/cluster/generate", json=body)
        if r.status_code != 200:
            raise PeerFailed(f"the peer answered {r.status_code}")
        lines = [json.loads(l) for l in r.text.splitlines() if l]

        def it():
            for i, l in enumerate(lines):
                if self.fail_after is not None and i > self.fail_after:       # line 0 names the node
                    raise ConnectionError("connection reset by peer")
                yield l

        def close():
            self.closed += 1

        return it(), close


def two_nodes(fail_after=None, refuse=False, same_weights=True, **settings):
    regB = ModelRegistry()
    llmB = fake_llm(REPLY)
    regB.add(llmB)
    cB = TestClient(create_app(regB, ServerSettings(node_id="B")))
    regA = ModelRegistry()
    llmA = fake_llm(REPLY)
    regA.add(llmA)
    appA = create_app(regA, ServerSettings(node_id="A", route_requests=True, **settings))
    ctx = appA.state.ctx
    ctx.membership = Membership("A")
    ctx.membership.observe("B", "http://b:1", models=["fake-model"], load=0.0, tok_per_s=500.0)
    ctx.open_peer_stream = Net(cB, fail_after, refuse)
    llmA._digest = "fp256:aa"
    llmB._digest = "fp256:aa" if same_weights else "fp256:bb"
    return TestClient(appA), ctx, llmA, llmB


def ask(c, **kw):
    return c.post("/v1/completions", json=dict({"model": "fake-model", "prompt": "Say it", "max_tokens": 64, "seed": 3}, **kw))


def test_a_request_is_answered_by_the_faster_peer():
    cA, ctx, llmA, llmB = two_nodes()
    r = ask(cA)
    assert r.status_code == 200 and r.json()["choices"][0]["text"] == REPLY
    assert len(llmB.engine.prompts) == 1 and llmA.engine.prompts == []
    assert ctx.metrics.counters["requests_forwarded"] == 1
    sent = ctx.open_peer_stream.bodies[0]
    assert sent["params"]["seed"] == 3 and "stop" not in sent["params"]
    # a stop string is found by the asking node, which then hangs up on the peer
    r = ask(cA, stop=["brown"])
    assert r.json()["choices"][0]["text"] == "The quick " and ctx.open_peer_stream.closed >= 1
    # structured output keeps its matcher here
    r = ask(cA, response_format={"type": "json_object"})
    assert len(llmA.engine.prompts) == 1


def test_an_answer_is_continued_here_when_the_peer_leaves():
    cA, ctx, llmA, llmB = two_nodes(fail_after=5)
    r = ask(cA)
    assert r.status_code == 200 and r.json()["choices"][0]["text"] == REPLY          # the client sees one whole answer
    assert r.json()["usage"]["completion_tokens"] == len(REPLY) + 1
    # this node was given the prompt plus the five tokens the peer had sent, and the position to go on from
    assert len(llmA.engine.prompts) == 1
    prompt_b = llmB.engine.prompts[0]
    assert llmA.engine.prompts[0] == prompt_b + list(REPLY.encode()[:5])
    got = llmA.engine.params_seen[0]
    assert got.resume_position == 5 and got.max_tokens == 64 - 5 and got.seed == 3
    assert ctx.metrics.counters["requests_taken_back"] == 1
    assert ctx.membership.alive() == []                                               # the peer sits out a few rounds
    r = ask(cA)                                                                       # and the next request stays here
    assert r.json()["choices"][0]["text"] == REPLY and len(llmA.engine.prompts) == 2


def test_other_weights_may_not_continue_an_answer_unless_allowed():
    cA, ctx, llmA, llmB = two_nodes(fail_after=5, same_weights=False)
    r = ask(cA)
    assert r.status_code >= 500 or "cannot be continued" in r.text
    assert llmA.engine.prompts == []
    cA, ctx, llmA, llmB = two_nodes(fail_after=5, same_weights=False, resume_unverified=True)
    assert ask(cA).json()["choices"][0]["text"] == REPLY


def test_a_peer_that_cannot_be_reached_costs_nothing_but_the_try():
    cA, ctx, llmA, llmB = two_nodes(refuse=True, same_weights=False)
    r = ask(cA)
    assert r.json()["choices"][0]["text"] == REPLY
    assert llmA.engine.params_seen[0].resume_position == 0 and llmB.engine.prompts == []              # nothing was emitted: a plain local run


def test_streaming_through_a_peer_that_leaves():
    cA, ctx, llmA, llmB = two_nodes(fail_after=9)
    with cA.stream("POST", "/v1/chat/completions", json={"model": "fake-model", "stream": True, "seed": 1,
                                                         "messages": [{"role": "user", "content": "hi"}]}) as r:
        text = "".join(json.loads(l[6:])["choices"][0]["delta"].get("content", "")
                       for l in r.iter_lines() if l.startswith("data: {") and json.loads(l[6:])["choices"])
    assert text == REPLY


def test_the_prefix_cache_enters_the_routing_arithmetic():
    from loken_b200.cluster.routing import Router

    m = Membership("A")
    m.observe("B", "http://b", models=["m"], load=0.0, tok_per_s=100.0, prefill_tok_per_s=1000.0)
    r = Router(m)
    # equal decode rates: the hop keeps a short request at home
    assert r.choose("m", 100, 0.0, 100.0).addr is None
    # a 4000-token prompt that B already holds: reading it here costs 4 s, there nothing
    c = r.choose("m", 100, 0.0, 100.0, prompt_tokens=4000, local_cached=0, local_prefill_rate=1000.0, peer_cached={"B": 3968})
    assert c.node_id == "B"
    # held here instead: it stays
    c = r.choose("m", 100, 0.0, 100.0, prompt_tokens=4000, local_cached=3968, local_prefill_rate=1000.0, peer_cached={"B": 0})
    assert c.addr is None


def test_long_prompts_ask_the_peers_what_they_hold():
    cA, ctx, llmA, llmB = two_nodes()
    ctx.membership.observe("B", "http://b:1", models=["fake-model"], load=0.0, tok_per_s=500.0, prefill_tok_per_s=1000.0)
    asked = []
    ctx.ask_prefix = lambda addr, model, ids, salt: asked.append((addr, model, len(ids))) or 128
    ctx.settings.prefix_ask_min_tokens = 100
    r = ask(cA, prompt="x" * 150)
    assert r.status_code == 200 and asked and asked[0][:2] == ("http://b:1", "fake-model") and asked[0][2] >= 150
    asked.clear()
    ask(cA, prompt="short")
    assert asked == []


def test_figures_name_the_nodes_that_wrote_the_answer():
    cA, ctx, llmA, llmB = two_nodes()
    lk = ask(cA).json()["usage"]["loken"]
    assert lk["nodes"] == [{"node": "B", "role": "answered", "tokens": len(REPLY) + 1}] and "decode_ms" in lk
    cA, ctx, llmA, llmB = two_nodes(fail_after=5)
    lk = ask(cA).json()["usage"]["loken"]
    assert [n["role"] for n in lk["nodes"]] == ["left", "continued"] and lk["nodes"][0]["tokens"] == 5
    assert lk["nodes"][1]["tokens"] == len(REPLY) + 1 - 5 and "ConnectionError" in lk["taken_back"]
    # a plain local request carries its figures on the completions route as on the chat route
    cB, _, _, _ = two_nodes(refuse=True)
    assert "queue_ms" in ask(cB).json()["usage"]["loken"]
