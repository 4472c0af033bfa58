"""Per-request figures: the energy ledger's split rule, the `loken` object, and its place in the
OpenAI / Messages answers, with the prompt-reading progress comment of a stream."""
import json

from fastapi.testclient import TestClient

from loken_b200.api.common import ModelRegistry
from loken_b200.api.server import create_app
from loken_b200.utils.figures import EnergyLedger, RequestFigures, sum_figures
from tests.fakes import fake_llm


def test_energy_is_split_by_tokens_computed_between_readings():
    gpu, cpu = [100.0], [10.0]
    led = EnergyLedger(lambda: gpu[0], lambda: cpu[0])
    a, b = RequestFigures(), RequestFigures()
    led.open(a)                         # reading 1
    led.note_tokens(a, 10)
    gpu[0], cpu[0] = 130.0, 12.0
    led.open(b)                         # reading 2: 30 J GPU, 2 J CPU, all a's (only a was active)
    assert a.gpu_joules == 30.0 and a.cpu_joules == 2.0 and a.shared and b.shared
    led.note_tokens(a, 30)
    led.note_tokens(b, 10)
    gpu[0], cpu[0] = 170.0, 16.0
    led.close(a)                        # reading 3: 40 J split 3 : 1
    assert abs(a.gpu_joules - 60.0) < 1e-9 and abs(b.gpu_joules - 10.0) < 1e-9
    assert abs(a.cpu_joules - 5.0) < 1e-9 and abs(b.cpu_joules - 1.0) < 1e-9
    gpu[0] = 180.0
    led.close(b)                        # no token since the last reading: split evenly among the active (b alone)
    assert abs(b.gpu_joules - 20.0) < 1e-9
    j = a.to_json()["energy"]
    assert j == {"joules": 65.0, "gpu_joules": 60.0, "cpu_joules": 5.0, "estimated": False, "share": "work"}
    # no CPU counter: cpu_joules null and the figure is marked estimated; no meter at all: no energy field
    led2 = EnergyLedger(lambda: gpu[0], None)
    c = RequestFigures()
    led2.open(c)
    gpu[0] = 185.0
    led2.close(c)
    e = c.to_json()["energy"]
    assert e["gpu_joules"] == 5.0 and e["cpu_joules"] is None and e["estimated"] is True and e["share"] == "alone"
    d = RequestFigures()
    led3 = EnergyLedger()
    led3.open(d)
    led3.close(d)
    assert "energy" not in d.to_json()


def test_figures_object_and_sum():
    f = RequestFigures(arrival=10.0, prefill_start=10.002, first_token=10.5, end=12.0, kv_used=40, kv_capacity=4096)
    j = f.to_json()
    assert j == {"queue_ms": 2.0, "prefill_ms": 498.0, "decode_ms": 1500.0,
                 "kv": {"used_tokens": 40, "capacity_tokens": 4096}}
    s = sum_figures([j, {"queue_ms": 1.0, "prefill_ms": 2.0, "decode_ms": 3.0,
                         "energy": {"joules": 2.0, "gpu_joules": 2.0, "cpu_joules": None, "estimated": True,
                                    "share": "work"}, "kv": {"used_tokens": 7, "capacity_tokens": 4096}}])
    assert s["queue_ms"] == 3.0 and s["decode_ms"] == 1503.0 and s["kv"]["used_tokens"] == 7
    assert s["energy"]["share"] == "work" and s["energy"]["estimated"] is True and s["energy"]["gpu_joules"] == 2.0


def _client(**kw):
    reg = ModelRegistry()
    reg.add(fake_llm("figures reply", **kw))
    return TestClient(create_app(reg, None)), reg


def test_usage_carries_the_loken_object_on_chat_and_messages():
    c, reg = _client()
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4}).json()
    lk = r["usage"]["loken"]
    assert set(lk) >= {"queue_ms", "prefill_ms", "decode_ms", "kv"} and lk["kv"]["capacity_tokens"] == 1600
    assert lk["kv"]["used_tokens"] == r["usage"]["prompt_tokens"] + r["usage"]["completion_tokens"]
    assert lk["queue_ms"] >= 0 and lk["prefill_ms"] >= 0 and lk["decode_ms"] >= 0
    # n = 2: the figures of both generations are added
    r2 = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3,
                                              "n": 2}).json()
    assert r2["usage"]["loken"]["decode_ms"] >= 0 and len(r2["choices"]) == 2
    # stream: the usage chunk carries it
    with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                         "max_tokens": 3, "stream": True,
                                                         "stream_options": {"include_usage": True}}) as s:
        chunks = [json.loads(l[6:]) for l in s.iter_lines() if l.startswith("data: ") and l != "data: [DONE]"]
    assert "loken" in [ch for ch in chunks if ch.get("usage")][-1]["usage"]
    m = c.post("/v1/messages", json={"model": "fake-model", "max_tokens": 4,
                                     "messages": [{"role": "user", "content": "hi"}]}).json()
    assert "loken" in m["usage"] and m["usage"]["cache_read_input_tokens"] == 0


def test_stream_reports_prompt_reading_after_250_ms():
    # a slow engine: the first token comes after more than 250 ms, so the stream carries comment lines
    c, reg = _client(step_delay=0.4)
    with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hello there"}],
                                                         "max_tokens": 2, "stream": True}) as s:
        lines = list(s.iter_lines())
    comments = [l for l in lines if l.startswith(": loken-prefill ")]
    assert comments, lines[:5]
    body = json.loads(comments[0][len(": loken-prefill "):])
    assert set(body) == {"done", "total"} and 0 <= body["done"] <= body["total"] and body["total"] > 0
    # the data lines are still a well-formed stream
    assert any(l.startswith("data: ") for l in lines) and lines[-1] == "" or "data: [DONE]" in lines
    # a fast engine sends none
    c2, _ = _client()
    with c2.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                          "max_tokens": 2, "stream": True}) as s:
        assert not [l for l in s.iter_lines() if l.startswith(": loken-prefill")]
