"""Operational routes that describe the node to its peers and its operator, and the blob upload of the Ollama
dialect: host logic over the fake engine."""
import hashlib
import json
import os

from fastapi.testclient import TestClient

from fakes import fake_llm
from loken_b200.api.common import ModelRegistry
from loken_b200.api.context import ServerSettings
from loken_b200.api.server import create_app
from loken_b200.cluster.gossip import GossipLoop, fold
from loken_b200.cluster.membership import Membership


def client(settings=None):
    reg = ModelRegistry()
    llm = fake_llm()
    reg.add(llm)
    app = create_app(reg, settings or ServerSettings(node_id="n1"))
    return TestClient(app), app.state.ctx, llm


def test_peers_prefix_measure_and_status():
    c, ctx, llm = client()
    r = c.get("/api/cluster/peers").json()
    assert r["clustered"] is False and r["peers"][0]["is_self"] and r["peers"][0]["node_id"] == "n1"
    ctx.membership.observe("n2", "http://n2:1", models=["fake-model"], load=1.0, tok_per_s=90.0,
                           layer_cost={"fake-model": {"card_ms": 0.2, "host_ms": 0.0, "card_bytes": 10}}, card_bytes_free=1 << 30)
    ctx.membership.timed("n2", 4.0)
    ctx.membership.timed("n2", 2.0)
    tags = c.get("/api/tags").json()["models"]
    assert [t.get("node") for t in tags] == [None, "n2"] and tags[1]["endpoint"] == "http://n2:1"
    r = c.get("/api/cluster/peers").json()
    p2 = [p for p in r["peers"] if p["node_id"] == "n2"][0]
    assert r["clustered"] and p2["alive"] and 2.0 < p2["rtt_ms"] < 4.0 and p2["state"]["layer_cost"]["fake-model"]["card_ms"] == 0.2
    # prefix: nothing cached, then three full blocks after a sequence published them
    toks = list(range(50))
    assert c.post("/api/cluster/prefix", json={"model": "fake-model", "prompt": toks}).json()["cached_tokens"] == 0
    alloc = llm.engine.alloc
    alloc.allocate_with_prefix(7, toks)
    alloc.commit_prefix(7, toks)
    alloc.free(7)
    assert c.post("/api/cluster/prefix", json={"model": "fake-model", "prompt": toks}).json() == {"cached_tokens": 48, "prompt_tokens": 50}
    assert c.post("/api/cluster/prefix", json={"model": "fake-model", "prompt": toks, "cache_salt": "x"}).json()["cached_tokens"] == 0
    assert c.post("/api/cluster/prefix", json={"model": "absent", "prompt": "hi"}).json() == {"cached_tokens": 0}
    # measure: the engine's per-layer time, published with the node's state
    m = c.post("/api/cluster/measure", json={"model": "fake-model"}).json()
    assert m["card_ms"] == 0.1 and m["host_ms"] == 0.0 and m["card_bytes"] > 0
    assert c.get("/api/cluster/state").json()["self_state"]["layer_cost"]["fake-model"]["card_ms"] == 0.1
    # a plan over this node and its peer from what both published: the peer is slower per layer and a hop away
    assert c.post("/api/cluster/plan", json={"model": "other"}).status_code == 409
    plan = c.post("/api/cluster/plan", json={"model": "fake-model", "self_bytes": 1 << 30}).json()
    assert [s["node"] for s in plan["segments"]] == ["n1"] and plan["crossing_ms"] == 0
    tight = c.post("/api/cluster/plan", json={"model": "fake-model", "self_bytes": m["card_bytes"] + 10}).json()
    assert [s["node"] for s in tight["segments"]] == ["n1", "n2"] and tight["segments"][0]["to"] == 1
    st = c.get("/api/multi-device/status").json()["models"][0]
    assert st["model"] == "fake-model" and st["tp"] == 1 and st["kv_blocks"] == 100 and st["disk_tier"] is None
    ds = c.get("/api/distributed/stats").json()
    assert ds["node"] == "n1" and ds["models"] == ["fake-model"] and ds["peers_alive"] == 1
    assert c.get("/api/distributed/recommend").json()["model"] is None


def test_gossip_carries_costs_and_times_the_round_trip():
    a, b = Membership("a"), Membership("b")
    desc = lambda: {"models": ["m"], "load": 0.0, "tok_per_s": 10.0, "free_kv_blocks": 5,
                    "layer_cost": {"m": {"card_ms": 0.3, "host_ms": 0.0, "card_bytes": 7}}, "card_bytes_free": 99}

    def post(url, payload, timeout):
        fold(b, payload)
        return b.gossip_payload("http://b", ["m"], 0.0, 20.0, 6, {"m": {"card_ms": 0.5, "host_ms": 0.0, "card_bytes": 7}}, 11)

    loop = GossipLoop(a, "http://a", ["http://b"], desc, post=post)
    loop.round()
    assert b.peers["a"].layer_cost["m"]["card_ms"] == 0.3 and b.peers["a"].card_bytes_free == 99
    assert a.peers["b"].layer_cost["m"]["card_ms"] == 0.5 and a.peers["b"].rtt_ms is not None and a.peers["b"].rtt_ms >= 0


def test_blob_upload_and_create_from_it(tmp_path):
    from loken_b200.store.catalogue import Catalogue

    c, ctx, llm = client()
    ctx.catalogue = Catalogue([str(tmp_path / "store")], [])
    data = os.urandom(70000)
    dg = "sha256:" + hashlib.sha256(data).hexdigest()
    assert c.head(f"/api/blobs/{dg}").status_code == 404
    assert c.post(f"/api/blobs/{dg}", content=data[:-1] + bytes([data[-1] ^ 1])).status_code == 400          # wrong bytes are not kept
    assert c.head(f"/api/blobs/{dg}").status_code == 404
    assert c.post(f"/api/blobs/{dg}", content=data).status_code == 201
    assert c.head(f"/api/blobs/{dg}").status_code == 200 and c.post(f"/api/blobs/{dg}", content=data).status_code == 200
    assert c.post("/api/blobs/sha256:zz", content=b"").status_code == 400
    assert not [f for f in os.listdir(tmp_path / "store" / "blobs") if "upload" in f]
    r = c.post("/api/create", json={"model": "mine:latest", "files": {"w.gguf": dg}, "system": "Be brief."})
    assert r.status_code == 200, r.text
    e = ctx.catalogue.ollama.find("mine:latest")
    assert e is not None and e.digest == dg and e.system == "Be brief."
    assert c.post("/api/create", json={"model": "x", "files": {"w.gguf": "sha256:" + "0" * 64}}).status_code == 400


def test_validate_and_repair(tmp_path):
    import dataclasses

    from loken_b200.models.config import tiny
    from loken_b200.models.loader import export_random_gguf

    c, ctx, llm = client()
    path = str(tmp_path / "m.gguf")
    export_random_gguf(path, dataclasses.replace(tiny("llama", n_layers=1), weight_format="q8_0"), seed=1)
    r = c.post("/api/models/validate", json={"path": path}).json()
    assert r["ok"] and r["tensors"] > 0
    with open(path, "r+b") as f:
        f.truncate(os.path.getsize(path) - 4096)
    bad = c.post("/api/models/repair", json={"path": path, "model": "m"}).json()
    assert not bad["ok"] and not bad["repaired"] and "api/pull" in bad["action"]
    assert c.post("/api/models/validate", json={"model": "nowhere"}).status_code == 404


def test_layers_swap_route(monkeypatch):
    import types

    from loken_b200.models import lora

    c, ctx, llm = client()
    assert c.post("/api/layers/swap", json={"model": "fake-model", "adapters": ["/x"]}).status_code == 400   # no weights here
    calls = []

    class FakeSet:
        def __init__(self, mw):
            self.mw = mw

        def apply(self, wanted):
            calls.append(dict(wanted))
            if "bad" in wanted:
                raise ValueError("adapter names layer 7")
            return {"attached": sorted(wanted), "detached": [], "kept": [], "projections": len(wanted)}

    monkeypatch.setattr(lora, "AdapterSet", FakeSet)
    llm.engine.weights = types.SimpleNamespace()
    toks = list(range(50))
    llm.engine.alloc.allocate_with_prefix(7, toks)
    llm.engine.alloc.commit_prefix(7, toks)
    llm.engine.alloc.free(7)
    r = c.post("/api/layers/swap", json={"model": "fake-model", "adapters": ["/a", {"path": "/b", "weight": 0.5}]})
    assert r.status_code == 200 and r.json()["attached"] == ["/a", "/b"] and r.json()["prefix_blocks_dropped"] == 3
    assert calls[-1] == {"/a": 1.0, "/b": 0.5}
    assert c.post("/api/layers/swap", json={"adapters": []}).json()["attached"] == []
    assert c.post("/api/layers/swap", json={"adapters": ["bad"]}).status_code == 400
    assert c.post("/api/layers/swap", json={"adapters": [{"weight": 2}]}).status_code == 400
