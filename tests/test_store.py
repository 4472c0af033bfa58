"""Model stores: Ollama manifests + blobs over several directories, the Hugging Face cache layout,
bare GGUF files, and resumable pulls against a scripted transport."""
import hashlib
import json
import os

import pytest

from loken_b200.store.catalogue import Catalogue, OllamaStore, split_ollama_name
from loken_b200.store.download import fetch, pull_huggingface, pull_ollama


def _gguf(path, payload=b"GGUF" + b"\0" * 100):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    open(path, "wb").write(payload)
    return path


def test_names():
    assert split_ollama_name("qwen3:0.6b") == ("registry.ollama.ai", "library", "qwen3", "0.6b")
    assert split_ollama_name("me/model") == ("registry.ollama.ai", "me", "model", "latest")
    assert split_ollama_name("host:5000/ns/model:tag") == ("host:5000", "ns", "model", "tag")


def test_ollama_store_over_two_directories(tmp_path):
    a, b = str(tmp_path / "nvme"), str(tmp_path / "hdd")
    src = _gguf(str(tmp_path / "m.gguf"))
    st = OllamaStore([a, b])
    e = st.create("qwen3:0.6b", src, template="{{ .Prompt }}", system="be brief", params={"temperature": 0.2})
    assert e.store == a and e.template == "{{ .Prompt }}" and e.system == "be brief" and e.params == {"temperature": 0.2}
    assert os.path.exists(e.path) and e.digest.startswith("sha256:") and e.path.endswith(e.digest.replace(":", "-"))
    # the same tag in the second directory is shadowed by the first
    OllamaStore([b]).create("qwen3:0.6b", _gguf(str(tmp_path / "other.gguf"), b"GGUF-other"))
    assert [m.name for m in st.list()] == ["qwen3:0.6b"] and st.find("qwen3:0.6b").store == a
    # a copy shares the blobs and stays beside them; deleting the source keeps the shared blob
    c = st.copy("qwen3:0.6b", "mine/qwen:latest")
    assert c.name == "mine/qwen:latest" and c.path == e.path and c.store == a
    assert st.delete("qwen3:0.6b") == 2                      # every copy of the manifest
    assert st.find("qwen3:0.6b") is None and os.path.exists(c.path)
    assert st.delete("mine/qwen:latest") == 1 and not os.path.exists(c.path)      # pruned with its last manifest
    # a manifest whose weights blob is missing is not listed
    mp = st.manifest_path(a, "ghost:latest")
    os.makedirs(os.path.dirname(mp), exist_ok=True)
    json.dump({"layers": [{"mediaType": "application/vnd.ollama.image.model", "digest": "sha256:" + "0" * 64,
                           "size": 1}]}, open(mp, "w"))
    assert st.find("ghost:latest") is None


def test_huggingface_cache_and_bare_gguf(tmp_path):
    hf = str(tmp_path / "hf")
    snap = os.path.join(hf, "hub", "models--Qwen--Qwen3-0.6B", "snapshots", "abc123")
    os.makedirs(snap)
    json.dump({"architectures": ["Qwen3ForCausalLM"]}, open(os.path.join(snap, "config.json"), "w"))
    open(os.path.join(snap, "model.safetensors"), "wb").write(b"x" * 10)
    os.makedirs(os.path.join(hf, "hub", "models--Qwen--Qwen3-0.6B", "refs"))
    open(os.path.join(hf, "hub", "models--Qwen--Qwen3-0.6B", "refs", "main"), "w").write("abc123")
    _gguf(os.path.join(hf, "tiny-q8.gguf"))
    cat = Catalogue(ollama_dirs=[str(tmp_path / "none")], huggingface_dirs=[hf])
    names = {m.name: m for m in cat.list()}
    assert set(names) == {"Qwen/Qwen3-0.6B", "tiny-q8.gguf"}
    assert names["Qwen/Qwen3-0.6B"].path == snap and names["Qwen/Qwen3-0.6B"].source == "huggingface"
    assert cat.resolve("tiny-q8").path.endswith("tiny-q8.gguf") and cat.resolve("tiny-q8:latest") is not None
    assert cat.resolve(snap).source == "huggingface"          # an existing path is taken as it is
    assert cat.resolve("nothing") is None
    assert cat.delete("Qwen/Qwen3-0.6B") == 1 and cat.resolve("Qwen/Qwen3-0.6B") is None


class Net:
    """A scripted transport: serves byte strings by URL, honours Range, can cut a transfer short."""

    def __init__(self, files):
        self.files, self.cut, self.calls = files, {}, []

    def __call__(self, url, headers):
        self.calls.append((url, dict(headers)))
        if url not in self.files:
            return 404, {}, iter(())
        data = self.files[url]
        start = 0
        if "Range" in headers:
            start = int(headers["Range"].split("=")[1].rstrip("-"))
            if start >= len(data):
                return 416, {}, iter(())
        body = data[start:]
        limit = self.cut.pop(url, None)
        hdr = {"Content-Range": f"bytes {start}-{len(data) - 1}/{len(data)}"} if start else {"Content-Length": str(len(body))}
        if limit is not None:
            body = body[:limit]
        return (206 if start else 200), hdr, iter([body[i:i + 7] for i in range(0, len(body), 7)])


def test_fetch_resumes_and_checks_the_digest(tmp_path):
    data = bytes(range(256)) * 5
    net = Net({"u": data})
    net.cut["u"] = 100
    target = str(tmp_path / "blob")
    with pytest.raises(IOError, match="resume"):
        fetch("u", target, opener=net)
    assert os.path.getsize(target + ".partial") == 100 and not os.path.exists(target)
    got = fetch("u", target, sha256=hashlib.sha256(data).hexdigest(), opener=net)
    assert got == len(data) - 100 and net.calls[-1][1]["Range"] == "bytes=100-" and open(target, "rb").read() == data
    with pytest.raises(IOError, match="sha256"):
        fetch("u", str(tmp_path / "bad"), sha256="0" * 64, opener=net)
    assert not os.path.exists(str(tmp_path / "bad.partial"))


def test_pull_ollama_and_huggingface(tmp_path):
    weights, tmpl = b"GGUF" + b"w" * 500, b"{{ .Prompt }}"
    dw, dt = "sha256:" + hashlib.sha256(weights).hexdigest(), "sha256:" + hashlib.sha256(tmpl).hexdigest()
    man = json.dumps({"layers": [{"mediaType": "application/vnd.ollama.image.model", "digest": dw, "size": len(weights)},
                                 {"mediaType": "application/vnd.ollama.image.template", "digest": dt, "size": len(tmpl)}]}
                     ).encode()
    base = "https://registry.ollama.ai"
    net = Net({f"{base}/v2/library/tiny/manifests/1b": man, f"{base}/v2/library/tiny/blobs/{dw}": weights,
               f"{base}/v2/library/tiny/blobs/{dt}": tmpl})
    st = OllamaStore([str(tmp_path / "a"), str(tmp_path / "b")])
    states = [s["status"] for s in pull_ollama(st, "tiny:1b", opener=net)]
    assert states[0] == "pulling manifest" and states[-1] == "success"
    e = st.find("tiny:1b")
    assert e is not None and e.store == str(tmp_path / "a") and e.template == "{{ .Prompt }}" and e.size == len(weights) + len(tmpl)
    n_calls = len(net.calls)
    list(pull_ollama(st, "tiny:1b", opener=net))             # a second pull fetches the manifest only
    assert len(net.calls) == n_calls + 1
    hf = str(tmp_path / "hf")
    net2 = Net({"https://huggingface.co/o/r/resolve/main/config.json": b"{}",
                "https://huggingface.co/o/r/resolve/main/model.safetensors": b"s" * 40})
    list(pull_huggingface(hf, "o/r", ["config.json", "model.safetensors"], opener=net2))
    assert Catalogue([str(tmp_path / "x")], [hf]).resolve("o/r").source == "huggingface"


def test_ollama_routes_use_the_stores(tmp_path):
    from fastapi.testclient import TestClient

    from loken_b200.api.common import ModelRegistry
    from loken_b200.api.server import create_app
    from tests.fakes import fake_llm

    st_dir = str(tmp_path / "ollama")
    cat = Catalogue([st_dir], [str(tmp_path / "hf")])
    cat.ollama.create("stored:1b", _gguf(str(tmp_path / "s.gguf")), template="T")
    reg = ModelRegistry()
    reg.add(fake_llm())
    app = create_app(reg, None)
    app.state.ctx.catalogue = cat
    c = TestClient(app)
    names = [m["name"] for m in c.get("/api/tags").json()["models"]]
    assert names == ["fake-model", "stored:1b"]
    assert c.post("/api/copy", json={"source": "stored:1b", "destination": "copy:1b"}).status_code == 200
    assert cat.ollama.find("copy:1b").path == cat.ollama.find("stored:1b").path
    assert c.post("/api/create", json={"model": "mine", "from": "stored:1b", "system": "terse"}).json()["status"] == "success"
    assert cat.ollama.find("mine").system == "terse" and cat.ollama.find("mine").template == "T"
    assert c.post("/api/pull", json={"model": "stored:1b"}).status_code == 200          # already here
    weights = b"GGUF" + b"p" * 64
    dw = "sha256:" + hashlib.sha256(weights).hexdigest()
    base = "https://registry.ollama.ai"
    app.state.ctx.opener = Net({f"{base}/v2/library/far/manifests/latest": json.dumps({"layers": [
        {"mediaType": "application/vnd.ollama.image.model", "digest": dw, "size": len(weights)}]}).encode(),
        f"{base}/v2/library/far/blobs/{dw}": weights})
    r = c.post("/api/pull", json={"model": "far"})
    assert r.status_code == 200 and '"success"' in r.text and cat.ollama.find("far") is not None
    assert c.post("/api/pull", json={"model": "nowhere"}).status_code == 502
    assert c.request("DELETE", "/api/delete", json={"model": "copy:1b"}).status_code == 200
    assert cat.ollama.find("copy:1b") is None and cat.ollama.find("stored:1b") is not None


def test_config_reads_store_directories():
    from loken_b200.config import load_config

    cfg = load_config(text="ollama_models_dir = [\"/a\", \"/b\"]\nhuggingface_models_dir = \"/hf\"\n")
    assert cfg.ollama_models_dir == ["/a", "/b"] and cfg.huggingface_models_dir == ["/hf"] and not cfg.notes


def test_draft_head_is_fetched_by_ranged_reads_only(tmp_path):
    """Two shards on a fake hub; the head's tensors sit in the second.  Only headers and the head's own bytes
    cross the wire, and the companion file carries the tensors under their short names."""
    import io
    import json as _json

    import torch
    from safetensors.torch import save

    from loken_b200.formats import gguf as G
    from loken_b200.store.download import fetch_draft_head

    g = torch.Generator().manual_seed(0)
    big = {"model.layers.0.mlp.up_proj.weight": torch.randn(512, 256, generator=g).bfloat16()}
    head = {"model.layers.0.self_attn.q_proj.weight": torch.randn(64, 64, generator=g).bfloat16(),
            "model.mtp.fc.weight": torch.randn(32, 64, generator=g).bfloat16(),
            "model.mtp.norm.weight": torch.randn(32, generator=g).float(),
            "model.mtp.layers.0.self_attn.q_proj.weight": torch.randn(32, 32, generator=g).half()}
    files = {"model-00001-of-00002.safetensors": save(big), "model-00002-of-00002.safetensors": save(head)}
    index = {"weight_map": {**{k: "model-00001-of-00002.safetensors" for k in big},
                            **{k: "model-00002-of-00002.safetensors" for k in head}}}
    files["model.safetensors.index.json"] = _json.dumps(index).encode()
    wire = {"bytes": 0, "whole": 0}

    def opener(url, headers):
        name = url.rsplit("/", 1)[-1]
        if name not in files:
            return 404, {}, iter(())
        data = files[name]
        rng = headers.get("Range")
        if rng:
            lo, hi = rng.split("=")[1].split("-")
            part = data[int(lo):int(hi) + 1]
            wire["bytes"] += len(part)
            return 206, {}, iter([part])
        wire["whole"] += len(data)
        return 200, {}, iter([data])

    out = str(tmp_path / "m.mtp.gguf")
    rep = fetch_draft_head("acme/model", out, opener=opener)
    assert rep["tensors"] == 3 and rep["shards"] == 1
    assert wire["whole"] == len(files["model.safetensors.index.json"])                    # no shard was fetched whole
    assert wire["bytes"] == rep["bytes_read"] < len(files["model-00002-of-00002.safetensors"])
    r = G.GGUFReader(out)
    assert r.meta["general.type"] == "draft-head" and set(r.tensors) == {"fc.weight", "norm.weight", "layers.0.self_attn.q_proj.weight"}
    assert torch.equal(torch.from_numpy(r.tensors["fc.weight"].to_float()), head["model.mtp.fc.weight"].float())
    assert torch.allclose(torch.from_numpy(r.tensors["norm.weight"].to_float()), head["model.mtp.norm.weight"])
    r.close()
    with pytest.raises(IOError):                                                           # a server without ranges is refused
        fetch_draft_head("acme/model", out, opener=lambda u, h: (200, {}, iter([files.get(u.rsplit("/", 1)[-1], b"")])))
    del files["model.safetensors.index.json"]
    with pytest.raises((IOError, ValueError)):
        fetch_draft_head("acme/other", str(tmp_path / "x.gguf"), opener=opener)
