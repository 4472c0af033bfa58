"""Requantise / calibrate / convert: per-tensor types by role, a calibration lifts the most sensitive
tensors, the converted file loads and stays close to its source, and the two routes."""
import dataclasses
import json
import os

import numpy as np
import pytest
import torch

from loken_b200.formats import gguf as G
from loken_b200.formats import requant as R
from loken_b200.models.config import tiny
from loken_b200.models.loader import export_random_gguf


@pytest.fixture(scope="module")
def src(tmp_path_factory):
    d = tmp_path_factory.mktemp("rq")
    cfg = dataclasses.replace(tiny("llama", hidden=256, intermediate=512, n_layers=2, vocab=512), weight_format="bf16")
    p = str(d / "src.gguf")
    export_random_gguf(p, cfg, seed=1)
    return p


def test_roles_and_types():
    assert R.role_of("blk.3.attn_v.weight") == "v" and R.role_of("blk.3.ffn_down.weight") == "down"
    assert R.role_of("blk.0.ffn_gate_exps.weight") == "expert" and R.role_of("blk.0.ffn_down_exps.weight") == "expert_down"
    assert R.role_of("token_embd.weight") == "embed" and R.role_of("output.weight") == "head"
    for keep in ("blk.0.attn_norm.weight", "output_norm.weight", "blk.0.attn_q.bias", "blk.0.attn_sinks.weight",
                 "blk.0.attn_q_norm.weight"):
        assert R.role_of(keep) == "keep", keep
    assert R.role_of("blk.0.ffn_gate_inp.weight") == "router" and R.target_type("router", "q4_k_m") is None
    assert R.target_type("v", "q4_k_m") == G.Q6_K and R.target_type("linear", "q4_k_m") == G.Q4_K
    assert R.target_type("linear", "mxfp4") == G.BF16 and R.target_type("expert", "mxfp4") == G.MXFP4
    assert R._fit(G.Q4_K, 256) == G.Q4_K and R._fit(G.Q4_K, 96) == G.Q8_0 and R._fit(G.Q4_K, 40) == G.BF16


def test_requantised_file_keeps_metadata_and_stays_close(src, tmp_path):
    out = str(tmp_path / "q4.gguf")
    seen = []
    rep = R.requantize_gguf(src, out, "q4_k_m", progress=lambda n, d, t: seen.append((d, t)))
    assert rep["types"] == {"Q6_K": 6, "Q4_K": 10, "F32": 5} and rep["bytes_out"] < 0.4 * rep["bytes_in"]
    assert seen[-1][0] == seen[-1][1] == rep["tensors"] and not os.path.exists(out + ".partial")
    a, b = G.GGUFReader(src), G.GGUFReader(out)
    assert b.meta["general.file_type"] == 15 and b.meta["llama.block_count"] == a.meta["llama.block_count"]
    for name in ("blk.0.attn_q.weight", "blk.1.ffn_down.weight", "token_embd.weight"):
        x, y = a.tensors[name].to_float(), b.tensors[name].to_float()
        rel = np.sqrt(((x - y) ** 2).mean() / (x ** 2).mean())
        assert rel < (0.03 if b.tensors[name].ggml_type == G.Q6_K else 0.1), (name, rel)
    assert np.array_equal(a.tensors["output_norm.weight"].data, b.tensors["output_norm.weight"].data)
    # and the result is a model the loader reads
    from loken_b200.models.loader import load_gguf

    w, _ = load_gguf(out, torch.device("cpu"))
    assert w.cfg.weight_format in ("q4_k", "q4_k_m") and len(w.layers) == 2
    with pytest.raises(ValueError):
        R.requantize_gguf(src, out, "q3_k")


def test_calibration_lifts_the_most_sensitive_tensor(src, tmp_path):
    from loken_b200.models.loader import load_gguf

    w, _ = load_gguf(src, torch.device("cpu"))
    g = torch.Generator().manual_seed(0)
    stats = R.calibrate(w, [torch.randint(0, 512, (30,), generator=g).tolist() for _ in range(3)], max_tokens=64)
    assert "blk.0.attn_q.weight" in stats and stats["blk.1.ffn_down.weight"]["k"] == 512.0
    stats["blk.1.ffn_gate.weight"]["act_ms"] *= 1e6          # make one tensor stand out
    rec = R.write_calibration(str(tmp_path / "c.json"), "c", "src", stats, 3, 64)
    assert abs(sum(rec["sensitivity"].values()) - 1.0) < 1e-6
    out = str(tmp_path / "cal.gguf")
    rep = R.requantize_gguf(src, out, "q4_k_m", calibration=str(tmp_path / "c.json"))
    assert rep["calibrated"]
    r = G.GGUFReader(out)
    assert r.tensors["blk.1.ffn_gate.weight"].ggml_type == G.Q6_K        # lifted from Q4_K
    assert r.tensors["blk.0.ffn_gate.weight"].ggml_type == G.Q4_K


def test_convert_and_calibrate_routes(src, tmp_path):
    from fastapi.testclient import TestClient

    from loken_b200.api.common import ModelRegistry
    from loken_b200.api.server import create_app
    from loken_b200.store.catalogue import Catalogue

    store = tmp_path / "ollama"
    app = create_app(ModelRegistry())
    app.state.ctx.catalogue = Catalogue([str(store)], [str(tmp_path / "hf")])
    c = TestClient(app)
    assert c.post("/api/convert", json={"name": "x:q4"}).status_code == 400
    assert c.post("/api/convert", json={"name": "x:q4", "model": src, "format": "q3_k"}).status_code == 400
    r = c.post("/api/calibrate", json={"name": "cal1", "model": src, "texts": ["hello world " * 8, "abc def"],
                                       "tokens": 48, "stream": False})
    assert r.status_code == 200, r.text
    assert r.json()["status"] == "success" and os.path.exists(r.json()["path"])
    r = c.post("/api/convert", json={"name": "tiny:q4", "model": src, "format": "q4_k_m", "calibration": "cal1"})
    lines = [json.loads(l) for l in r.text.strip().splitlines()]
    assert lines[0]["status"] == "converting" and lines[-1]["status"] == "success", lines[-1]
    assert lines[-1]["model"].startswith("tiny") and lines[-1]["calibrated"] is True
    entry = app.state.ctx.catalogue.resolve("tiny:q4")
    assert entry is not None and G.GGUFReader(entry.path).meta["general.file_type"] == 15
    assert c.post("/api/convert", json={"name": "y:q8", "model": str(tmp_path / "none.gguf"), "stream": False}).status_code == 400
    assert c.post("/api/convert", json={"name": "y", "model": src, "calibration": "nope"}).status_code == 404


def test_conversion_with_activation_rows_keeps_the_model_closer(src, tmp_path):
    """A record that carries activation rows makes the conversion error-compensated: the converted model's
    logits on text like the calibration text are closer to the source's than a plain conversion's."""
    from loken_b200.models.loader import load_gguf
    from loken_b200.models.reference import forward_ref

    w, _ = load_gguf(src, torch.device("cpu"))
    g = torch.Generator().manual_seed(0)
    texts = [torch.randint(0, 64, (48,), generator=g).tolist() for _ in range(4)]       # a narrow "language": 64 of 512 ids
    kept = {}
    stats = R.calibrate(w, texts, max_tokens=192, keep_rows=96, rows_out=kept)
    assert kept["blk.0.attn_q.weight"].shape == (96, 256) and kept["blk.1.ffn_down.weight"].shape[1] == 512
    assert kept["blk.0.attn_q.weight"] is not None and kept["blk.0.attn_k.weight"].shape == kept["blk.0.attn_q.weight"].shape
    R.write_calibration(str(tmp_path / "c.json"), "c", "src", stats, 4, 192, rows=kept)
    assert os.path.exists(str(tmp_path / "c.json.rows.npz"))
    plain = R.requantize_gguf(src, str(tmp_path / "plain.gguf"), "q4_k")
    comp = R.requantize_gguf(src, str(tmp_path / "comp.gguf"), "q4_k", calibration=str(tmp_path / "c.json"))
    assert plain["compensated"] == 0 and comp["compensated"] >= 8
    held = torch.randint(0, 64, (40,), generator=g).tolist()
    want = forward_ref(w, held).float()
    err = {}
    for name in ("plain", "comp"):
        wq, _ = load_gguf(str(tmp_path / f"{name}.gguf"), torch.device("cpu"))
        err[name] = float((forward_ref(wq, held).float() - want).pow(2).mean())
    # the lifted tensors of the calibrated plan help too; what is asserted is the whole effect a user gets
    assert err["comp"] < err["plain"], err
