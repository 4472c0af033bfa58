"""Configuration loading and the CLI's offline commands."""
import io
import json

import numpy as np
import pytest

from loken_b200.cli import loken, lokend
from loken_b200.config import load_config


def test_config_sections_env_and_obsolete_keys():
    cfg = load_config(text="""
[server]
port = 8080
api_keys = ["a"]
workers = 4
[inference]
model = "llama-3.1-8b"
tp = 8
fidelity = "reference"
gpu_layers = 99
frobnicate = 1
[weird]
x = 1
""", env={"LOKEN_API_KEY": "b", "OLLAMA_KEEP_ALIVE": "10m"})
    assert cfg.server.port == 8080 and cfg.server.api_keys == ["a", "b"]
    assert cfg.inference.tp == 8 and cfg.kv_format == "bf16"
    assert cfg.inference.keep_alive_s == 600.0
    notes = "\n".join(cfg.notes)
    assert "workers is obsolete" in notes and "gpu_layers is obsolete" in notes
    assert "unknown key frobnicate" in notes and "unknown section [weird]" in notes
    with pytest.raises(ValueError):
        load_config(text='[inference]\nfidelity = "sloppy"', env={})
    with pytest.raises(ValueError):
        load_config(text="[server]\nrequire_auth = true", env={})
    assert load_config(text="", env={}).kv_format == "q8"


def test_lokend_flags_override_file():
    args = lokend.build_parser().parse_args(["serve", "--model", "x.gguf", "--port", "9000", "--tp", "2"])
    cfg = lokend.apply_flags(load_config(text="[server]\nport = 1234", env={}), args)
    assert cfg.server.port == 9000 and cfg.inference.model == "x.gguf" and cfg.inference.tp == 2


def test_loken_convert_and_validate(tmp_path):
    out = io.StringIO()
    path = str(tmp_path / "m.gguf")
    # a small real file through the writer, then validate it
    from loken_b200.models.config import tiny
    from loken_b200.models.loader import export_random_gguf

    export_random_gguf(path, tiny("llama", weight_format="q8_0"), seed=0)
    assert loken.main(["validate", path], out=out) == 0
    rep = json.loads(out.getvalue())
    assert rep["ok"] and rep["architecture"] == "llama" and rep["tensors"] > 10
    # truncate a payload: the reader refuses or the validator reports it
    raw = open(path, "rb").read()
    bad = str(tmp_path / "bad.gguf")
    open(bad, "wb").write(raw[:len(raw) // 2])
    with pytest.raises((IOError, OSError, SystemExit)):
        loken.validate_gguf(bad)
    out2 = io.StringIO()
    assert loken.main(["popular"], out=out2) == 0 and "Qwen/Qwen3-8B" in out2.getvalue() and "loken pull" in out2.getvalue()
    with pytest.raises(SystemExit, match="cannot reach"):       # calibration runs in the daemon
        txt = tmp_path / "t.txt"
        txt.write_text("some text to calibrate on")
        loken.main(["--server", "http://127.0.0.1:9", "calibrate", path, "-n", "c1", "-t", str(txt)], out=out2)
    with pytest.raises(SystemExit, match="cannot reach"):       # a pull goes through the daemon, which is not running
        loken.main(["--server", "http://127.0.0.1:9", "pull", "whatever"], out=out2)


def test_draft_head_companion_is_cut_from_a_checkpoint(tmp_path):
    """`loken draft-head` collects a checkpoint's mtp.* tensors into a companion (GGUF or safetensors) that the
    draft-head loader reads back as the same head."""
    import io

    import torch
    from safetensors.torch import save_file

    from loken_b200.cli import loken
    from loken_b200.models.config import tiny
    from loken_b200.serve.draft_head import load_draft_head

    cfg = tiny("llama", hidden=128, n_q=2, n_kv=2, head_dim=64, intermediate=256)
    H, I, g = cfg.hidden, cfg.intermediate, torch.Generator().manual_seed(0)
    rn = lambda *s: (torch.randn(*s, generator=g) * 0.05).bfloat16()
    mtp = {"eh_proj.weight": rn(H, 2 * H), "enorm.weight": torch.ones(H) + 0.1, "hnorm.weight": torch.ones(H) - 0.1,
           "layers.0.input_layernorm.weight": torch.ones(H), "layers.0.post_attention_layernorm.weight": torch.ones(H),
           "layers.0.self_attn.q_proj.weight": rn(H, H), "layers.0.self_attn.k_proj.weight": rn(H, H),
           "layers.0.self_attn.v_proj.weight": rn(H, H), "layers.0.self_attn.o_proj.weight": rn(H, H),
           "layers.0.mlp.gate_proj.weight": rn(I, H), "layers.0.mlp.up_proj.weight": rn(I, H),
           "layers.0.mlp.down_proj.weight": rn(H, I)}
    ckpt = tmp_path / "ckpt"
    ckpt.mkdir()
    save_file({"model.mtp." + k: v for k, v in mtp.items()} | {"model.embed_tokens.weight": rn(16, H)},
              str(ckpt / "model.safetensors"))
    heads = []
    for out_path in (str(tmp_path / "m.mtp.gguf"), str(tmp_path / "headdir")):
        buf = io.StringIO()
        assert loken.main(["draft-head", str(ckpt), out_path], out=buf) == 0, buf.getvalue()
        assert json.loads(buf.getvalue())["tensors"] == len(mtp)
        heads.append(load_draft_head(out_path, cfg, torch.device("cpu")))
    for h in heads:
        assert h.kind == "mtp" and torch.equal(h.fc.float(), mtp["eh_proj.weight"].float())
        assert torch.allclose(h.enorm, mtp["enorm.weight"]) and torch.allclose(h.hnorm, mtp["hnorm.weight"])
        assert torch.equal(h.layer.wo.weight.float(), mtp["layers.0.self_attn.o_proj.weight"].float())
    empty = tmp_path / "none"
    empty.mkdir()
    save_file({"model.embed_tokens.weight": rn(16, H)}, str(empty / "model.safetensors"))
    buf = io.StringIO()
    assert loken.main(["draft-head", str(empty), str(tmp_path / "x.gguf")], out=buf) == 1 and "no mtp" in buf.getvalue()
