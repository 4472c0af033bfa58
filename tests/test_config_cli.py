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
    assert loken.main(["popular"], out=out2) == 1 and "no hub catalogue" in out2.getvalue()
    with pytest.raises(SystemExit, match="cannot reach"):       # a pull goes through the daemon, which is not running
        loken.main(["--server", "http://127.0.0.1:9", "pull", "whatever"], out=out2)
