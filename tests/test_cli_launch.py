"""`loken launch`: which model the agent gets, what it is configured with, and that nothing starts
with --config."""
import io
import json
import os

import pytest

from loken_b200.cli import launch as L


def test_pick_model_prefers_asked_then_the_one_loaded_then_the_one_held():
    assert L.pick_model("m", ["a", "b"], []) == "m"
    assert L.pick_model(None, ["a"], ["x", "y"]) == "a"
    assert L.pick_model(None, [], ["x"]) == "x"
    with pytest.raises(ValueError, match="a, b"):
        L.pick_model(None, ["a", "b"], ["x", "y"])
    with pytest.raises(ValueError, match="no model"):
        L.pick_model(None, [], [])
    with pytest.raises(ValueError, match="12 models"):
        L.pick_model(None, [], [f"m{i}" for i in range(12)])


def test_messages_agent_gets_every_role_pointed_at_the_model_and_config_only_starts_nothing():
    l = L.Launch("http://127.0.0.1:11434/", "qwen3:8b", "secret", 40960)
    env = L.messages_env(l)
    assert env["ANTHROPIC_BASE_URL"] == "http://127.0.0.1:11434" and env["ANTHROPIC_AUTH_TOKEN"] == "secret"
    assert {env[k] for k in env if k.endswith("_MODEL")} == {"qwen3:8b"}
    started = []
    out = io.StringIO()
    assert L.launch("claude", l, True, [], out, run=lambda *a, **k: started.append(a) or 0) == 0
    assert not started and "export ANTHROPIC_MODEL=qwen3:8b" in out.getvalue()
    out = io.StringIO()
    rc = L.launch("claude", l, False, ["-p", "hi"], out, run=lambda argv, env: started.append((argv, env)) or 7)
    assert rc == 7
    argv, env = started[0]
    assert argv == ["claude", "--model", "qwen3:8b", "-p", "hi"] and env["ANTHROPIC_MODEL"] == "qwen3:8b"

    def missing(argv, env):
        raise FileNotFoundError(argv[0])

    with pytest.raises(ValueError, match="not installed"):
        L.launch("claude", l, False, [], io.StringIO(), run=missing)
    with pytest.raises(ValueError, match="unknown agent"):
        L.launch("codex", l, True, [], io.StringIO())


def test_openai_agent_settings_are_merged_not_replaced(tmp_path):
    d = tmp_path / ".cline" / "data"
    d.mkdir(parents=True)
    (d / "globalState.json").write_text(json.dumps({"theme": "dark", "apiProvider": "other"}))
    l = L.Launch("http://h:1", "llama3.1:8b", "k", 8192)
    out = io.StringIO()
    assert L.launch("cline", l, True, [], out, home=str(tmp_path)) == 0
    st = json.loads((d / "globalState.json").read_text())
    assert st["theme"] == "dark" and st["apiProvider"] == "openai" and st["openAiBaseUrl"] == "http://h:1/v1"
    assert st["openAiModelInfo"]["contextWindow"] == 8192
    assert json.loads((d / "secrets.json").read_text()) == {"openAiApiKey": "k"}
    assert oct(os.stat(d / "secrets.json").st_mode & 0o777) == "0o600"
