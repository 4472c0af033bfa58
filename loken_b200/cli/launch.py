"""`loken launch AGENT`: run a coding agent against this daemon.

The agent is configured to talk to the daemon's Messages (or OpenAI) routes instead of a hosted API,
then the terminal is handed to it; `--config` prints the configuration and starts nothing.  The
model is the one asked for, else the one loaded model, else the one model held; otherwise the error
lists what there is.  `LOKEN_API_KEY` is the key handed to the agent when the daemon requires one.
The reference does the same for the same two agents (`src/bin/loken.rs:190-296`, `src/api/launch.rs`).
"""
from __future__ import annotations

import json
import os
import shlex
import subprocess
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

NAMES_SHOWN = 8

TOOLS = {
    # binary, how to get it
    "claude": ("claude", "npm install -g @anthropic-ai/claude-code"),
    "cline": ("cline", "npm install -g cline"),
}


@dataclass
class Launch:
    server: str
    model: str
    api_key: Optional[str] = None
    window: Optional[int] = None


def pick_model(asked: Optional[str], loaded: List[str], held: List[str]) -> str:
    if asked:
        return asked
    if len(loaded) == 1:
        return loaded[0]
    if len(held) == 1:
        return held[0]
    names = loaded or held
    if not names:
        has = "no model"
    elif len(names) > NAMES_SHOWN:
        has = f"{len(names)} models; loken list shows them"
    else:
        has = ", ".join(names)
    raise ValueError(f"pass --model; the daemon has {has}")


def messages_env(l: Launch) -> Dict[str, str]:
    """Environment of an agent that speaks the Messages API: base URL, key, and every model role
    pointed at the one model the daemon serves."""
    env = {
        "ANTHROPIC_BASE_URL": l.server.rstrip("/"),
        "ANTHROPIC_AUTH_TOKEN": l.api_key or "loken",
        "ANTHROPIC_MODEL": l.model,
        "ANTHROPIC_SMALL_FAST_MODEL": l.model,
        "ANTHROPIC_DEFAULT_SONNET_MODEL": l.model,
        "ANTHROPIC_DEFAULT_OPUS_MODEL": l.model,
        "ANTHROPIC_DEFAULT_HAIKU_MODEL": l.model,
        "CLAUDE_CODE_DISABLE_NONESSENTIAL_TRAFFIC": "1",
    }
    if l.window:
        # the window the checkpoint declares is the most the daemon grants a request
        env["CLAUDE_CODE_MAX_OUTPUT_TOKENS"] = str(max(1024, min(l.window // 4, 32000)))
    return env


def messages_args(l: Launch) -> List[str]:
    return ["--model", l.model]


def write_cline(home: str, l: Launch) -> List[str]:
    """An OpenAI-compatible provider entry in the agent's settings; returns the files written."""
    d = os.path.join(home, ".cline", "data")
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, "globalState.json")
    state = {}
    if os.path.exists(path):
        try:
            with open(path) as f:
                state = json.load(f)
        except (OSError, ValueError):
            state = {}
    state.update({
        "apiProvider": "openai",
        "openAiBaseUrl": l.server.rstrip("/") + "/v1",
        "openAiModelId": l.model,
        "planModeApiProvider": "openai", "actModeApiProvider": "openai",
        "planModeOpenAiModelId": l.model, "actModeOpenAiModelId": l.model,
    })
    if l.window:
        state["openAiModelInfo"] = {"contextWindow": l.window, "supportsImages": False}
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(state, f, indent=1)
    os.replace(tmp, path)
    written = [path]
    if l.api_key:
        secrets = os.path.join(d, "secrets.json")
        with open(secrets, "w") as f:
            json.dump({"openAiApiKey": l.api_key}, f)
        os.chmod(secrets, 0o600)
        written.append(secrets)
    return written


def launch(tool: str, l: Launch, config_only: bool, extra: List[str], out, home: Optional[str] = None,
           run=subprocess.call) -> int:
    if tool not in TOOLS:
        raise ValueError(f"unknown agent {tool} (known: {', '.join(sorted(TOOLS))})")
    binary, hint = TOOLS[tool]
    env = dict(os.environ)
    argv = [binary]
    if tool == "claude":
        add = messages_env(l)
        if config_only:
            for k, v in add.items():
                print(f"export {k}={shlex.quote(v)}", file=out)
            print(" ".join([binary] + messages_args(l)), file=out)
            return 0
        env.update(add)
        argv += messages_args(l)
    else:
        for p in write_cline(home or os.path.expanduser("~"), l):
            print(f"wrote {p}", file=out)
        if config_only:
            return 0
    print(f"{binary} on {l.model} at {l.server}" + (f", window {l.window}" if l.window else ""), file=out)
    try:
        return int(run(argv + list(extra), env=env))
    except FileNotFoundError:
        raise ValueError(f"{binary} is not installed. Install it with:\n  {hint}")
