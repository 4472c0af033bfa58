"""Server configuration: one TOML file, a few flags, three environment variables.

Schema (a subset of the reference's `src/config.rs:15-243` plus explicit parallel degrees, which
the reference derives from measurement and a B200 node wants stated):

    [server]     host, port, require_auth, api_keys, allowed_origins, rate_limit_rps, rate_limit_burst,
                 max_body_mb, request_timeout_s
    [inference]  model_id, model (GGUF path or built-in shape), replicas, tp, tp_sum, ep, pp, dp, fidelity
                 (reference | balanced | fast), kv_format, max_seqs, max_ctx, max_prefill_tokens,
                 kv_disk_dir, kv_disk_host_mb, kv_disk_max_gb, prefill_peer, draft_model, draft_k, lora, models_dir, expert_slots
    [energy]     enabled, grid_g_co2_per_kwh
    [cluster]    node_id, listen, peers, heartbeat_ms, suspect_phi, name, discovery, route_requests, resume_unverified

Keys that older files carry and that no longer mean anything load fine and are reported
(`config.rs:134`); unknown keys are reported as well, never fatal.  `LOKEN_API_KEY` adds an API key,
`OLLAMA_KEEP_ALIVE` sets the idle time before a model is parked, `HF_TOKEN` is passed to pulls.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, fields
from typing import Dict, List, Optional

try:
    import tomllib
except ModuleNotFoundError:      # pragma: no cover
    tomllib = None

OBSOLETE_KEYS = {
    "inference": {"gpu_layers", "n_threads", "batch_size", "use_mmap", "flash_attention", "kv_quant",
                  "speculative", "tensor_split"},
    "server": {"workers", "tls_cert", "tls_key"},
}

FIDELITY_KV = {"reference": "bf16", "balanced": "q8", "fast": "q8"}


@dataclass
class ServerSection:
    host: str = "127.0.0.1"
    port: int = 11434
    require_auth: bool = False
    api_keys: List[str] = field(default_factory=list)
    allowed_origins: List[str] = field(default_factory=list)
    rate_limit_rps: float = 0.0
    rate_limit_burst: int = 0
    max_body_mb: int = 64
    request_timeout_s: float = 600.0


@dataclass
class InferenceSection:
    model_id: Optional[str] = None
    model: Optional[str] = None
    replicas: int = 1
    tp: int = 1
    tp_sum: str = "boundary"    # boundary (one kernel per layer boundary: reduce-scatter + residual + norm +
                                # all-gather over peer memory) | push (peer-memory all-reduce kernel) |
                                # fused (GEMM epilogue) | nccl
    expert_slots: int = 0       # mixture models: experts per layer resident on the card, the rest streamed (0 = all resident)
    ep: int = 1
    pp: int = 1
    dp: int = 1
    fidelity: str = "balanced"
    kv_format: Optional[str] = None
    max_seqs: int = 256
    max_ctx: int = 8192
    max_prefill_tokens: int = 8192
    kv_disk_dir: Optional[str] = None     # finished conversations' cache blocks are kept here and found again after a restart
    kv_disk_host_mb: int = 256            # of which the most recently used stay in host memory as well
    kv_disk_max_gb: float = 0.0           # the directory is trimmed to this size, oldest blocks first (0: no bound)
    prefill_peer: Optional[str] = None
    draft_model: Optional[str] = None
    lora: Optional[str] = None         # PEFT adapter directory merged into the checkpoint at load
    draft_k: int = 4
    models_dir: Optional[str] = None
    keep_alive_s: float = 300.0


@dataclass
class EnergySection:
    enabled: bool = True
    grid_g_co2_per_kwh: float = 400.0


@dataclass
class ClusterSection:
    node_id: Optional[str] = None
    listen: Optional[str] = None
    peers: List[str] = field(default_factory=list)
    heartbeat_ms: int = 500
    suspect_phi: float = 8.0
    name: str = "loken"         # discovery ignores announcements that name another cluster
    discovery: bool = False     # announce on, and listen to, the multicast group (cluster/discovery.py)
    route_requests: bool = False     # a request goes to the peer predicted to finish it sooner (cluster/forward.py)
    resume_unverified: bool = False  # continue an answer a peer left unfinished although its weights are not known to be the same


@dataclass
class Config:
    # top-level keys: the model stores, each a directory or a list of directories on several disks
    ollama_models_dir: List[str] = field(default_factory=lambda: ["~/.ollama/models"])
    huggingface_models_dir: List[str] = field(default_factory=lambda: ["~/.cache/huggingface/hub"])
    server: ServerSection = field(default_factory=ServerSection)
    inference: InferenceSection = field(default_factory=InferenceSection)
    energy: EnergySection = field(default_factory=EnergySection)
    cluster: ClusterSection = field(default_factory=ClusterSection)
    notes: List[str] = field(default_factory=list)     # obsolete / unknown keys met while loading

    @property
    def kv_format(self) -> str:
        return self.inference.kv_format or FIDELITY_KV.get(self.inference.fidelity, "q8")

    def validate(self) -> "Config":
        i = self.inference
        if i.fidelity not in FIDELITY_KV:
            raise ValueError(f"[inference] fidelity must be one of {sorted(FIDELITY_KV)}")
        for k in ("tp", "ep", "pp", "dp", "replicas"):
            if getattr(i, k) < 1:
                raise ValueError(f"[inference] {k} must be >= 1")
        if i.tp_sum not in ("boundary", "push", "fused", "nccl"):
            raise ValueError("[inference] tp_sum must be boundary, push, fused or nccl")
        if not (0 < self.server.port < 65536):
            raise ValueError("[server] port out of range")
        if self.server.require_auth and not self.server.api_keys:
            raise ValueError("[server] require_auth is set but there is no key (api_keys or LOKEN_API_KEY)")
        return self


def _parse_duration(v: str) -> float:
    v = v.strip()
    if not v:
        return 300.0
    mult = {"s": 1, "m": 60, "h": 3600}
    if v[-1] in mult:
        return float(v[:-1]) * mult[v[-1]]
    return float(v)


def load_config(path: Optional[str] = None, env: Optional[Dict[str, str]] = None, text: Optional[str] = None) -> Config:
    env = os.environ if env is None else env
    cfg = Config()
    data = {}
    if text is not None:
        data = tomllib.loads(text)
    elif path:
        with open(path, "rb") as f:
            data = tomllib.load(f)
    for section, obj in (("server", cfg.server), ("inference", cfg.inference), ("energy", cfg.energy),
                         ("cluster", cfg.cluster)):
        known = {f.name: f for f in fields(obj)}
        for k, v in (data.get(section) or {}).items():
            if k in known:
                setattr(obj, k, v)
            elif k in OBSOLETE_KEYS.get(section, ()):
                cfg.notes.append(f"[{section}] {k} is obsolete and ignored")
            else:
                cfg.notes.append(f"[{section}] unknown key {k} ignored")
    for key in ("ollama_models_dir", "huggingface_models_dir"):
        if key in data:
            v = data[key]
            setattr(cfg, key, [v] if isinstance(v, str) else [str(x) for x in v])     # a single string reads as a list of 1
    for section in data:
        if section not in ("server", "inference", "energy", "cluster", "ollama_models_dir", "huggingface_models_dir"):
            cfg.notes.append(f"unknown section [{section}] ignored")
    key = env.get("LOKEN_API_KEY")
    if key and key not in cfg.server.api_keys:
        cfg.server.api_keys.append(key)
    if env.get("OLLAMA_KEEP_ALIVE"):
        cfg.inference.keep_alive_s = _parse_duration(env["OLLAMA_KEEP_ALIVE"])
    return cfg.validate()
