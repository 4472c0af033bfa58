"""The CPU decode path: a dense GGUF model run token by token on the host cores by the C++
executor (`csrc/host/cpu_decode.cpp`), weights read in place from the file mapping.

    m = CpuModel.from_gguf("qwen3-1.7b-q8_0.gguf")
    out = m.generate(prompt_ids, max_tokens=64)

This is the path of the reference's CPU configuration (Qwen3-1.7B Q8_0: Q8_0 x Q8_0 integer
dots with AVX-512 VNNI / AVX2 / scalar versions, a Q8_0 KV cache, a persistent GEMV pool —
`src/inference/kernel/cpu_decode_exec.rs`, `src/tensor/quant_cpu/`), and it doubles as an
independent oracle for the GPU kernels.
"""
from __future__ import annotations

import ctypes as C
import random
import time
from typing import List, Optional, Sequence

import numpy as np

from ..formats import gguf as G
from ..models.config import ModelConfig
from ..ops._lib import host_lib

ROLE = {"attn_norm": 0, "attn_q": 1, "attn_k": 2, "attn_v": 3, "attn_output": 4, "attn_q_norm": 5, "attn_k_norm": 6,
        "ffn_norm": 7, "ffn_gate": 8, "ffn_up": 9, "ffn_down": 10}
BIAS_ROLE = {"attn_q": 11, "attn_k": 12, "attn_v": 13}
G_EMBED, G_OUT_NORM, G_LM_HEAD = 100, 101, 102


class CpuConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "hidden", "n_q", "n_kv", "head_dim", "intermediate", "vocab",
                                       "rope_dim", "rope_pairing")] + [("rope_theta", C.c_float),
                                                                       ("rms_eps", C.c_float)]


def _lib():
    L = host_lib()
    L.lkcpu_create.restype = C.c_void_p
    L.lkcpu_dot_q8_0.restype = C.c_float
    return L


class CpuModel:
    def __init__(self, cfg: ModelConfig, threads: int = 0, max_level: int = -1):
        if cfg.is_moe:
            raise ValueError("the CPU path runs dense models")
        self.cfg = cfg
        c = CpuConfig(cfg.n_layers, cfg.hidden, cfg.n_q, cfg.n_kv, cfg.head_dim, cfg.intermediate, cfg.vocab,
                      cfg.rope_dim or 0, cfg.rope_pairing, cfg.rope_theta, cfg.rms_eps)
        self._h = C.c_void_p(_lib().lkcpu_create(C.byref(c), threads, max_level))
        if not self._h:
            raise ValueError("shape not supported by the CPU path (dims must be multiples of 32)")
        inv, _ = cfg.rope_tables()
        a = np.asarray(inv, dtype=np.float32)
        _lib().lkcpu_set_inv_freq(self._h, a.ctypes.data_as(C.c_void_p), a.size)
        self._keep = []          # arrays / readers the C side points into
        self.pos = 0
        self.logits = np.zeros(cfg.vocab, dtype=np.float32)

    @classmethod
    def from_gguf(cls, path: str, threads: int = 0, max_level: int = -1) -> "CpuModel":
        r = G.GGUFReader(path)
        meta = dict(r.meta)
        if "token_embd.weight" in r.tensors:
            meta["_vocab"] = r.tensors["token_embd.weight"].shape[0]
        cfg = ModelConfig.from_gguf_meta(meta, meta.get("general.name", "gguf"))
        if not cfg.vocab:
            cfg.vocab = int(meta["_vocab"])
        cfg.qk_norm = "blk.0.attn_q_norm.weight" in r.tensors
        m = cls(cfg, threads, max_level)
        m._keep.append(r)
        m.meta = meta

        def put(layer, role, name):
            t = r.tensors.get(name)
            if t is None:
                return False
            rc = _lib().lkcpu_set_tensor(m._h, layer, role, C.c_void_p(t.data.ctypes.data), t.ggml_type)
            if rc != 0:
                raise ValueError(f"cannot bind {name}")
            return True

        put(-1, G_EMBED, "token_embd.weight")
        put(-1, G_OUT_NORM, "output_norm.weight")
        put(-1, G_LM_HEAD, "output.weight")
        for il in range(cfg.n_layers):
            for stem, role in ROLE.items():
                put(il, role, f"blk.{il}.{stem}.weight")
            for stem, role in BIAS_ROLE.items():
                put(il, role, f"blk.{il}.{stem}.bias")
        if not _lib().lkcpu_ready(m._h):
            raise ValueError(f"{path}: a tensor the dense decoder needs is missing")
        return m

    @property
    def simd_level(self) -> int:
        return _lib().lkcpu_level(self._h)

    @property
    def threads(self) -> int:
        return _lib().lkcpu_threads(self._h)

    def reset(self):
        self.pos = 0

    def feed(self, token: int, want_logits: bool = True) -> Optional[np.ndarray]:
        out = self.logits.ctypes.data_as(C.c_void_p) if want_logits else None
        rc = _lib().lkcpu_decode(self._h, int(token), self.pos, out)
        if rc != 0:
            raise RuntimeError(f"lkcpu_decode failed ({rc}) at position {self.pos}")
        self.pos += 1
        return self.logits if want_logits else None

    def prefill(self, tokens: Sequence[int]) -> np.ndarray:
        for t in tokens[:-1]:
            self.feed(t, want_logits=False)
        return self.feed(tokens[-1])

    def generate(self, prompt: Sequence[int], max_tokens: int = 32, temperature: float = 0.0, top_k: int = 0,
                 seed: Optional[int] = None, eos: Sequence[int] = ()) -> dict:
        """Greedy or temperature / top-k sampling on the host; returns tokens and timings."""
        self.reset()
        # the draw for token N depends on (seed, N) alone, as on the device path (serve/replay.py)
        from ..serve.replay import PositionRng

        rng = PositionRng(seed if seed is not None else random.SystemRandom().getrandbits(63))
        t0 = time.perf_counter()
        logits = self.prefill(list(prompt))
        t1 = time.perf_counter()
        out: List[int] = []
        for _ in range(max_tokens):
            if temperature < 1e-7:
                tok = int(np.argmax(logits))
            else:
                x = logits.astype(np.float64) / temperature
                if top_k > 0:
                    kth = np.partition(x, -top_k)[-top_k]
                    x = np.where(x >= kth, x, -np.inf)
                p = np.exp(x - x.max())
                p /= p.sum()
                tok = int(np.searchsorted(np.cumsum(p), rng.random()))
                tok = min(tok, len(p) - 1)
            out.append(tok)
            if tok in eos:
                break
            logits = self.feed(tok)
        t2 = time.perf_counter()
        return {"tokens": out, "prefill_s": t1 - t0, "decode_s": t2 - t1,
                "tok_per_s": (len(out) - 1) / (t2 - t1) if len(out) > 1 and t2 > t1 else None}

    def close(self):
        if self._h:
            _lib().lkcpu_free(self._h)
            self._h = None
        for k in self._keep:
            if hasattr(k, "close"):
                k.close()
        self._keep = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
