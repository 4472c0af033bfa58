"""KV hand-over: a peer reads the prompt and this node continues from its cache
(disaggregated prefill, `src/inference/engine/llm_engine/handover.rs`, `docs/CONFIGURATION.md:171-218`).

The paged cache rows of a sequence are exported layer by layer as they are stored (q8 codes +
f16 scales, or bf16), so the hop carries 1.06 bytes per cached value instead of the reference's
f32 rows.  Container: a small JSON header (shape, format, token ids for the prefix hash) and the
raw planes.  Import allocates blocks on the receiving side, writes the planes to its slots and
publishes the prefix so later requests can share it.  `HandoverRate` decides whether asking a
peer is worth it: only when the measured hand-over rate beats local prefill.
"""
from __future__ import annotations

import json
import struct
from typing import List, Optional

import torch

MAGIC = b"LKKV1\0"


def export_sequence(runner, alloc, seq_id: int, tokens: List[int], n_tokens: Optional[int] = None) -> bytes:
    """Serialises the first `n_tokens` cached positions of a sequence."""
    n = n_tokens if n_tokens is not None else len(tokens)
    slots = torch.tensor(alloc.slots_for_range(seq_id, 0, n), dtype=torch.int64, device=runner.device)
    planes = []
    fmt = None
    for layer in runner.kv:
        if layer is None:
            continue
        if layer.q8:
            fmt = "q8"
            parts = [layer.k[slots], layer.k_scale[slots], layer.v[slots], layer.v_scale[slots]]
        else:
            fmt = "bf16"
            parts = [layer.k[slots], layer.v[slots]]
        planes.append([p.contiguous().cpu() for p in parts])
    head = {"format": fmt, "tokens": [int(t) for t in tokens[:n]], "n": n, "layers": len(planes),
            "n_kv": runner.w.n_kv_local, "head_dim": runner.cfg.head_dim, "model": model_identity(runner),
            "planes": [[list(p.shape), str(p.dtype)] for p in planes[0]] if planes else []}
    hb = json.dumps(head).encode()
    out = [MAGIC, struct.pack("<I", len(hb)), hb]
    for parts in planes:
        for p in parts:
            out.append(p.view(torch.uint8).numpy().tobytes())
    return b"".join(out)


def model_identity(runner) -> str:
    """What two engines must share for one's cache rows to mean anything to the other: the model's
    shape and name, this rank's share of the kv heads, and (when the loader recorded one) a digest
    of the weights."""
    cfg, w = runner.cfg, runner.w
    n_layers = sum(1 for layer in runner.kv if layer is not None)
    return "|".join(str(v) for v in (cfg.name, cfg.arch, n_layers, cfg.hidden, cfg.n_q, cfg.n_kv, cfg.head_dim,
                                     cfg.vocab, w.n_kv_local, getattr(w, "digest", "")))


_DTYPES = {"torch.int8": torch.int8, "torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16}


def _parse(runner, blob: bytes):
    """Checks the container against this engine before anything is allocated: header, model
    identity, layer count, plane shapes and dtypes, token count and total length.  Returns
    (header, byte offset of the first plane, [(shape, dtype, nbytes)] of one layer)."""
    if blob[:len(MAGIC)] != MAGIC:
        raise ValueError("not a KV hand-over container")
    off = len(MAGIC)
    if len(blob) < off + 4:
        raise ValueError("hand-over container is cut short")
    (hl,) = struct.unpack_from("<I", blob, off)
    off += 4
    if hl <= 0 or off + hl > len(blob):
        raise ValueError("hand-over header length is out of range")
    try:
        head = json.loads(blob[off:off + hl])
    except Exception:
        raise ValueError("hand-over header is not JSON")
    off += hl
    for key in ("n", "n_kv", "head_dim", "format", "layers", "planes", "tokens"):
        if key not in head:
            raise ValueError(f"hand-over header lacks '{key}'")
    n = head["n"]
    if not isinstance(n, int) or n <= 0:
        raise ValueError("hand-over of no positions")
    if head["n_kv"] != runner.w.n_kv_local or head["head_dim"] != runner.cfg.head_dim:
        raise ValueError("hand-over from a model of another shape")
    ident = head.get("model")
    if ident is not None and ident != model_identity(runner):
        raise ValueError("hand-over from another model")
    local = [l for l in runner.kv if l is not None]
    if head["layers"] != len(local):
        raise ValueError(f"hand-over carries {head['layers']} layers, this engine holds {len(local)}")
    want_fmt = "q8" if local[0].q8 else "bf16"
    if head["format"] != want_fmt:
        raise ValueError(f"hand-over cache format {head['format']} differs from this node's {want_fmt}")
    toks = head["tokens"]
    if not isinstance(toks, list) or len(toks) != n:
        raise ValueError("hand-over token list does not match its position count")
    if any((not isinstance(t, int)) or t < 0 or t >= runner.cfg.vocab for t in toks):
        raise ValueError("hand-over token id outside the vocabulary")
    L = local[0]
    dests = [L.k, L.k_scale, L.v, L.v_scale] if L.q8 else [L.k, L.v]
    if len(head["planes"]) != len(dests):
        raise ValueError("hand-over plane count differs from the cache layout")
    planes, per_layer = [], 0
    for dest, spec in zip(dests, head["planes"]):
        shape, dname = spec
        if dname not in _DTYPES or _DTYPES[dname] != dest.dtype:
            raise ValueError(f"hand-over plane dtype {dname} differs from the cache's {dest.dtype}")
        if list(shape) != [n] + list(dest.shape[1:]):
            raise ValueError(f"hand-over plane shape {shape} does not fit {n} positions of {list(dest.shape[1:])}")
        nbytes = n * dest[0].numel() * dest.element_size()
        planes.append((list(shape), dest.dtype, nbytes))
        per_layer += nbytes
    if len(blob) - off != per_layer * len(local):
        raise ValueError("hand-over payload length does not match its header")
    return head, off, planes


def import_sequence(runner, alloc, seq_id: int, blob: bytes, salt: int = 0) -> int:
    """Allocates the sequence on this node and fills its cache; returns the number of positions
    now cached (the caller continues prefill or decode from there).  The container is checked in
    full before any block is taken, and a failure while copying gives the blocks back, so a bad
    blob from the network can neither leak blocks nor publish content hashes over foreign rows."""
    head, off, planes = _parse(runner, blob)
    n = head["n"]
    if not alloc.allocate(seq_id, n):
        raise MemoryError("no room for the handed-over cache")
    try:
        slots = torch.tensor(alloc.slots_for_range(seq_id, 0, n), dtype=torch.int64, device=runner.device)
        for layer in runner.kv:
            if layer is None:
                continue
            dests = [layer.k, layer.k_scale, layer.v, layer.v_scale] if layer.q8 else [layer.k, layer.v]
            for dest, (shape, t, nbytes) in zip(dests, planes):
                src = torch.frombuffer(bytearray(blob[off:off + nbytes]), dtype=t).view(shape)
                dest[slots] = src.to(runner.device)
                off += nbytes
        alloc.commit_prefix(seq_id, head["tokens"], salt)
    except Exception:
        alloc.free(seq_id)
        raise
    return n


class HandoverRate:
    """Tokens per second a peer's prefill + transfer has delivered, against local prefill."""

    def __init__(self):
        self.peer_rate = 0.0
        self.local_rate = 0.0

    def observe_peer(self, tokens: int, seconds: float):
        if seconds > 0:
            r = tokens / seconds
            self.peer_rate = r if self.peer_rate == 0 else 0.7 * self.peer_rate + 0.3 * r

    def observe_local(self, tokens: int, seconds: float):
        if seconds > 0:
            r = tokens / seconds
            self.local_rate = r if self.local_rate == 0 else 0.7 * self.local_rate + 0.3 * r

    def ask_peer(self, prompt_tokens: int, min_tokens: int = 512) -> bool:
        if prompt_tokens < min_tokens:
            return False
        if self.peer_rate == 0:
            return True                # first long prompt: measure it
        return self.peer_rate > self.local_rate
