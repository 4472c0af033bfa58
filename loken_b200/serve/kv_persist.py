"""The engine's side of the cache's disk tier: what a finished sequence leaves behind, and what a new one finds.

When a sequence finishes, the cache rows of its full 256-token blocks are written under the chain hashes of
their tokens (`serve/kv_disk.py`; blocks another conversation already wrote are skipped), before its device
blocks are released.  When a request arrives whose prompt reaches further into the disk tier than into
the device's prefix cache, the stored rows are written into fresh device blocks and published in the prefix
cache, so the request's prefill starts after them.  Both directions go through the hand-over container
(`cluster/handover.py`): the same gather, the same checks against this engine's cache layout before anything
is allocated, the same "a failure gives the blocks back".

The block keys are salted with the model's identity (shape, name, rank share, weights digest): two models
that share a tokenizer and a directory never read each other's rows.
(reference: `src/inference/cache/kv_disk.rs:86`, `docs/CONFIGURATION.md:255-358`)
"""
from __future__ import annotations

import json
import struct
from typing import List, Optional, Sequence

import numpy as np

from .kv_disk import DISK_BLOCK, KvDiskTier


def _fnv64(text: str) -> int:
    h = 0xCBF29CE484222325
    for b in text.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


class DiskPersistence:
    def __init__(self, runner, alloc, tier: KvDiskTier):
        from ..cluster.handover import model_identity

        self.runner, self.alloc, self.tier = runner, alloc, tier
        self._identity = model_identity(runner)
        self.ident = _fnv64(self._identity)
        self.saved_blocks = 0
        self.restored_tokens = 0
        self.failures = 0

    def rescope(self, what: str):
        """The weights changed in place (adapters were swapped): rows written under the old weights are no longer
        this model's, so the keys move to a scope of their own."""
        self.ident = _fnv64(self._identity + ("|" + what if what else ""))

    def _salt(self, salt: int) -> int:
        return (int(salt) * 0x9E3779B97F4A7C15 ^ self.ident) & 0x7FFFFFFFFFFFFFFF

    # ---- out: called for a finished sequence while it still owns its blocks ----
    def save(self, seq_id: int, tokens: Sequence[int], n_cached: int, salt: int = 0, key: Optional[str] = None) -> int:
        """Writes the full disk blocks among the first `n_cached` positions; returns block files written."""
        from ..cluster.handover import _parse, export_sequence

        n_full = (min(n_cached, len(tokens)) // DISK_BLOCK) * DISK_BLOCK
        if n_full == 0:
            return 0
        toks = [int(t) for t in tokens[:n_full]]
        dsalt = self._salt(salt)
        if self.tier.match(toks, dsalt) >= n_full:
            return 0                                    # every block is there already (a shared prefix, a repeat)
        try:
            blob = export_sequence(self.runner, self.alloc, seq_id, toks, n_full)
            _head, off, planes = _parse(self.runner, blob)
            n_layers = sum(1 for l in self.runner.kv if l is not None)
            views: List[np.ndarray] = []
            for _ in range(n_layers):
                for _shape, _dt, nbytes in planes:
                    views.append(np.frombuffer(blob, dtype=np.uint8, count=nbytes, offset=off).reshape(n_full, nbytes // n_full))
                    off += nbytes
            written = self.tier.save(key or f"seq-{seq_id}", toks, lambda s, e: [v[s:e] for v in views], dsalt)
        except (ValueError, OSError, RuntimeError):
            self.failures += 1
            return 0
        self.saved_blocks += written
        return written

    # ---- in: called for a new request before it is scheduled ----
    def restore(self, tokens: Sequence[int], salt: int = 0) -> int:
        """Brings rows from disk into the device's prefix cache when that covers more of `tokens` than the
        device already holds; returns the positions restored (0 when there was nothing to gain)."""
        from ..cluster.handover import MAGIC, import_sequence, model_identity

        toks = [int(t) for t in tokens]
        if len(toks) <= DISK_BLOCK:
            return 0
        dsalt = self._salt(salt)
        have = len(self.alloc.match_prefix(toks, salt)[0]) * self.alloc.block_size
        n = self.tier.match(toks[:len(toks) - 1], dsalt)             # the last token is always computed
        if n <= have or not self.alloc.can_allocate(n):
            return 0
        chunks: List[list] = []
        got = self.tier.load(toks[:n], lambda s, e, planes: chunks.append(planes), dsalt)
        if got <= have or not chunks:
            return 0
        local = [l for l in self.runner.kv if l is not None]
        L = local[0]
        dests = [L.k, L.k_scale, L.v, L.v_scale] if L.q8 else [L.k, L.v]
        per_layer = len(dests)
        if any(len(c) != per_layer * len(local) for c in chunks):
            self.failures += 1
            return 0
        head = {"format": "q8" if L.q8 else "bf16", "tokens": toks[:got], "n": got, "layers": len(local),
                "n_kv": self.runner.w.n_kv_local, "head_dim": self.runner.cfg.head_dim, "model": model_identity(self.runner),
                "planes": [[[got] + list(d.shape[1:]), str(d.dtype)] for d in dests]}
        hb = json.dumps(head).encode()
        parts = [MAGIC, struct.pack("<I", len(hb)), hb]
        for i in range(per_layer * len(local)):
            for c in chunks:
                parts.append(np.ascontiguousarray(c[i]).tobytes())
        tmp = -(1 << 40) - self.restored_tokens - 1                   # an id no request or hand-over uses
        try:
            import_sequence(self.runner, self.alloc, tmp, b"".join(parts), salt)
        except (ValueError, MemoryError):
            self.failures += 1
            return 0
        self.alloc.free(tmp)              # the blocks stay published (idle, evictable) under their content hashes
        self.restored_tokens += got
        return got

    def stats(self) -> dict:
        out = {"saved_blocks": self.saved_blocks, "restored_tokens": self.restored_tokens, "failures": self.failures,
               "disk_bytes": self.tier.bytes_used()}
        if self.tier.tiers is not None:
            out["tiers"] = self.tier.tiers.stats()
        return out
