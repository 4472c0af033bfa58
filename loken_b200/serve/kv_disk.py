"""Disk tier of the KV cache: finished conversations' cache blocks survive a restart.

Layout (`src/inference/cache/kv_disk.rs`): the cache of a sequence is cut into blocks of 256
tokens; a block's file name is the FNV-1a chain hash of the tokens up to and including it, so
equal prefixes of different conversations share files; a manifest per sequence lists its block
hashes and token ids.  Each block file is a container with a 20-byte header — magic "LKKD",
u16 version, u16 flags (bit 0: zlib-compressed payload), u32 crc32 of the payload, u64 payload
length — followed by the planes of every layer for those positions.  The reference offers zstd
for the payload (`docs/CONFIGURATION.md:286-294`); this build compresses with zlib, which is in the
standard library.
"""
from __future__ import annotations

import json
import os
import struct
import zlib
from typing import Dict, List, Optional, Sequence

import numpy as np

from .kv_manager import block_hashes

MAGIC = b"LKKD"
VERSION = 1
DISK_BLOCK = 256
HEADER = struct.Struct("<4sHHIQ")      # 20 bytes


def pack_container(payload: bytes, compress: bool = False) -> bytes:
    flags = 0
    if compress:
        payload = zlib.compress(payload, 3)
        flags |= 1
    return HEADER.pack(MAGIC, VERSION, flags, zlib.crc32(payload) & 0xFFFFFFFF, len(payload)) + payload


def unpack_container(blob: bytes) -> bytes:
    if len(blob) < HEADER.size:
        raise ValueError("truncated container")
    magic, ver, flags, crc, n = HEADER.unpack_from(blob)
    if magic != MAGIC or ver != VERSION:
        raise ValueError("not a KV disk container")
    payload = blob[HEADER.size:HEADER.size + n]
    if len(payload) != n or (zlib.crc32(payload) & 0xFFFFFFFF) != crc:
        raise ValueError("container payload is damaged")
    return zlib.decompress(payload) if flags & 1 else payload


class KvDiskTier:
    """`host_bytes` > 0 keeps the most recently written or read block files in host memory as well
    (`serve/kv_tiers.py`: a host tier in front of the directory, written through, every block verified
    against its digest when it comes back), so a conversation that returns soon is restored without a read."""

    def __init__(self, directory: str, compress: bool = False, max_bytes: Optional[int] = None, host_bytes: int = 0):
        self.dir = directory
        self.compress = compress
        self.max_bytes = max_bytes
        os.makedirs(os.path.join(directory, "blocks"), exist_ok=True)
        os.makedirs(os.path.join(directory, "manifests"), exist_ok=True)
        self.tiers = None
        if host_bytes > 0:
            from .kv_tiers import DirStore, Tier, TieredKv

            self.tiers = TieredKv({Tier.DISK: DirStore(os.path.join(directory, "blocks"), ".kv")}, host_bytes, write_through=True)

    def _block_path(self, h: int) -> str:
        return os.path.join(self.dir, "blocks", f"{h:016x}.kv")

    def has_block(self, h: int) -> bool:
        return os.path.exists(self._block_path(h))

    # ---- write ----
    def save(self, key: str, tokens: Sequence[int], read_block, salt: int = 0) -> int:
        """Stores the full 256-token blocks of `tokens`.  `read_block(start, end)` returns the cache
        planes of positions [start, end) as a list of numpy arrays (all layers, fixed order).
        Returns the number of block files written (shared prefixes are not rewritten)."""
        hashes = block_hashes(list(tokens), DISK_BLOCK, salt)
        written = 0
        for b, h in enumerate(hashes):
            if self.has_block(h):
                continue
            planes = read_block(b * DISK_BLOCK, (b + 1) * DISK_BLOCK)
            head = json.dumps([[list(p.shape), str(p.dtype)] for p in planes]).encode()
            body = struct.pack("<I", len(head)) + head + b"".join(np.ascontiguousarray(p).tobytes() for p in planes)
            blob = pack_container(body, self.compress)
            if self.tiers is not None:
                self.tiers.admit(h, blob)           # host memory and, written through, the block file
            else:
                tmp = self._block_path(h) + ".tmp"
                with open(tmp, "wb") as f:
                    f.write(blob)
                os.replace(tmp, self._block_path(h))
            written += 1
        man = {"key": key, "tokens": [int(t) for t in tokens[:len(hashes) * DISK_BLOCK]], "salt": salt,
               "blocks": [f"{h:016x}" for h in hashes]}
        with open(os.path.join(self.dir, "manifests", _safe(key) + ".json"), "w") as f:
            json.dump(man, f)
        if self.max_bytes:
            self.evict_to(self.max_bytes)
        return written

    # ---- read ----
    def match(self, tokens: Sequence[int], salt: int = 0) -> int:
        """Number of leading tokens whose blocks are on disk."""
        n = 0
        for h in block_hashes(list(tokens), DISK_BLOCK, salt):
            if not self.has_block(h):
                break
            n += DISK_BLOCK
        return n

    def load(self, tokens: Sequence[int], write_block, salt: int = 0) -> int:
        """Feeds the stored blocks of the longest on-disk prefix to `write_block(start, end, planes)`;
        returns the number of tokens restored.  A damaged block ends the restore at its start."""
        n = 0
        for b, h in enumerate(block_hashes(list(tokens), DISK_BLOCK, salt)):
            if not self.has_block(h):
                break
            try:
                if self.tiers is not None:
                    body = unpack_container(self.tiers.promote(h))
                else:
                    with open(self._block_path(h), "rb") as f:
                        body = unpack_container(f.read())
            except (ValueError, OSError, zlib.error, KeyError, RuntimeError):
                break
            (hl,) = struct.unpack_from("<I", body)
            desc = json.loads(body[4:4 + hl])
            off = 4 + hl
            planes = []
            for shape, dt in desc:
                a = np.frombuffer(body, dtype=np.dtype(dt), count=int(np.prod(shape)), offset=off).reshape(shape)
                off += a.nbytes
                planes.append(a)
            write_block(b * DISK_BLOCK, (b + 1) * DISK_BLOCK, planes)
            os.utime(self._block_path(h))
            n += DISK_BLOCK
        return n

    def manifests(self) -> List[dict]:
        out = []
        d = os.path.join(self.dir, "manifests")
        for name in sorted(os.listdir(d)):
            try:
                with open(os.path.join(d, name)) as f:
                    out.append(json.load(f))
            except (OSError, ValueError):
                continue
        return out

    def bytes_used(self) -> int:
        d = os.path.join(self.dir, "blocks")
        return sum(os.path.getsize(os.path.join(d, n)) for n in os.listdir(d))

    def evict_to(self, max_bytes: int) -> int:
        """Removes the least recently used block files until the tier fits."""
        d = os.path.join(self.dir, "blocks")
        files = sorted(((os.path.getmtime(os.path.join(d, n)), n) for n in os.listdir(d) if n.endswith(".kv")))
        used = self.bytes_used()
        removed = 0
        for _, n in files:
            if used <= max_bytes:
                break
            p = os.path.join(d, n)
            used -= os.path.getsize(p)
            os.remove(p)
            removed += 1
        return removed


def _safe(key: str) -> str:
    return "".join(c if c.isalnum() or c in "-_." else "_" for c in key)[:120] or "seq"


def runner_block_io(runner, alloc, seq_id: int):
    """(read_block, write_block) over a runner's paged cache for one sequence."""
    import torch

    def planes_of(layer):
        return [layer.k, layer.k_scale, layer.v, layer.v_scale] if layer.q8 else [layer.k, layer.v]

    def read_block(start, end):
        slots = torch.tensor(alloc.slots_for_range(seq_id, start, end), dtype=torch.int64, device=runner.device)
        out = []
        for layer in runner.kv:
            if layer is None:
                continue
            for p in planes_of(layer):
                t = p[slots].contiguous().cpu()
                out.append(t.view(torch.int16).numpy() if t.dtype in (torch.bfloat16,) else t.numpy())
        return out

    def write_block(start, end, planes):
        slots = torch.tensor(alloc.slots_for_range(seq_id, start, end), dtype=torch.int64, device=runner.device)
        it = iter(planes)
        for layer in runner.kv:
            if layer is None:
                continue
            for p in planes_of(layer):
                a = torch.from_numpy(np.array(next(it)))
                if p.dtype == torch.bfloat16:
                    a = a.view(torch.bfloat16)
                p[slots] = a.to(runner.device)

    return read_block, write_block
