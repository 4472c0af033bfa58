"""Where a cache block lives when it is not on the card, and what must hold when it comes back.

A block that leaves device memory is not dead: reading it back from host memory, from disk or from a peer
is cheaper than prefilling its tokens again.  So eviction is a move between tiers (host, disk, peer), and
the one property everything rests on is that a block that comes back is the block that left: a cache is
read as exact state, a single changed byte yields fluent text from a context that never existed.  Every
round trip is therefore checked against a digest taken before the move, and a mismatch is an error, never
a warning (reference: `src/distributed/kv_tiers.rs:1-19`, `:101-167`).

This module is the bookkeeping and the integrity rule over pluggable stores (memory, a directory, a pair
of functions that reach a peer).  The disk tier of the cache (`serve/kv_disk.py`) keeps its recently used
blocks in a host tier through it, so a conversation that returns within minutes is restored from memory.
"""
from __future__ import annotations

import enum
import hashlib
import os
import threading
from collections import OrderedDict
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple


class Tier(enum.IntEnum):
    """Cheapest to reach first."""
    HOST = 1      # host memory: one copy over the bus away
    DISK = 2      # survives an unload and a restart, costs a read
    PEER = 3      # another node's memory: the only tier that can fail because something else died


class IntegrityError(RuntimeError):
    """A block came back different from how it left."""


def digest(data: bytes) -> int:
    """64 bits of BLAKE2b.  Guards against truncated reads, stale buffers and partial transfers; what matters
    is that it is exact and stable, so a mismatch always means the bytes changed."""
    return int.from_bytes(hashlib.blake2b(data, digest_size=8).digest(), "little")


@dataclass
class BlockLocation:
    tier: Tier
    digest: int
    nbytes: int


class MemoryStore:
    def __init__(self):
        self.blocks: Dict[int, bytes] = {}

    def put(self, key: int, data: bytes):
        self.blocks[key] = bytes(data)

    def get(self, key: int) -> bytes:
        try:
            return self.blocks[key]
        except KeyError:
            raise KeyError(f"block {key:016x} is not in this store")

    def drop(self, key: int):
        self.blocks.pop(key, None)

    def has(self, key: int) -> bool:
        return key in self.blocks


class DirStore:
    """One file per block, written to a temporary name and renamed."""

    def __init__(self, directory: str, suffix: str = ".blk"):
        self.dir, self.suffix = directory, suffix
        os.makedirs(directory, exist_ok=True)

    def path(self, key: int) -> str:
        return os.path.join(self.dir, f"{key:016x}{self.suffix}")

    def put(self, key: int, data: bytes):
        tmp = self.path(key) + ".tmp"
        with open(tmp, "wb") as f:
            f.write(data)
        os.replace(tmp, self.path(key))

    def get(self, key: int) -> bytes:
        try:
            with open(self.path(key), "rb") as f:
                return f.read()
        except OSError as e:
            raise KeyError(f"block {key:016x}: {e}")

    def drop(self, key: int):
        try:
            os.remove(self.path(key))
        except OSError:
            pass

    def has(self, key: int) -> bool:
        return os.path.exists(self.path(key))


class PeerStore:
    """Blocks kept in another node's memory, reached through two functions (HTTP in a server, plain calls in
    tests).  Any failure of the peer reads as "not there"."""

    def __init__(self, put: Callable[[int, bytes], None], get: Callable[[int], bytes], drop: Optional[Callable[[int], None]] = None):
        self._put, self._get, self._drop = put, get, drop

    def put(self, key: int, data: bytes):
        self._put(key, data)

    def get(self, key: int) -> bytes:
        try:
            return self._get(key)
        except KeyError:
            raise
        except Exception as e:
            raise KeyError(f"block {key:016x}: the peer did not answer ({e})")

    def drop(self, key: int):
        if self._drop is not None:
            try:
                self._drop(key)
            except Exception:
                pass

    def has(self, key: int) -> bool:
        try:
            self._get(key)
            return True
        except Exception:
            return False


class TieredKv:
    """The map block -> (tier, digest, size), the moves between tiers, and the host tier's budget.

    `admit` puts a block into host memory; when the host tier is over `host_bytes` its least recently used
    blocks are demoted to the next tier that exists (disk, else peer) or, with none, dropped.  `promote`
    returns a block's bytes from wherever it is, checked against its digest, and moves it back to the host
    tier.  With `write_through` a block admitted to the host tier is also written to the disk tier at once
    (persistence does not wait for memory pressure)."""

    def __init__(self, stores: Dict[Tier, object], host_bytes: int = 256 << 20, write_through: bool = False):
        self.stores = dict(stores)
        self.stores.setdefault(Tier.HOST, MemoryStore())
        self.host_bytes = int(host_bytes)
        self.write_through = write_through and Tier.DISK in self.stores
        self.map: Dict[int, BlockLocation] = {}
        self.lru: "OrderedDict[int, None]" = OrderedDict()        # blocks in the host tier, oldest first
        self.host_used = 0
        self.hits = {t: 0 for t in Tier}
        self.integrity_failures = 0
        self._evicted: List[Tuple[int, Tier]] = []
        self.lock = threading.RLock()

    # ---- where ----
    def locate(self, key: int) -> Optional[BlockLocation]:
        return self.map.get(key)

    def has(self, key: int) -> bool:
        with self.lock:
            loc = self.map.get(key)
            if loc is not None:
                return True
            # a block the disk tier holds from an earlier run is adopted on first sight (digest taken on read)
            d = self.stores.get(Tier.DISK)
            return d is not None and d.has(key)

    # ---- in ----
    def admit(self, key: int, data: bytes):
        data = bytes(data)
        with self.lock:
            dg = digest(data)
            old = self.map.get(key)
            if old is not None and old.tier == Tier.HOST:
                self.host_used -= old.nbytes
            self.stores[Tier.HOST].put(key, data)
            self.map[key] = BlockLocation(Tier.HOST, dg, len(data))
            self.lru[key] = None
            self.lru.move_to_end(key)
            self.host_used += len(data)
            if self.write_through:
                self.stores[Tier.DISK].put(key, data)
            self._shrink()

    def _next_tier(self) -> Optional[Tier]:
        for t in (Tier.DISK, Tier.PEER):
            if t in self.stores:
                return t
        return None

    def _shrink(self):
        while self.host_used > self.host_bytes and self.lru:
            key, _ = self.lru.popitem(last=False)
            to = self._next_tier()
            if to is None:
                self._forget(key, Tier.HOST)
                continue
            try:
                self.demote(key, to)
            except (IntegrityError, KeyError):
                continue                    # a damaged block is forgotten by demote; the admit that made room goes on

    def _forget(self, key: int, tier: Tier):
        loc = self.map.pop(key, None)
        self.stores[tier].drop(key)
        if loc is not None and loc.tier == Tier.HOST:
            self.host_used -= loc.nbytes
        self.lru.pop(key, None)
        self._evicted.append((key, tier))

    # ---- between tiers ----
    def demote(self, key: int, to: Tier):
        """Moves a block down (host -> disk / peer, disk -> peer).  The bytes are verified on the way."""
        with self.lock:
            loc = self.map.get(key)
            if loc is None:
                raise KeyError(f"block {key:016x} is not known")
            if to <= loc.tier:
                raise ValueError("demote moves a block to a slower tier")
            data = self.stores[loc.tier].get(key)
            if digest(data) != loc.digest:
                self.integrity_failures += 1
                self._forget(key, loc.tier)
                raise IntegrityError(f"block {key:016x} changed while it sat in the {loc.tier.name.lower()} tier")
            already = to == Tier.DISK and self.write_through and self.stores[to].has(key)
            if not already:
                self.stores[to].put(key, data)
            self.stores[loc.tier].drop(key)
            if loc.tier == Tier.HOST:
                self.host_used -= loc.nbytes
                self.lru.pop(key, None)
            self.map[key] = BlockLocation(to, loc.digest, loc.nbytes)

    def promote(self, key: int) -> bytes:
        """The block's bytes, verified; afterwards it sits in the host tier (its slower copy is kept when the
        disk tier writes through, else removed)."""
        with self.lock:
            loc = self.map.get(key)
            if loc is None:
                d = self.stores.get(Tier.DISK)
                if d is None or not d.has(key):
                    raise KeyError(f"block {key:016x} is not known")
                data = d.get(key)                       # left by an earlier run: trusted as the container format checks it
                loc = BlockLocation(Tier.DISK, digest(data), len(data))
                self.map[key] = loc
            else:
                try:
                    data = self.stores[loc.tier].get(key)
                except KeyError:
                    self._forget(key, loc.tier)
                    raise
            if digest(data) != loc.digest or len(data) != loc.nbytes:
                self.integrity_failures += 1
                self._forget(key, loc.tier)
                raise IntegrityError(f"block {key:016x} came back from the {loc.tier.name.lower()} tier different from how it left")
            self.hits[loc.tier] += 1
            if loc.tier == Tier.HOST:
                self.lru.move_to_end(key)
                return data
            keep = loc.tier == Tier.DISK and self.write_through
            if not keep:
                self.stores[loc.tier].drop(key)
            self.stores[Tier.HOST].put(key, data)
            self.map[key] = BlockLocation(Tier.HOST, loc.digest, loc.nbytes)
            self.lru[key] = None
            self.host_used += loc.nbytes
            self._shrink()
            return data

    def drop(self, key: int):
        with self.lock:
            loc = self.map.get(key)
            if loc is not None:
                self._forget(key, loc.tier)
            if self.write_through:
                self.stores[Tier.DISK].drop(key)

    def evicted(self) -> List[Tuple[int, Tier]]:
        """Blocks that were dropped since the last call (no slower tier to go to, or damaged)."""
        with self.lock:
            out, self._evicted = self._evicted, []
            return out

    def stats(self) -> dict:
        with self.lock:
            per = {t.name.lower(): 0 for t in Tier}
            for loc in self.map.values():
                per[loc.tier.name.lower()] += 1
            return {"blocks": per, "host_bytes": self.host_used, "host_budget": self.host_bytes,
                    "hits": {t.name.lower(): n for t, n in self.hits.items()}, "integrity_failures": self.integrity_failures}
