"""Paged KV block allocator with automatic prefix caching.

Semantics follow the reference's `PagedKvAllocator` / `PrefixCache`
(`src/inference/cache/paged_kv.rs:53-510`):
  * fixed-size blocks (16 tokens by default), LIFO free list;
  * a content hash per FULL block, chained through its parent's hash (FNV-1a), so equal
    prefixes of different requests map to the same blocks; only full blocks are cached;
  * cached blocks are reference counted; a block whose count drops to zero stays in the cache
    and is evictable (oldest first), and evictable blocks count as free capacity;
  * a finished prompt's full blocks are committed; an abandoned partial prefill is not;
  * `trim` cuts a sequence back (speculative rejects), `free` releases it.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

FNV_OFFSET = 0xCBF29CE484222325
FNV_PRIME = 0x100000001B3
MASK64 = (1 << 64) - 1


def fnv1a_block(parent: int, tokens: Sequence[int], salt: int = 0) -> int:
    h = (FNV_OFFSET ^ (parent & MASK64) ^ (salt & MASK64)) & MASK64
    h = (h * FNV_PRIME) & MASK64
    for t in tokens:
        v = int(t) & 0xFFFFFFFF
        for _ in range(4):
            h ^= v & 0xFF
            h = (h * FNV_PRIME) & MASK64
            v >>= 8
    return h


def block_hashes(tokens: Sequence[int], block_size: int, salt: int = 0) -> List[int]:
    """Hash chain over the full blocks of `tokens`."""
    out, parent = [], 0
    for b in range(len(tokens) // block_size):
        parent = fnv1a_block(parent, tokens[b * block_size:(b + 1) * block_size], salt)
        out.append(parent)
    return out


@dataclass
class _Seq:
    blocks: List[int] = field(default_factory=list)
    length: int = 0                 # tokens whose KV the sequence owns
    hashes: List[int] = field(default_factory=list)   # hash of each committed (cached) leading block
    publish_limit: Optional[int] = None   # after a context shift: only blocks below this index may be published


class PagedKvAllocator:
    def __init__(self, num_blocks: int, block_size: int = 16, enable_prefix_cache: bool = True):
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.enable_prefix_cache = enable_prefix_cache
        self.free_list: List[int] = list(range(num_blocks - 1, -1, -1))   # pop() yields block 0 first
        self.seqs: Dict[int, _Seq] = {}
        self.ref: List[int] = [0] * num_blocks
        self.block_hash: List[Optional[int]] = [None] * num_blocks
        self.cached: Dict[int, int] = {}                  # hash -> block
        self.evictable: "OrderedDict[int, None]" = OrderedDict()   # idle cached blocks, oldest first
        self.hits = 0
        self.queries = 0

    # ---- capacity ----
    def free_blocks(self) -> int:
        return len(self.free_list) + len(self.evictable)

    def blocks_needed(self, n_tokens: int) -> int:
        return (n_tokens + self.block_size - 1) // self.block_size

    def can_allocate(self, n_tokens: int, have_blocks: int = 0) -> bool:
        return self.blocks_needed(n_tokens) - have_blocks <= self.free_blocks()

    def _take(self) -> Optional[int]:
        if self.free_list:
            return self.free_list.pop()
        if self.evictable:
            b, _ = self.evictable.popitem(last=False)
            h = self.block_hash[b]
            if h is not None and self.cached.get(h) == b:
                del self.cached[h]
            self.block_hash[b] = None
            return b
        return None

    def _release(self, b: int):
        self.ref[b] -= 1
        assert self.ref[b] >= 0
        if self.ref[b] == 0:
            if self.block_hash[b] is not None and self.cached.get(self.block_hash[b]) == b:
                self.evictable[b] = None
            else:
                self.block_hash[b] = None
                self.free_list.append(b)

    # ---- sequences ----
    def match_prefix(self, tokens: Sequence[int], salt: int = 0) -> Tuple[List[int], List[int]]:
        """Longest run of cached leading blocks for `tokens` (never the whole prompt: the last
        token is always computed so there are logits to sample from)."""
        if not self.enable_prefix_cache:
            return [], []
        hs = block_hashes(tokens, self.block_size, salt)
        blocks, used = [], []
        max_full = (len(tokens) - 1) // self.block_size
        for h in hs[:max_full]:
            b = self.cached.get(h)
            if b is None:
                break
            blocks.append(b)
            used.append(h)
        return blocks, used

    def allocate_with_prefix(self, seq_id: int, tokens: Sequence[int], salt: int = 0) -> Optional[int]:
        """Reserves blocks for all of `tokens`; returns the number of leading tokens whose KV is
        already cached, or None when the pool cannot hold the request."""
        assert seq_id not in self.seqs
        self.queries += 1
        blocks, hs = self.match_prefix(tokens, salt)
        # matched blocks that sit in the evictable set stop being free capacity once claimed
        idle = sum(1 for b in blocks if self.ref[b] == 0)
        need = self.blocks_needed(len(tokens)) - len(blocks)
        if need > self.free_blocks() - idle:
            return None
        for b in blocks:
            if self.ref[b] == 0:
                self.evictable.pop(b, None)
            self.ref[b] += 1
        s = _Seq(list(blocks), len(tokens), list(hs))
        for _ in range(need):
            b = self._take()
            assert b is not None
            self.ref[b] = 1
            s.blocks.append(b)
        self.seqs[seq_id] = s
        if blocks:
            self.hits += 1
        return len(blocks) * self.block_size

    def allocate(self, seq_id: int, n_tokens: int) -> bool:
        assert seq_id not in self.seqs
        need = self.blocks_needed(n_tokens)
        if need > self.free_blocks():
            return False
        s = _Seq([], n_tokens, [])
        for _ in range(need):
            b = self._take()
            self.ref[b] = 1
            s.blocks.append(b)
        self.seqs[seq_id] = s
        return True

    def append(self, seq_id: int, n: int = 1) -> bool:
        """Grows the sequence by n tokens, taking new blocks as needed."""
        s = self.seqs[seq_id]
        need = self.blocks_needed(s.length + n) - len(s.blocks)
        if need > self.free_blocks():
            return False
        for _ in range(need):
            b = self._take()
            self.ref[b] = 1
            s.blocks.append(b)
        s.length += n
        return True

    def commit_prefix(self, seq_id: int, tokens: Sequence[int], salt: int = 0):
        """Publishes the sequence's full blocks (their KV is complete) under their content hash."""
        if not self.enable_prefix_cache:
            return
        s = self.seqs[seq_id]
        hs = block_hashes(tokens[:s.length], self.block_size, salt)
        top = min(len(hs), len(s.blocks)) if s.publish_limit is None else min(len(hs), len(s.blocks), s.publish_limit)
        for i in range(len(s.hashes), top):
            h, b = hs[i], s.blocks[i]
            if h in self.cached and self.cached[h] != b:
                pass    # an equal block is already published; keep ours private
            elif self.block_hash[b] is None:
                self.cached[h] = b
                self.block_hash[b] = h
            s.hashes.append(h)

    def trim(self, seq_id: int, new_len: int):
        s = self.seqs[seq_id]
        assert new_len <= s.length
        keep = self.blocks_needed(new_len)
        while len(s.blocks) > keep:
            self._release(s.blocks.pop())
        s.hashes = s.hashes[:min(len(s.hashes), new_len // self.block_size)]
        s.length = new_len

    def shift(self, seq_id: int, n_keep: int, n_discard: int):
        """Context shift: positions [n_keep, n_keep + n_discard) leave the sequence and everything after
        them moves down by n_discard.  Whole blocks inside the kept head stay as they are (they may be
        shared); the rest of the sequence moves into fresh blocks, so nothing shared is written and the
        copy never overlaps its source.  Returns (src slots, dst slots, deltas) for the positions that
        move, new position order, or None when the pool has no room for the copy.  The old blocks are
        released here: the caller enqueues the copy on the stream before anything else can reuse them.
        Blocks past the kept head are never published: their keys were computed in a context that no
        longer exists."""
        s = self.seqs[seq_id]
        bs = self.block_size
        L = s.length
        assert 0 <= n_keep and n_discard > 0 and n_keep + n_discard <= L
        new_len = L - n_discard
        kb = n_keep // bs
        need = self.blocks_needed(new_len) - kb
        if need > self.free_blocks():
            return None
        old = s.blocks
        fresh = []
        for _ in range(need):
            b = self._take()
            self.ref[b] = 1
            fresh.append(b)
        new = old[:kb] + fresh
        src, dst, delta = [], [], []
        for p in range(kb * bs, new_len):
            q = p if p < n_keep else p + n_discard
            src.append(old[q // bs] * bs + q % bs)
            dst.append(new[p // bs] * bs + p % bs)
            delta.append(0 if p < n_keep else -n_discard)
        for b in reversed(old[kb:]):
            self._release(b)
        s.blocks = new
        s.length = new_len
        s.hashes = s.hashes[:min(len(s.hashes), kb)]
        s.publish_limit = kb
        return src, dst, delta

    def free(self, seq_id: int):
        s = self.seqs.pop(seq_id, None)
        if s is None:
            return
        for b in reversed(s.blocks):
            self._release(b)

    def num_free(self) -> int:
        """Blocks a new sequence could take right now (free list + idle cached blocks)."""
        return self.free_blocks()

    def reset_prefix_cache(self) -> int:
        """Drops every idle cached block; returns how many went back to the free list.  Blocks
        still referenced by a running sequence stay published."""
        dropped = len(self.evictable)
        for b in list(self.evictable):
            self.block_hash[b] = None
            self.free_list.append(b)
        self.evictable.clear()
        self.cached = {h: b for h, b in self.cached.items() if self.ref[b] > 0}
        return dropped

    # ---- views ----
    def length(self, seq_id: int) -> int:
        return self.seqs[seq_id].length

    def block_table(self, seq_id: int) -> List[int]:
        return self.seqs[seq_id].blocks

    def slot(self, seq_id: int, pos: int) -> int:
        s = self.seqs[seq_id]
        return s.blocks[pos // self.block_size] * self.block_size + pos % self.block_size

    def slots_for_range(self, seq_id: int, start: int, end: int) -> List[int]:
        s = self.seqs[seq_id]
        bs = self.block_size
        return [s.blocks[p // bs] * bs + p % bs for p in range(start, end)]
