"""Cache blocks off the card: the tier map with its integrity rule, and the engine-side glue of the disk tier
(a finished sequence's rows go out, a returning prompt's rows come back) on a CPU stand-in of the runner."""
import os
import types

import pytest
import torch

from loken_b200.serve.kv_disk import DISK_BLOCK, KvDiskTier
from loken_b200.serve.kv_manager import PagedKvAllocator
from loken_b200.serve.kv_persist import DiskPersistence
from loken_b200.serve.kv_tiers import DirStore, IntegrityError, MemoryStore, PeerStore, Tier, TieredKv, digest


def blk(i, n=1000):
    return bytes((i * 7 + j) & 255 for j in range(n))


def test_blocks_move_down_under_pressure_and_come_back_exact(tmp_path):
    t = TieredKv({Tier.DISK: DirStore(str(tmp_path))}, host_bytes=3500)
    for i in range(6):
        t.admit(i, blk(i))
    assert t.host_used <= 3500 and t.stats()["blocks"] == {"host": 3, "disk": 3, "peer": 0}
    assert t.locate(0).tier == Tier.DISK and t.locate(5).tier == Tier.HOST
    assert t.promote(0) == blk(0) and t.locate(0).tier == Tier.HOST           # back in memory, something else went down
    assert t.stats()["blocks"]["host"] == 3 and not os.path.exists(DirStore(str(tmp_path)).path(0))
    assert t.promote(5) == blk(5) and t.hits[Tier.HOST] == 1 and t.hits[Tier.DISK] == 1
    with pytest.raises(KeyError):
        t.promote(99)
    with pytest.raises(ValueError):
        t.demote(1, Tier.HOST)
    t.drop(5)
    assert t.locate(5) is None and (5, Tier.HOST) in t.evicted() and t.evicted() == []
    # without a slower tier, pressure drops the oldest block and says so
    solo = TieredKv({}, host_bytes=2500)
    for i in range(4):
        solo.admit(i, blk(i))
    assert [k for k, _ in solo.evicted()] == [0, 1] and solo.has(3) and not solo.has(0)


def test_a_block_that_changed_is_an_error_never_a_warning(tmp_path):
    d = DirStore(str(tmp_path))
    t = TieredKv({Tier.DISK: d}, host_bytes=1500)
    t.admit(1, blk(1))
    t.admit(2, blk(2))                                   # 1 goes to disk
    assert t.locate(1).tier == Tier.DISK
    raw = bytearray(open(d.path(1), "rb").read())
    raw[500] ^= 1                                        # one flipped bit
    open(d.path(1), "wb").write(raw)
    with pytest.raises(IntegrityError):
        t.promote(1)
    assert t.locate(1) is None and t.integrity_failures == 1 and not d.has(1)
    # a truncated host copy is caught on the way down too
    t.stores[Tier.HOST].blocks[2] = blk(2)[:-1]
    with pytest.raises(IntegrityError):
        t.demote(2, Tier.DISK)
    assert digest(blk(1)) != digest(bytes(raw)) and digest(b"") == digest(b"")


def test_peer_tier_and_write_through(tmp_path):
    remote = MemoryStore()
    down = {"on": False}

    def get(k):
        if down["on"]:
            raise ConnectionError("peer is gone")
        return remote.get(k)

    t = TieredKv({Tier.PEER: PeerStore(remote.put, get, remote.drop)}, host_bytes=1500)
    t.admit(1, blk(1))
    t.admit(2, blk(2))
    assert t.locate(1).tier == Tier.PEER and remote.has(1)
    down["on"] = True
    with pytest.raises(KeyError):
        t.promote(1)                                     # the only tier that fails because something else died
    assert t.locate(1) is None
    # written through: the disk copy exists at once and survives a new process
    wt = TieredKv({Tier.DISK: DirStore(str(tmp_path))}, host_bytes=1500, write_through=True)
    wt.admit(7, blk(7))
    assert DirStore(str(tmp_path)).has(7) and wt.locate(7).tier == Tier.HOST
    wt.admit(8, blk(8))
    assert wt.locate(7).tier == Tier.DISK
    again = TieredKv({Tier.DISK: DirStore(str(tmp_path))}, host_bytes=1500, write_through=True)
    assert again.has(7) and again.promote(7) == blk(7) and DirStore(str(tmp_path)).has(7)


def engine(tmp, n_layers=2, name="a", blocks=64, host_bytes=1 << 20):
    from loken_b200.models.config import tiny
    from loken_b200.ops.rows import KVCacheLayer

    cfg = tiny("llama", n_layers=n_layers)
    cfg.name = name
    kv = [KVCacheLayer(blocks * 16, 2, cfg.head_dim, "cpu", q8=True) for _ in range(n_layers)]
    runner = types.SimpleNamespace(cfg=cfg, kv=kv, device=torch.device("cpu"), w=types.SimpleNamespace(n_kv_local=2))
    alloc = PagedKvAllocator(blocks, 16)
    return runner, alloc, DiskPersistence(runner, alloc, KvDiskTier(str(tmp), host_bytes=host_bytes))


def fill(runner, alloc, sid, n, seed):
    assert alloc.allocate(sid, n)
    g = torch.Generator().manual_seed(seed)
    slots = torch.tensor(alloc.slots_for_range(sid, 0, n))
    for l in runner.kv:
        l.k[slots] = torch.randint(-100, 100, l.k[slots].shape, generator=g, dtype=torch.int8)
        l.v[slots] = torch.randint(-100, 100, l.v[slots].shape, generator=g, dtype=torch.int8)
        l.k_scale[slots] = torch.rand(l.k_scale[slots].shape, generator=g).to(l.k_scale.dtype)
        l.v_scale[slots] = torch.rand(l.v_scale[slots].shape, generator=g).to(l.v_scale.dtype)
    return slots


def test_a_finished_sequence_leaves_its_blocks_and_a_new_engine_finds_them(tmp_path):
    r1, a1, d1 = engine(tmp_path)
    toks = [(i * 31) % 200 for i in range(2 * DISK_BLOCK + 40)]
    s1 = fill(r1, a1, 1, len(toks), seed=3)
    assert d1.save(1, toks, len(toks)) == 2                                    # two full blocks; the tail of 40 stays
    assert d1.save(1, toks, len(toks)) == 0                                    # nothing new the second time
    # "restart": another process, an empty device cache, the same directory
    r2, a2, d2 = engine(tmp_path)
    prompt = toks + [5, 6, 7]
    assert d2.restore(prompt) == 2 * DISK_BLOCK
    blocks, _ = a2.match_prefix(prompt)
    assert len(blocks) * 16 == 2 * DISK_BLOCK                                  # the request's prefill starts after them
    got = torch.tensor([b * 16 + j for b in blocks for j in range(16)])
    for l1, l2 in zip(r1.kv, r2.kv):
        assert torch.equal(l2.k[got], l1.k[s1[:2 * DISK_BLOCK]]) and torch.equal(l2.v_scale[got], l1.v_scale[s1[:2 * DISK_BLOCK]])
    assert d2.restore(prompt) == 0                                             # the device holds them now
    assert a2.free_blocks() == 64 and d2.stats()["restored_tokens"] == 2 * DISK_BLOCK
    # a prompt that shares only the first block restores one
    r3, a3, d3 = engine(tmp_path)
    assert d3.restore(toks[:DISK_BLOCK] + [9] * 300) == DISK_BLOCK
    # another model with the same tokenizer sees nothing, and neither does another cache scope
    r4, a4, d4 = engine(tmp_path, name="b")
    assert d4.restore(prompt) == 0
    r5, a5, d5 = engine(tmp_path)
    assert d5.restore(prompt, salt=77) == 0
    # a damaged block file ends the restore where the damage starts
    r6, a6, d6 = engine(tmp_path, host_bytes=0)
    files = sorted(os.listdir(os.path.join(str(tmp_path), "blocks")))
    assert len(files) == 2
    hs = __import__("loken_b200.serve.kv_manager", fromlist=["block_hashes"]).block_hashes(toks[:2 * DISK_BLOCK], DISK_BLOCK, d6._salt(0))
    second = os.path.join(str(tmp_path), "blocks", f"{hs[1]:016x}.kv")
    raw = bytearray(open(second, "rb").read())
    raw[100] ^= 4
    open(second, "wb").write(raw)
    assert d6.restore(prompt) == DISK_BLOCK
    # no room on the device: nothing is taken
    r7, a7, d7 = engine(tmp_path, blocks=8)
    assert d7.restore(prompt) == 0 and a7.free_blocks() == 8
