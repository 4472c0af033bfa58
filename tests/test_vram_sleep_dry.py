"""Device-memory authority (reclaim order, eviction, epochs), sleeping models and the dry plan with
its heap replay: all on injected probes, no GPU."""
import os

from loken_b200.models.config import get_config
from loken_b200.place.dry import HeapReplay, dry_demand, fits
from loken_b200.place.sleep import SleepRegistry, model_files
from loken_b200.place.vram import GiB, VramAuthority, host_budget_bytes


def test_headroom_trims_then_reclaims_then_evicts():
    state = {"free": 2 * GiB, "cached": 1 * GiB}
    log = []

    def trim():
        state["free"] += state["cached"]
        state["cached"] = 0
        log.append("trim")

    va = VramAuthority(probe=lambda d: (state["free"], 80 * GiB), trim=trim, reserve_bytes=0)

    def pool(need):
        log.append("pool")
        state["free"] += 3 * GiB
        return 3 * GiB

    def arena(need):
        log.append("arena")
        state["free"] += 1 * GiB
        return 1 * GiB

    va.register("parked-kv-pool", pool, priority=1)
    va.register("capture-arena", arena, priority=0)
    models = ["old", "new"]

    def evict():
        if not models:
            return None
        state["free"] += 10 * GiB
        return models.pop(0)

    va.set_evictor(evict)
    r = va.ensure_headroom(2 * GiB)
    assert r.ok and not r.trimmed and not r.reclaimed and not r.evicted          # already there: nothing touched
    r = va.ensure_headroom(3 * GiB)
    assert r.ok and r.trimmed and not r.reclaimed and log == ["trim"]            # the allocator's cache first
    r = va.ensure_headroom(int(6.5 * GiB))
    assert r.ok and [n for n, _ in r.reclaimed] == ["capture-arena", "parked-kv-pool"] and not r.evicted
    e0 = va.residency_epoch
    r = va.ensure_headroom(20 * GiB)
    assert r.ok and r.evicted == ["old", "new"][:len(r.evicted)] and r.evicted[0] == "old"
    assert va.residency_epoch == e0 + len(r.evicted)
    r = va.ensure_headroom(500 * GiB)
    assert not r.ok and r.free_after < 500 * GiB
    with va.load_admission():
        assert not va._load_lock.acquire(blocking=False)


def test_host_budget_reads_meminfo_and_cgroup(tmp_path):
    mi = tmp_path / "meminfo"
    mi.write_text("MemTotal: 100 kB\nMemAvailable:   8000000 kB\n")
    assert host_budget_bytes(str(mi), cgroup_paths=(), cgroup_usage_paths=()) == int(8000000 * 1024 * 0.75)
    lim, use = tmp_path / "max", tmp_path / "cur"
    lim.write_text(str(4 << 30))
    use.write_text(str(1 << 30))
    assert host_budget_bytes(str(mi), (str(lim),), (str(use),)) == int((3 << 30) * 0.75)
    lim.write_text("max")
    assert host_budget_bytes(str(mi), (str(lim),), (str(use),)) == int(8000000 * 1024 * 0.75)


def test_sleeping_models(tmp_path):
    f = tmp_path / "m.gguf"
    f.write_bytes(b"GGUF" + os.urandom(3 << 20))
    big = tmp_path / "big.gguf"
    big.write_bytes(b"x" * (1 << 20))
    budget = [8 << 20]
    reg = SleepRegistry(budget=lambda: budget[0])
    m = reg.put_to_sleep("m", str(f), {"max_ctx": 4096})
    assert m is not None and m.host_bytes == f.stat().st_size and m.files == [str(f)] and reg.bytes_held() == m.host_bytes
    assert reg.put_to_sleep("shape-only", "llama-3.1-8b") is None            # nothing on disk to keep warm
    budget[0] = 1 << 19
    assert reg.put_to_sleep("big", str(big)) is None                          # does not fit the host budget: unloaded
    budget[0] = 8 << 20
    w = reg.wake("m")
    assert w is m and w.load_kwargs == {"max_ctx": 4096} and reg.wake("m") is None
    w.release()
    reg.put_to_sleep("a", str(f))
    reg.put_to_sleep("b", str(big))
    budget[0] = 0
    assert reg.make_room(1 << 20) == ["a"] and set(reg.sleeping) == {"b"}    # longest asleep goes first
    assert reg.drop("b") and not reg.drop("b")
    d = tmp_path / "ckpt"
    d.mkdir()
    for n in ("config.json", "model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors", "notes.md"):
        (d / n).write_text("{}")
    assert [os.path.basename(p) for p in model_files(str(d))] == ["config.json", "model-00001-of-00002.safetensors",
                                                                   "model-00002-of-00002.safetensors"]


def test_dry_demand_and_heap_replay():
    cfg = get_config("llama-3.3-70b")
    d1 = dry_demand(cfg, tp=1, max_seqs=64, max_ctx=1280, num_blocks=64 * 80 + 256)
    d8 = dry_demand(cfg, tp=8, max_seqs=64, max_ctx=1280, num_blocks=64 * 80 + 256)
    g1, g8 = d1.by_group(), d8.by_group()
    assert 68e9 < g1["weights"] < 76e9                      # 70.6 GB of e4m3 + scales + bf16 embeddings
    assert g8["weights"] < g1["weights"] / 4 and g8["kv"] * 8 == g1["kv"]
    assert "symmetric_heap" in g8 and "symmetric_heap" not in g1
    ok, d, heap = fits(cfg, 180 << 30, tp=1, max_seqs=64, max_ctx=1280, num_blocks=64 * 80 + 256)
    assert ok and heap.peak >= d.total and not heap.failed
    ok, _, heap = fits(cfg, 40 << 30, tp=1, max_seqs=64, max_ctx=1280)
    assert not ok and heap.failed
    moe = dry_demand(get_config("gpt-oss-120b"), tp=8, ep=8, max_seqs=128, max_ctx=2560)
    assert 6e9 < moe.by_group()["weights"] < 12e9           # 1/8 of 60 GB of MXFP4 experts + bf16 attention + embeddings
    # fragmentation: free the odd blocks of a full heap, the largest free run stays one block
    h = HeapReplay(64 << 20)
    for i in range(16):
        assert h.alloc(f"b{i}", 4 << 20)
    for i in range(1, 16, 2):
        h.free(f"b{i}")
    assert h.largest_free == 4 << 20 and abs(h.fragmentation() - 7 / 8) < 1e-9
    assert not h.alloc("big", 8 << 20) and h.alloc("fits", 3 << 20)
    assert HeapReplay.round(1) == 512 and HeapReplay.round((1 << 20) + 1) == 2 << 20


def test_give_way_is_one_rung_at_a_time():
    state = {"free": 0}
    va = VramAuthority(probe=lambda d: (state["free"], 80 * GiB), trim=lambda: None, reserve_bytes=0)
    models = ["a", "b"]
    va.set_evictor(lambda: models.pop(0) if models else None)
    r = va.give_way()
    assert r.evicted == ["a"] and models == ["b"] and va.residency_epoch == 1       # one model, not all of them
    va.register("pool", lambda need: 5)
    r = va.give_way()
    assert r.reclaimed == [("pool", 5)] and not r.evicted and models == ["b"]       # a reclaimer gave: nobody is unloaded
    va.unregister("pool")
    assert va.give_way().evicted == ["b"] and not va.give_way().evicted


def test_keep_alive_takes_an_idle_model_down_and_a_request_brings_it_back(tmp_path):
    """The reaper unloads a model nobody used for the keep-alive (files kept warm when they fit the host), and the
    next request that names it, or names nothing while it is the only one, loads it again with what it was loaded with."""
    from fastapi.testclient import TestClient

    from fakes import fake_llm
    from loken_b200.api.common import ModelRegistry
    from loken_b200.api.context import ServerSettings
    from loken_b200.api.server import create_app

    f = tmp_path / "m.gguf"
    f.write_bytes(b"x" * 4096)
    reg = ModelRegistry()
    llm = fake_llm(model_id="m1")
    llm.path, llm.load_kwargs = str(f), {"max_seqs": 8}
    reg.add(llm)
    app = create_app(reg, ServerSettings(keep_alive_s=60.0))
    ctx = app.state.ctx
    c = TestClient(app)
    loads = []

    def loader(path, model_id=None, **kw):
        loads.append((path, model_id, kw))
        m = fake_llm(model_id=model_id)
        m.path, m.load_kwargs = path, kw
        return m

    ctx.loader = loader
    assert c.post("/v1/completions", json={"model": "m1", "prompt": "x", "max_tokens": 2}).status_code == 200
    import time as _t

    now = _t.time()
    assert ctx.reap_idle(now + 30) == []                                      # used half a minute ago: stays
    assert ctx.reap_idle(now + 120) == ["m1"] and reg.list() == []
    assert ctx.asleep["m1"]["sleeping"] and ctx.sleepers.bytes_held() >= 4096   # its file stays read into host memory
    assert ctx.metrics.counters["models_put_to_sleep"] == 1
    r = c.post("/v1/completions", json={"model": "m1", "prompt": "x", "max_tokens": 2})
    assert r.status_code == 200 and loads == [(str(f), "m1", {"max_seqs": 8})]
    assert [m.model_id for m in reg.list()] == ["m1"] and ctx.sleepers.bytes_held() == 0 and ctx.asleep == {}
    # asleep again; a request that names nothing wakes the only model there is
    assert ctx.reap_idle(_t.time() + 120) == ["m1"]
    assert c.post("/v1/completions", json={"prompt": "x", "max_tokens": 2}).status_code == 200 and len(loads) == 2
    # -1 keeps a model for ever; a model with requests in flight is never taken down
    ctx.settings.keep_alive_s = -1
    assert ctx.reap_idle(_t.time() + 1e6) == []
    ctx.settings.keep_alive_s = 1.0
    reg.list()[0].worker.tickets[99] = object()
    assert ctx.reap_idle(_t.time() + 1e6) == []
    reg.list()[0].worker.tickets.pop(99)


def test_a_model_without_files_is_never_reaped():
    from fakes import fake_llm
    from loken_b200.api.common import ModelRegistry
    from loken_b200.api.context import ServerSettings
    from loken_b200.api.server import create_app

    reg = ModelRegistry()
    reg.add(fake_llm(model_id="shape"))                 # no path: random weights of a built-in shape
    ctx = create_app(reg, ServerSettings(keep_alive_s=1.0)).state.ctx
    import time as _t

    assert ctx.reap_idle(_t.time() + 1e6) == [] and [m.model_id for m in reg.list()] == ["shape"]
