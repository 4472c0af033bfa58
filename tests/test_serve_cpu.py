"""Host-side serving logic without a GPU: block allocator + prefix cache, scheduler policy,
sampling-parameter bounds, draft-length learning, n-gram drafts."""
import pytest

from loken_b200.serve.kv_manager import PagedKvAllocator, block_hashes
from loken_b200.serve.params import GREEDY, ParamError, SamplingParams, openai_penalty
from loken_b200.serve.scheduler import Scheduler, Sequence


def test_prefix_cache_shares_full_blocks_only():
    a = PagedKvAllocator(16, 4)
    toks = list(range(10))
    assert a.allocate_with_prefix(1, toks) == 0
    a.commit_prefix(1, toks)
    # a second request with the same first 8 tokens reuses the two full blocks, not the partial one
    assert a.allocate_with_prefix(2, toks[:8] + [99, 98, 97]) == 8
    assert a.block_table(1)[:2] == a.block_table(2)[:2]
    assert a.block_table(1)[2] != a.block_table(2)[2]
    # a different salt never matches
    assert a.allocate_with_prefix(3, toks, salt=7) == 0
    # a full match keeps the last token to compute (something must produce logits)
    a.free(3)
    assert a.allocate_with_prefix(4, toks[:8]) in (4, 7, 8 - 4)


def test_evictable_blocks_count_as_free_and_are_reused():
    a = PagedKvAllocator(4, 4)
    toks = list(range(8))
    a.allocate_with_prefix(1, toks)
    a.commit_prefix(1, toks)
    a.free(1)
    assert a.free_blocks() == 4                 # cached but idle blocks are capacity
    assert a.allocate_with_prefix(2, toks + [1]) == 8
    a.free(2)
    # a request that needs everything evicts the idle cached blocks
    assert a.allocate_with_prefix(3, list(range(100, 116))) == 0
    assert a.free_blocks() == 0
    assert a.allocate_with_prefix(4, [1]) is None
    a.free(3)
    assert a.allocate_with_prefix(5, toks) == 0   # the old prefix is gone


def test_trim_append_and_hash_chain():
    a = PagedKvAllocator(8, 4)
    assert a.allocate(1, 6)
    assert a.length(1) == 6 and len(a.block_table(1)) == 2
    assert a.append(1, 3) and len(a.block_table(1)) == 3
    a.trim(1, 4)
    assert a.length(1) == 4 and len(a.block_table(1)) == 1
    assert a.slot(1, 3) == a.block_table(1)[0] * 4 + 3
    h1 = block_hashes(list(range(8)), 4)
    h2 = block_hashes([0, 1, 2, 3, 9, 9, 9, 9], 4)
    assert h1[0] == h2[0] and h1[1] != h2[1] and len(block_hashes(list(range(7)), 4)) == 1


def _seq(i, n, **kw):
    return Sequence(i, [1000 * (i + 1) + j for j in range(n)], SamplingParams(**kw))


def test_scheduler_admits_fcfs_under_token_budget_and_chunks_long_prompts():
    a = PagedKvAllocator(64, 4)
    s = Scheduler(a, max_running=8, max_prefill_tokens=10)
    s.add_request(_seq(0, 6))
    s.add_request(_seq(1, 6))
    s.add_request(_seq(2, 25))
    p = s.schedule()
    assert [(it.seq.seq_id, it.start, it.end) for it in p.prefills] == [(0, 0, 6)]      # 6 + 6 > 10
    s.on_step_done(p)
    s.seqs = None
    for q in [s.running[0]]:
        q.output.append(5)
    p = s.schedule()
    assert [q.seq_id for q in p.decodes] == [0]
    # the rest of the step's token budget goes to the first chunk of the long prompt
    assert [(it.seq.seq_id, it.start, it.end, it.is_last_chunk) for it in p.prefills] == \
        [(1, 0, 6, True), (2, 0, 4, False)]
    s.on_step_done(p)
    for q in s.running[:2]:
        q.output.append(5)
    p = s.schedule()
    assert sorted(q.seq_id for q in p.decodes) == [0, 1]
    assert [(it.seq.seq_id, it.start, it.end, it.is_last_chunk) for it in p.prefills] == [(2, 4, 14, False)]
    s.on_step_done(p)
    p = s.schedule()
    assert [(it.start, it.end, it.is_last_chunk) for it in p.prefills] == [(14, 24, False)]
    s.on_step_done(p)
    p = s.schedule()
    # one prompt token left: feeding it is an ordinary decode row
    assert p.prefills == [] and 2 in [q.seq_id for q in p.decodes]


def test_scheduler_preempts_newest_and_recomputes():
    a = PagedKvAllocator(4, 4, enable_prefix_cache=False)
    s = Scheduler(a, max_running=8, max_prefill_tokens=64)
    s.add_request(_seq(0, 8))
    s.add_request(_seq(1, 7))
    p = s.schedule()
    assert len(p.prefills) == 2
    s.on_step_done(p)
    for q in s.running:
        q.output.append(3)
    p = s.schedule()          # seq 0 needs a third block for its 9th token; none is free: the newest goes
    assert [q.seq_id for q in p.decodes] == [0]
    assert [q.seq_id for q in p.preempted] == [1]
    assert s.waiting[0].seq_id == 1 and s.waiting[0].computed == 0 and s.waiting[0].preemptions == 1
    s.on_step_done(p)
    s.finish(s.running[0], "stop")
    p = s.schedule()          # readmitted: prompt and generated token are recomputed
    assert (p.prefills[0].seq.seq_id, p.prefills[0].start, p.prefills[0].end) == (1, 0, 8)


def test_sampling_param_bounds_and_penalty_mapping():
    with pytest.raises(ParamError):
        SamplingParams(stop=["a"] * 5).validate()
    with pytest.raises(ParamError):
        SamplingParams(stop=["x" * 257]).validate()
    with pytest.raises(ParamError):
        SamplingParams(top_logprobs=21).validate()
    with pytest.raises(ParamError):
        SamplingParams(n=17).validate()
    with pytest.raises(ParamError):
        SamplingParams(max_tokens=131073).validate()
    assert SamplingParams(temperature=0.0).greedy and GREEDY.greedy
    assert openai_penalty(None, None) == 1.0
    assert openai_penalty(1.5, 1.5) == 3.0            # clamped to 2, mapped to 1 + pen
    assert openai_penalty(0.5, None, repetition=1.3) == 1.3
    assert openai_penalty(0.5, None, repetition=1.3, repeat=1.1) == 1.1
    a, b = SamplingParams(seed=4).rng(), SamplingParams(seed=4).rng()
    assert a.random() == b.random()


def test_prompt_lookup_and_draft_length():
    from loken_b200.serve.speculative import DraftLength, PromptLookupDrafter

    s = Sequence(0, [1, 2, 3, 4, 9, 9, 1, 2, 3, 4], GREEDY)
    assert PromptLookupDrafter().propose([s], 3) == [[9, 9, 1]]
    assert PromptLookupDrafter().propose([Sequence(1, [1, 2, 3], GREEDY)], 3) == [[]]
    dl = DraftLength()
    for _ in range(6):
        dl.observe(4, 4, 0.010)
    dl.observe_plain(0.008)
    assert dl.choose() >= 4
    bad = DraftLength()
    for _ in range(6):
        bad.observe(4, 0, 0.020)
    bad.observe_plain(0.008)
    assert bad.choose() == 0 and bad.holdoff == 48
    for _ in range(48):
        bad.observe_plain(0.008)
    assert bad.holdoff == 0
    assert DraftLength(fixed=4).choose() == 4


def test_request_that_can_never_fit_is_rejected_not_queued_for_ever():
    a = PagedKvAllocator(4, 16)
    s = Scheduler(a, max_running=8, max_prefill_tokens=512)
    big = Sequence(1, list(range(100)), GREEDY)      # needs 7 blocks of a 4-block pool
    s.add_request(big)
    assert big.state == "finished" and big.finish_reason == "error" and not s.has_work()
    # a sequence that outgrew the pool while it ran (preempted with its output) is dropped at readmission
    ok = Sequence(2, list(range(40)), GREEDY)
    s.add_request(ok)
    plan = s.schedule()
    assert [it.seq.seq_id for it in plan.prefills] == [2]
    s.on_step_done(plan)
    ok.output = list(range(30))
    s._preempt(ok)
    plan = s.schedule()
    assert plan.empty and plan.rejected == [ok] and ok.finish_reason == "error" and not s.has_work()
    # a prompt that fits the pool but not what is free now waits while something runs, and is
    # finished once nothing is left that could free a block
    a2 = PagedKvAllocator(4, 16)
    s2 = Scheduler(a2, max_running=8, max_prefill_tokens=512)
    assert a2.allocate(99, 40)                       # blocks held by somebody outside the scheduler
    waiting = Sequence(3, list(range(40)), GREEDY)
    s2.add_request(waiting)
    plan = s2.schedule()
    assert plan.empty and plan.rejected == [waiting] and not s2.has_work()


def test_handover_import_checks_the_container_before_it_allocates():
    import types

    import torch

    from loken_b200.cluster.handover import export_sequence, import_sequence
    from loken_b200.models.config import tiny
    from loken_b200.ops.rows import KVCacheLayer

    def engine(n_layers=2, name="a"):
        cfg = tiny("llama", n_layers=n_layers)
        cfg.name = name
        kv = [KVCacheLayer(8 * 16, 2, cfg.head_dim, "cpu", q8=True) for _ in range(n_layers)]
        runner = types.SimpleNamespace(cfg=cfg, kv=kv, device=torch.device("cpu"),
                                       w=types.SimpleNamespace(n_kv_local=2))
        return runner, PagedKvAllocator(8, 16)

    src, sa = engine()
    toks = list(range(40))
    assert sa.allocate(1, 40)
    for l in src.kv:
        l.k.random_(-100, 100)
        l.v.random_(-100, 100)
        l.k_scale.fill_(0.5)
        l.v_scale.fill_(0.25)
    blob = export_sequence(src, sa, 1, toks)
    dst, da = engine()
    assert import_sequence(dst, da, 5, blob) == 40
    s_src = torch.tensor(sa.slots_for_range(1, 0, 40))
    s_dst = torch.tensor(da.slots_for_range(5, 0, 40))
    assert torch.equal(dst.kv[1].k[s_dst], src.kv[1].k[s_src])
    da.free(5)
    free0 = da.free_blocks()
    # wrong layer count, another model, a short payload, a token list that does not match
    for bad_engine, bad_blob in ((engine(n_layers=3), blob), (engine(name="b"), blob), (engine(), blob[:-7]),
                                 (engine(), blob.replace(b'"n": 40', b'"n": 39'))):
        r, al = bad_engine
        f0 = al.free_blocks()
        with pytest.raises(ValueError):
            import_sequence(r, al, 9, bad_blob)
        assert al.free_blocks() == f0 and 9 not in al.seqs
    assert da.free_blocks() == free0
