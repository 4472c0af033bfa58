"""End-to-end: the engine's tokens and logits against the fp32 PyTorch oracle of the same model."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()


def _mk(arch, fmt, **kw):
    from loken_b200.models.config import tiny
    from loken_b200.models.weights import random_weights

    cfg = tiny(arch, weight_format=fmt, **kw)
    w = random_weights(cfg, torch.device(DEV), seed=1, std=0.05)
    return cfg, w


@pytest.mark.parametrize("arch,fmt,kw", [
    ("llama", "bf16", {}),
    ("llama", "fp8_block", dict(head_dim=128, n_q=4, n_kv=2, hidden=512, intermediate=1024)),
    ("qwen3", "bf16", dict(head_dim=128, n_q=8, n_kv=2)),
    ("gpt-oss", "bf16", {}),
    ("gpt-oss", "mxfp4", {}),
    ("llama", "q8_0", {}),
    ("llama", "q4_k_m", {}),
    # the q / k norm over all heads of a token, routing weights not renormalised
    ("olmoe", "bf16", dict(n_experts=8, top_k=2, expert_intermediate=128, n_q=4, n_kv=4, head_dim=64)),
    ("olmoe", "bf16", dict(n_experts=8, top_k=2, expert_intermediate=128, n_q=2, n_kv=2, head_dim=128)),
    # five query heads per kv head: prefill in the eight-slot tile shape, decode on the SIMT kernel
    ("qwen2", "bf16", dict(n_q=10, n_kv=2, head_dim=128, hidden=256)),
    # quantised mixture layers: decode steps run the attention half with fused fronts and the experts as GEMV slots
    ("olmoe", "q8_0", dict(n_experts=8, top_k=2, expert_intermediate=256, n_q=4, n_kv=4, head_dim=64)),
    ("qwen3moe", "q4_k_m", dict(n_experts=8, top_k=2, expert_intermediate=256, n_q=4, n_kv=2, head_dim=128, hidden=512)),
])
def test_prefill_logits_match_oracle(arch, fmt, kw):
    from loken_b200.models.reference import forward_ref
    from loken_b200.serve.engine import LLMEngine
    from loken_b200.serve.params import GREEDY

    cfg, w = _mk(arch, fmt, **kw)
    eng = LLMEngine(cfg, weights=w, num_blocks=64, max_seqs=8, max_prefill_tokens=512, max_ctx=512, use_graphs=False)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (45,), generator=g).tolist()
    ref = forward_ref(w, prompt)
    eng.add_request(prompt, GREEDY)
    eng.step()
    got = eng.runner.model.buf.logits[0].clone()
    sid = next(iter(eng.seqs))
    for _ in range(3):
        eng.step()                                   # decode steps: the single-row paths of every family
    assert eng.runner.wsp.read_status() == 0
    # the logits of the last decode step against the oracle over the prompt plus what was generated before it
    out_toks = list(eng.seqs[sid].output)
    ref_dec = forward_ref(w, prompt + out_toks[:-1])[-1]
    assert _cos(eng.runner.model.buf.logits[0], ref_dec) > (0.985 if fmt in ("fp8_block", "mxfp4") else 0.995)
    # e4m3 activations carry ~3% rounding per element into every product of the fp8 model, and into the
    # expert products of an MXFP4 model (block-scaled MMA: weights as stored, activations e4m3)
    assert _cos(got, ref[-1]) > (0.99 if fmt in ("fp8_block", "mxfp4") else 0.998)
    # the greedy token must agree wherever the oracle's lead over the runner-up is clear of the measured
    # noise (six times the rms difference: a difference of two elements has sqrt(2) of it)
    gap = torch.topk(ref[-1], 2).values
    noise = (got.float() - ref[-1].float().to(got.device)).pow(2).mean().sqrt()
    if (gap[0] - gap[1]) > max(0.05 * float(ref[-1].abs().max()), 6.0 * float(noise)):
        assert int(got.argmax()) == int(ref[-1].argmax())


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_decode_matches_oracle_and_batch_invariance(graphs):
    from loken_b200.models.reference import forward_ref
    from loken_b200.serve.engine import LLMEngine
    from loken_b200.serve.params import SamplingParams

    cfg, w = _mk("llama", "bf16", kv_format="bf16")
    sp = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, max_tokens=8)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (9, 33, 70)]
    eng = LLMEngine(cfg, weights=w, num_blocks=128, max_seqs=8, max_prefill_tokens=512, max_ctx=512,
                    use_graphs=graphs)
    batch = eng.generate(prompts, sp)
    # teacher-forced oracle: each generated token is the oracle's argmax unless the top-2 gap is tiny
    for r, p in zip(batch, prompts):
        seq = list(p)
        for t in r.output:
            ref = forward_ref(w, seq)[-1]
            top = torch.topk(ref, 2)
            if (top.values[0] - top.values[1]) > 0.02 * ref.abs().max():
                assert t == int(top.indices[0])
            seq.append(t)
    # a sequence decoded alone produces the same tokens as beside neighbours of other lengths
    eng2 = LLMEngine(cfg, weights=w, num_blocks=128, max_seqs=8, max_prefill_tokens=512, max_ctx=512,
                     use_graphs=graphs)
    for r, p in zip(batch, prompts):
        alone = eng2.generate([p], sp)[0]
        assert alone.output == r.output


def test_prefix_cache_chunked_prefill_and_preemption():
    from loken_b200.serve.engine import LLMEngine
    from loken_b200.serve.params import SamplingParams

    cfg, w = _mk("llama", "bf16")
    sp = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, max_tokens=6)
    g = torch.Generator().manual_seed(5)
    common = torch.randint(0, cfg.vocab, (64,), generator=g).tolist()
    tails = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (5, 17)]
    eng = LLMEngine(cfg, weights=w, num_blocks=64, max_seqs=4, max_prefill_tokens=32, max_ctx=256, use_graphs=False)
    a = eng.generate([common + tails[0]], sp)[0]          # chunked: 69 tokens through a 32-token budget
    b = eng.generate([common + tails[1]], sp)[0]
    assert a.cached_tokens == 0 and b.cached_tokens == 64
    eng2 = LLMEngine(cfg, weights=w, num_blocks=64, max_seqs=4, max_prefill_tokens=512, max_ctx=256,
                     use_graphs=False, enable_prefix_cache=False)
    b2 = eng2.generate([common + tails[1]], sp)[0]
    assert b2.cached_tokens == 0 and b2.output == b.output
    # a pool too small for all sequences at once: the newest is preempted and recomputed
    eng3 = LLMEngine(cfg, weights=w, num_blocks=14, max_seqs=4, max_prefill_tokens=512, max_ctx=256,
                     use_graphs=False, enable_prefix_cache=False)
    sp2 = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, max_tokens=40)
    ps = [torch.randint(0, cfg.vocab, (60,), generator=g).tolist() for _ in range(3)]
    rs = eng3.generate(ps, sp2)
    assert all(len(r.output) == 40 for r in rs)
    assert eng3.stats.preemptions > 0
    solo = [LLMEngine(cfg, weights=w, num_blocks=64, max_seqs=4, max_ctx=256, use_graphs=False)
            .generate([p], sp2)[0].output for p in ps[:1]]
    assert solo[0] == rs[0].output


def test_sampled_generation_is_reproducible_with_seed():
    from loken_b200.serve.engine import LLMEngine
    from loken_b200.serve.params import SamplingParams

    cfg, w = _mk("llama", "bf16")
    sp = SamplingParams(temperature=0.9, top_k=20, top_p=0.9, max_tokens=12, seed=1234, repeat_penalty=1.1)
    p = list(range(20))
    outs = []
    for _ in range(2):
        eng = LLMEngine(cfg, weights=w, num_blocks=32, max_seqs=4, max_ctx=256)
        outs.append(eng.generate([p], sp)[0].output)
    assert outs[0] == outs[1] and len(outs[0]) == 12


def test_embeddings_are_unit_vectors_and_leave_the_cache_clean():
    from loken_b200.serve.engine import LLMEngine

    cfg, w = _mk("llama", "bf16")
    eng = LLMEngine(cfg, weights=w, num_blocks=64, max_seqs=8, max_prefill_tokens=512, max_ctx=512, use_graphs=False)
    free0 = eng.alloc.free_blocks()
    a = eng.embed([5, 6, 7, 8, 9])
    b = eng.embed([5, 6, 7, 8, 9])
    c = eng.embed([9, 8, 7, 6, 5, 4, 3])
    m = eng.embed([5, 6, 7, 8, 9], pooling="mean")
    assert a.shape == (cfg.hidden,) and abs(float(a.norm()) - 1.0) < 1e-3
    assert torch.equal(a, b) and not torch.allclose(a, c) and not torch.allclose(a, m)
    assert eng.alloc.free_blocks() == free0
    assert eng.runner.wsp.read_status() == 0


def test_layer_perf_reports_every_layer():
    from loken_b200.serve.engine import LLMEngine

    cfg, w = _mk("llama", "bf16")
    eng = LLMEngine(cfg, weights=w, num_blocks=64, max_seqs=8, max_prefill_tokens=512, max_ctx=512, use_graphs=False)
    t = eng.layer_perf(4)
    assert [x["stage"] for x in t] == ["embed"] + [f"layer {i}" for i in range(cfg.n_layers)] + ["head"]
    assert all(x["ms"] > 0 for x in t)
    assert eng.runner.wsp.read_status() == 0


def test_beam_search_over_the_engine():
    """Beam width 1 is greedy decoding; wider beams come back best first and their cumulative
    log-probabilities are the oracle's, token by token."""
    from loken_b200.engine.llm import LLM, GenerationParams
    from loken_b200.models.reference import forward_ref
    from loken_b200.serve.beam import run_beam_search
    from loken_b200.serve.engine import LLMEngine
    from loken_b200.text.tokenizer import ByteTokenizer

    cfg, w = _mk("llama", "bf16", kv_format="bf16")
    eng = LLMEngine(cfg, weights=w, num_blocks=128, max_seqs=8, max_prefill_tokens=512, max_ctx=512)
    llm = LLM(eng, ByteTokenizer(cfg.vocab), "tiny")
    try:
        g = torch.Generator().manual_seed(11)
        prompt = torch.randint(0, cfg.vocab, (21,), generator=g).tolist()
        greedy = llm.generate(prompt, GenerationParams(max_tokens=5, temperature=0.0, ignore_eos=True))
        one = run_beam_search(llm, prompt, 1, 5, ignore_eos=True)
        assert one[0].tokens == greedy.token_ids
        beams = run_beam_search(llm, prompt, 3, 5, ignore_eos=True)
        assert len(beams) == 3 and all(len(b.tokens) == 5 for b in beams)
        assert all(beams[i].score >= beams[i + 1].score for i in range(2))
        assert beams[0].cum_logprob >= one[0].cum_logprob - 1e-3
        for b in beams:
            seq, cum = list(prompt), 0.0
            for t in b.tokens:
                cum += torch.log_softmax(forward_ref(w, seq)[-1].float(), dim=-1)[t].item()
                seq.append(t)
            assert abs(cum - b.cum_logprob) < 0.05 * max(1.0, abs(cum))
    finally:
        llm.close()



def test_disk_tier_restores_a_returning_prompt_after_a_restart(tmp_path):
    """A finished request leaves its full 256-token blocks in the directory; a new engine over the same directory
    starts the same prompt from them and decodes the same tokens."""
    from loken_b200.serve.engine import LLMEngine
    from loken_b200.serve.params import SamplingParams

    cfg, w = _mk("llama", "bf16")
    mk = lambda **kw: LLMEngine(cfg, weights=w, num_blocks=128, max_seqs=4, max_prefill_tokens=1024, max_ctx=1024, **kw)
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, cfg.vocab, (600,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, max_tokens=6, ignore_eos=True)
    a = mk(kv_disk_dir=str(tmp_path))
    first = a.generate([prompt], sp)[0]
    assert first.cached_tokens == 0 and a.disk.saved_blocks == 2
    b = mk(kv_disk_dir=str(tmp_path))                                     # "restart": an empty device cache
    again = b.generate([prompt], sp)[0]
    assert again.cached_tokens == 512 and b.disk.restored_tokens == 512
    assert again.output == first.output
    assert mk().generate([prompt], sp)[0].output == first.output          # and the same as an engine without the tier
    assert b.alloc.free_blocks() == 128


def test_kv_handover_between_two_engines():
    """Engine A reads the prompt and exports its cache; engine B imports it, finds the prompt in its
    prefix cache and decodes the tokens B would have produced on its own."""
    from loken_b200.serve.engine import LLMEngine
    from loken_b200.serve.params import SamplingParams

    cfg, w = _mk("llama", "bf16")
    mk = lambda: LLMEngine(cfg, weights=w, num_blocks=128, max_seqs=8, max_prefill_tokens=512, max_ctx=512)
    a, b, c = mk(), mk(), mk()
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (70,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, max_tokens=6, ignore_eos=True)
    # a request already running on A keeps all its tokens while A serves the export
    other = a.add_request(prompt[:20], sp)
    blob = a.export_prefix(prompt)
    got = []
    while a.has_work():
        for o in a.step():
            if o.seq_id == other:
                got += o.new_tokens
    assert len(got) == 6
    assert len(blob) > 70 * cfg.n_layers * cfg.n_kv * cfg.head_dim     # at least a byte per cached value
    assert b.import_prefix(blob) == 70
    cached, _ = b.alloc.match_prefix(prompt)
    assert len(cached) == 70 // 16                                       # every full block is published
    want = c.generate([prompt], sp)[0].output
    assert b.generate([prompt], sp)[0].output == want
    with pytest.raises(ValueError):
        b.import_prefix(b"not a container")


def test_adapters_swapped_in_place_under_captured_graphs():
    """An adapter attached to a running engine changes its tokens to those of a model merged at load, and a
    detach brings the original tokens back: the decode graphs captured before the swap read the rewritten
    weights through the same pointers."""
    from loken_b200.models.lora import AdapterSet, adapter_from_tensors, merge_lora
    from loken_b200.models.weights import random_weights
    from loken_b200.serve.engine import LLMEngine
    from loken_b200.serve.params import SamplingParams

    cfg, w = _mk("llama", "bf16")
    g = torch.Generator().manual_seed(11)
    t = {}
    for il in range(cfg.n_layers):
        for blk, proj, out, inn in (("self_attn", "q_proj", cfg.n_q * cfg.head_dim, cfg.hidden),
                                    ("mlp", "down_proj", cfg.hidden, cfg.intermediate)):
            base = f"base_model.model.model.layers.{il}.{blk}.{proj}"
            t[base + ".lora_A.weight"] = torch.randn(4, inn, generator=g) * 0.3
            t[base + ".lora_B.weight"] = torch.randn(out, 4, generator=g) * 0.3
    ad = adapter_from_tensors(t, 4, 8.0)
    merged = random_weights(cfg, torch.device(DEV), seed=1, std=0.05)
    merge_lora(merged, ad, 1.0)
    mk = lambda ww: LLMEngine(cfg, weights=ww, num_blocks=64, max_seqs=4, max_prefill_tokens=256, max_ctx=256)
    sp = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, max_tokens=12, ignore_eos=True)
    prompt = torch.randint(0, cfg.vocab, (20,), generator=g).tolist()
    eng = mk(w)
    plain = eng.generate([prompt], sp)[0].output                    # captures the decode graph over the base weights
    want = mk(merged).generate([prompt], sp)[0].output
    assert want != plain                                            # the adapter is strong enough to be seen
    s = AdapterSet(eng.weights)
    s.apply({"a": 1.0}, loader=lambda _p: ad)
    eng.reset_prefix_cache()
    assert eng.generate([prompt], sp)[0].output == want
    s.apply({}, loader=lambda _p: ad)
    eng.reset_prefix_cache()
    assert eng.generate([prompt], sp)[0].output == plain
