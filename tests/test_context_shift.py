"""Context shift: the allocator's bookkeeping (CPU), the key re-phasing kernel against an fp32
reference, and a generation that runs past its window (GPU)."""
import math

import pytest
import torch

from loken_b200.serve.kv_manager import PagedKvAllocator
from loken_b200.serve.params import SamplingParams
from loken_b200.serve.scheduler import Sequence


def test_allocator_shift_keeps_whole_head_blocks_and_moves_the_rest_into_fresh_ones():
    a = PagedKvAllocator(16, block_size=4)
    toks = list(range(100, 122))                      # 22 tokens -> 6 blocks
    assert a.allocate_with_prefix(1, toks) is not None
    a.commit_prefix(1, toks)
    old = list(a.block_table(1))
    src, dst, delta = a.shift(1, n_keep=5, n_discard=8)
    new = a.block_table(1)
    assert a.length(1) == 14 and new[0] == old[0]     # the whole block inside the kept head stays (it is published)
    assert set(new[1:]).isdisjoint(old)               # the copy never lands on its own source
    # positions 4 (kept, moves only) and 5.. (came from 13..): slots and turns
    assert len(src) == 10 and delta == [0] + [-8] * 9
    assert src[0] == old[1] * 4 + 0 and dst[0] == new[1] * 4 + 0
    assert src[1] == old[3] * 4 + 1 and dst[1] == new[1] * 4 + 1     # old position 13 -> new position 5
    # blocks past the kept head are never published again
    a.commit_prefix(1, toks[:5] + toks[13:] + [1, 2, 3, 4, 5, 6])
    assert len(a.seqs[1].hashes) <= 1
    free_before = a.free_blocks()
    a.free(1)
    assert a.free_blocks() == free_before + len(new)


def test_allocator_shift_refuses_without_room():
    a = PagedKvAllocator(4, block_size=4)
    assert a.allocate(1, 16)
    assert a.shift(1, 1, 4) is None and a.length(1) == 16


def test_sequence_positions_follow_the_cache_while_prompt_and_output_stay_whole():
    s = Sequence(1, [1, 2, 3, 4, 5, 6], SamplingParams(), output=[7, 8, 9])
    assert s.tokens == [1, 2, 3, 4, 5, 6, 7, 8, 9] and s.total_len == 9
    s.drop_positions(2, 3)
    assert s.tokens == [1, 2, 6, 7, 8, 9] and s.total_len == 6
    s.output.append(10)
    assert s.tokens == [1, 2, 6, 7, 8, 9, 10] and s.total_len == 7
    assert s.prompt == [1, 2, 3, 4, 5, 6] and s.output == [7, 8, 9, 10] and s.shifts == 1
    s.drop_positions(1, 2)
    assert s.tokens == [1, 7, 8, 9, 10]


def _rope(x, pos, inv_freq, pairing):
    hd = x.shape[-1]
    ang = pos[:, None, None].double() * inv_freq[None, None].double()
    c, s = ang.cos(), ang.sin()
    x = x.double()
    if pairing == 1:
        a, b = x[..., :hd // 2], x[..., hd // 2:]
        return torch.cat([a * c - b * s, a * s + b * c], -1)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2)


@pytest.mark.gpu
@pytest.mark.parametrize("q8", [True, False])
@pytest.mark.parametrize("pairing", [0, 1])
def test_kv_shift_kernel_rephases_keys_and_copies_values(q8, pairing):
    from loken_b200.ops import rows

    dev = torch.device("cuda")
    torch.manual_seed(1)
    hd, n_kv, slots, n = 128, 2, 96, 40
    inv_freq = (10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) / (hd // 2))).float().to(dev)
    cache = rows.KVCacheLayer(slots, n_kv, hd, dev, q8=q8)
    k0 = torch.randn(n, n_kv, hd, device=dev)
    v0 = torch.randn(n, n_kv, hd, device=dev)
    pos = torch.arange(100, 100 + n, device=dev)
    # write keys rotated at their positions through the production kernel
    qkv = torch.cat([torch.zeros(n, 1, hd, device=dev), k0, v0], 1).reshape(n, -1).bfloat16()
    src_slots = torch.arange(0, n, device=dev, dtype=torch.int32)
    rows.rope_kv(qkv, pos.int(), src_slots, cache, 1, inv_freq, pairing=pairing)
    dst_slots = torch.arange(48, 48 + n, device=dev, dtype=torch.int32)
    delta = torch.full((n,), -37, device=dev, dtype=torch.int32)
    delta[:5] = 0
    rows.kv_shift(cache, src_slots, dst_slots, delta, inv_freq, pairing=pairing)
    torch.cuda.synchronize()
    k_new, v_new = cache.dequant_rows(dst_slots.long()) if hasattr(cache, "dequant_rows") else _deq(cache, dst_slots, q8)
    want_k = _rope(k0.bfloat16().float().cpu(), (pos.cpu() + delta.cpu()), inv_freq.cpu(), pairing)
    err = (k_new.double().cpu() - want_k).abs().max() / want_k.abs().max()
    assert err < (0.03 if q8 else 0.012), err        # two int8 roundings (write, re-phase) / two bf16 roundings
    k_old, v_old = _deq(cache, src_slots, q8)
    assert torch.equal(v_new, v_old)                 # values are copied as stored
    assert torch.equal(_deq(cache, dst_slots[:5], q8)[0], k_old[:5]) or not q8      # delta 0: the key only moves


def _deq(cache, slots, q8):
    i = slots.long()
    if not q8:
        return cache.k[i].float(), cache.v[i].float()
    hd = cache.hd
    ks = cache.k_scale[i].float().repeat_interleave(32, dim=-1).view(len(i), cache.n_kv, hd)
    vs = cache.v_scale[i].float().repeat_interleave(32, dim=-1).view(len(i), cache.n_kv, hd)
    return cache.k[i].float().view(len(i), cache.n_kv, hd) * ks, cache.v[i].float().view(len(i), cache.n_kv, hd) * vs


@pytest.mark.gpu
def test_generation_runs_past_its_window_by_shifting():
    from loken_b200.models.config import tiny
    from loken_b200.models.weights import random_weights
    from loken_b200.serve.engine import LLMEngine

    dev = torch.device("cuda")
    cfg = tiny("llama", head_dim=64, n_q=4, n_kv=2, n_layers=2)
    w = random_weights(cfg, dev, seed=0, std=0.05)
    eng = LLMEngine(cfg, weights=w, device=dev, num_blocks=64, max_seqs=4, max_prefill_tokens=256, max_ctx=64,
                    use_graphs=False)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=120, ignore_eos=True, context_shift=True, num_keep=4)
    sid = eng.add_request(prompt, sp)
    plain = eng.add_request(prompt, SamplingParams(temperature=0.0, max_tokens=120, ignore_eos=True))
    while eng.has_work():
        eng.step()
    s, p = eng.seqs[sid], eng.seqs[plain]
    assert len(s.output) == 120 and s.finish_reason == "length" and s.shifts >= 2     # three windows' worth of text
    assert len(p.output) < 30 and p.finish_reason == "length"                         # the window ended it
    assert s.output[:len(p.output) - 1] == p.output[:len(p.output) - 1]               # identical until the first shift
    assert s.total_len <= 64 and eng.stats.context_shifts == s.shifts
    assert eng.runner.wsp.read_status() == 0
    # the shifted cache is what a decode step reads: the next token after a shift matches a forward over the
    # re-phased cache being coherent -> the logits stay finite and the model keeps producing valid ids
    assert all(0 <= t < cfg.vocab for t in s.output)
