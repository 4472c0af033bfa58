"""Context parallelism: the maths of parts (CPU), ranks holding ranges (gloo), and the decode kernel's parts
merged over two caches against the attention over one (GPU)."""
import os
import subprocess
import sys

import pytest
import torch

from loken_b200.parallel import context_parallel as cp


def test_ranges_cover_the_context_on_block_boundaries():
    for total, world in ((1000, 4), (33, 2), (16, 3), (5, 4), (4096, 8)):
        r = cp.plan_ranges(total, world)
        assert len(r) == world and r[0][0] == 0 and r[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all(lo % 16 == 0 for lo, _ in r if lo < total)
        sizes = [hi - lo for lo, hi in r]
        assert total < 16 * world or max(sizes) - min(sizes) < 32        # a block, plus the ragged end of the last range
    r = cp.plan_ranges(100, 3)
    assert cp.owner_of(0, r) == 0 and cp.owner_of(99, r) == 2 and cp.owner_of(100, r) == 2
    assert cp.owner_of(r[1][0], r) == 1


@pytest.mark.parametrize("n_q,n_kv", [(4, 4), (8, 2), (6, 2)])
@pytest.mark.parametrize("world", [1, 2, 5])
def test_parts_of_ranges_make_the_whole_attention(n_q, n_kv, world):
    from loken_b200.ops.attention import attention_ref

    torch.manual_seed(world + n_q)
    T, rows, hd = 150, 7, 16
    k, v = torch.randn(T, n_kv, hd), torch.randn(T, n_kv, hd)
    q = torch.randn(rows, n_q, hd)
    sinks = torch.randn(n_q)
    q_pos = 60                                         # rows at 60..66: later ranges are partly or wholly masked
    ranges = cp.plan_ranges(T, world)
    for sk in (None, sinks):
        got = cp.attention_over_ranges(q, k, v, ranges, hd ** -0.5, q_pos, sk)
        want = attention_ref(q, k[:q_pos + rows], v[:q_pos + rows], q_pos, scale=hd ** -0.5, sinks=sk).float()
        assert (got - want).abs().max().item() < 1e-5
    # merging is associative up to rounding: any order gives the same attention
    parts = [cp.partial(q, k[lo:hi], v[lo:hi], hd ** -0.5, q_pos, lo) for lo, hi in ranges]
    acc = None
    for p in reversed(parts):
        acc = cp.merge(acc, p)
    assert (cp.finish(acc) - cp.attention_over_ranges(q, k, v, ranges, hd ** -0.5, q_pos)).abs().max().item() < 1e-5
    # a range no row can see contributes nothing and makes no NaN
    empty = cp.partial(q, k[140:], v[140:], hd ** -0.5, q_pos, 140)
    assert torch.isinf(empty.max).all() and (empty.sum == 0).all() and torch.isfinite(cp.finish(cp.merge(acc, empty))).all()


def test_ranks_holding_ranges_agree_on_the_attention():
    worker = os.path.join(os.path.dirname(__file__), "mp_cp_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29633", worker]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "CP_OK 3" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize("hd,n_q,n_kv,q8", [(128, 8, 2, True), (64, 4, 4, False), (128, 10, 2, True)])
def test_decode_kernel_parts_of_two_caches_merge_into_one_attention(hd, n_q, n_kv, q8):
    """Two paged caches hold the two ranges of every sequence (as two ranks would); the decode kernel's parts,
    merged, equal the kernel's own attention over one cache that holds everything."""
    from loken_b200.ops import attention, rows

    dev = torch.device("cuda")
    torch.manual_seed(hd + n_q)
    bs, lens = 16, [1, 40, 300, 777]
    B = len(lens)
    cut = [cp.plan_ranges(L, 2)[0][1] for L in lens]             # positions [0, cut) on "rank 0", the rest on "rank 1"
    mb = (max(lens) + bs - 1) // bs
    caches = [rows.KVCacheLayer((B * mb + 2) * bs, n_kv, hd, dev, q8=q8) for _ in range(3)]   # rank 0, rank 1, whole
    bt = torch.arange(B * mb, device=dev, dtype=torch.int32).view(B, mb)
    inv = (10000.0 ** (-torch.arange(hd // 2, dtype=torch.float32) / (hd // 2))).to(dev)
    for s, L in enumerate(lens):
        kv = torch.randn(L, (1 + 2 * n_kv) * hd, device=dev).bfloat16()      # one dummy query head + k + v
        pos = torch.arange(L, device=dev, dtype=torch.int32)
        for which, (lo, hi) in ((0, (0, cut[s])), (1, (cut[s], L)), (2, (0, L))):
            if hi > lo:
                t = torch.arange(hi - lo, device=dev)
                slots = (bt[s, (t // bs).long()].long() * bs + t % bs).int()
                rows.rope_kv(kv[lo:hi].contiguous(), pos[lo:hi].contiguous(), slots, caches[which], 1, inv, pairing=1)
    q = torch.randn(B, n_q, hd, device=dev).bfloat16()
    sl = lambda xs: torch.tensor(xs, device=dev, dtype=torch.int32)
    whole = attention.decode(q, caches[2], bt, sl(lens), block_size=bs, nsplit=2).float()
    p0 = cp.decode_part(q, caches[0], bt, sl(cut), block_size=bs, nsplit=1)
    p1 = cp.decode_part(q, caches[1], bt, sl([L - c for L, c in zip(lens, cut)]), block_size=bs, nsplit=3)
    got = cp.finish(cp.merge(p0, p1))
    torch.cuda.synchronize()
    assert torch.isinf(p1.max[0]).all()                           # the one-token sequence has nothing on the second rank
    assert (got - whole).abs().max().item() < 2e-2 * whole.abs().max().item()      # bf16 rounding of the whole's output
