"""Worker of tests/test_context_parallel.py: every gloo rank holds one range of a context, answers the same
queries with its part, and all ranks must end with the attention over the whole context."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from loken_b200.ops.attention import attention_ref          # noqa: E402
from loken_b200.parallel import context_parallel as cp      # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(5)                    # the same tensors on every rank
    T, rows, n_q, n_kv, hd = 83, 3, 6, 2, 32
    k = torch.randn(T, n_kv, hd, generator=g)
    v = torch.randn(T, n_kv, hd, generator=g)
    q = torch.randn(rows, n_q, hd, generator=g)
    sinks = torch.randn(n_q, generator=g)
    ranges = cp.plan_ranges(T, world)
    lo, hi = ranges[rank]
    q_pos = T - rows
    part = cp.partial(q, k[lo:hi], v[lo:hi], hd ** -0.5, q_pos, lo)
    for sk in (None, sinks):
        got = cp.gather_merge(part, sinks=sk)
        want = attention_ref(q, k, v, q_pos, scale=hd ** -0.5, sinks=sk)
        err = (got - want.float()).abs().max().item()
        assert err < 1e-5, (rank, err)
        all_out = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(all_out, got)
        assert all(torch.equal(all_out[0], o) for o in all_out)     # merged in rank order: the same bits everywhere
    if rank == 0:
        print("CP_OK", world, ranges)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
