"""Row-parallel projection + all-reduce, timed four ways on the ranks of one node:

    gemm          the fp8 GEMM alone (no sum: the floor)
    gemm+sum_norm GEMM, then the layer-boundary kernel: reduce-scatter + residual + RMSNorm + e4m3
                  quantise + all-gather (what the decoder runs by default; the others are followed by
                  the stand-alone add + RMSNorm + quantise kernel in "+norm" columns)
    gemm+push     GEMM, then this library's one-shot all-reduce kernel over peer memory
    gemm+nccl     GEMM, then ncclAllReduce
    fused         the GEMM whose epilogue pushes its tiles to the peers and sums them

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m loken_b200.utils.comm_bench --rows 64

Each variant is captured in a CUDA graph of `--inner` back-to-back calls and replayed; the time
is taken with CUDA events on the launching stream and reduced with MAX over the ranks.  Shapes
are the two row-parallel layers of a Llama-70B block at this tensor-parallel degree.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from ..ops import gemm, rows as row_ops
from ..ops._lib import Workspace
from ..parallel.comm import init_distributed
from ..parallel.symm import SymmComm


def _graph_time(fn, inner: int, reps: int) -> float:
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(inner):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) * 1e3 / (reps * inner)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--inter", type=int, default=28672)
    ap.add_argument("--inner", type=int, default=20)
    ap.add_argument("--reps", type=int, default=10)
    args = ap.parse_args()
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    comm = SymmComm(dev, max_rows=max(args.rows, 256), hidden=args.hidden)
    wsp = Workspace.get(dev)
    M, H = args.rows, args.hidden
    rows = []
    for name, K in (("o_proj", H // world), ("down_proj", args.inter // world)):
        torch.manual_seed(7 + rank)
        w = gemm.quantize_weight_fp8(torch.randn(H, K, device=dev) * 0.02)
        x = gemm.quantize_act_fp8_ref((torch.randn(M, K, device=dev)).bfloat16())
        res = torch.randn(M, H, device=dev).bfloat16()
        out = torch.empty(M, H, device=dev, dtype=torch.bfloat16)

        def plain():
            gemm.linear_fp8(x, w, out=out)

        def with_push():
            gemm.linear_fp8(x, w, out=out)
            comm.all_reduce(out, M, residual=res)

        def with_nccl():
            gemm.linear_fp8(x, w, out=out)
            comm.nccl.all_reduce(out, M)
            out.add_(res)

        def fused():
            gemm.linear_fp8(x, w, out=out, residual=res, symm=comm.heap)

        # what follows a row-parallel layer in the decoder: residual add + RMSNorm + e4m3 quantise
        xres = torch.randn(M, H, device=dev).bfloat16()
        wn = torch.ones(H, device=dev)
        h8 = row_ops.alloc_fp8_act(M, H, dev)

        def push_norm():
            gemm.linear_fp8(x, w, out=out)
            comm.all_reduce(out, M)
            row_ops.add_rmsnorm(xres, wn, 1e-5, delta=out, out_fp8=h8, rows=M)

        def nccl_norm():
            gemm.linear_fp8(x, w, out=out)
            comm.nccl.all_reduce(out, M)
            row_ops.add_rmsnorm(xres, wn, 1e-5, delta=out, out_fp8=h8, rows=M)

        def sum_norm():
            gemm.linear_fp8(x, w, out=out)
            comm.sum_norm(out, xres, wn, 1e-5, M, out_fp8=h8)

        def sum_norm_alone():
            comm.sum_norm(out, xres, wn, 1e-5, M, out_fp8=h8)

        # the fused result must be the sum the library computes
        with_nccl()
        ref = out.float().clone()
        fused()
        torch.cuda.synchronize()
        assert gemm.gemm_raw.last_fused, "the fused path was not taken"
        err = float(((out.float() - ref).abs().max() / ref.abs().max()).item())
        r = {"layer": name, "M": M, "N": H, "K": K, "rel_err_fused_vs_nccl": err}
        for key, fn in (("gemm", plain), ("gemm+push", with_push), ("gemm+nccl", with_nccl), ("fused", fused),
                        ("gemm+push+norm", push_norm), ("gemm+nccl+norm", nccl_norm), ("gemm+sum_norm", sum_norm),
                        ("sum_norm_alone", sum_norm_alone)):
            r[key + "_us"] = round(_graph_time(fn, args.inner, args.reps), 2)
        rows.append(r)
    status = wsp.read_status()
    if rank == 0:
        print(json.dumps({"world": world, "status": status, "cases": rows}))
    torch.cuda.synchronize()
    dist.barrier()
    comm.close()
    import os
    os._exit(0)


if __name__ == "__main__":
    main()
