#!/usr/bin/env python
"""Headline benchmark: output tokens/s of batched decode on a Llama-3.3-70B-shaped model in
block-scaled fp8, tensor-parallel over N GPUs of one node (the third config of BASELINE.json).

    python bench.py --gpus 1 --steps 32 --warmup 4
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

A step is one decode step of the whole batch (every sequence emits one token) after a real
prefill of the prompts.  Two numbers come out of one run:
  value      K steps timed on the device (CUDA events), sampled token fed back on the device
  e2e.value  K steps through LLMEngine.step(): scheduler, pinned-host staging, H2D copy of the
             step's inputs, the captured decode graph, sampler, D2H copy of the new tokens
Weights are random-init N(0, 0.02) quantised to e4m3 with 128x128 block scales; prompts are
uniform random token ids.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "output tok/s (max over ranks) at 1/2/4/8 B200, 70B TP8 + gpt-oss EP8; p50 TTFT"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-3.3-70b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--comm", default="auto", choices=["auto", "sum_norm", "fused", "push", "nccl"],
                    help="tensor-parallel layer boundaries: sum_norm = one kernel over peer memory that does "
                         "reduce-scatter + residual + RMSNorm + quantise + all-gather with the residual stream "
                         "sharded by rows (the default); fused = all-reduce inside the GEMM epilogue; push = the "
                         "stand-alone peer-memory all-reduce kernel; nccl = the library baseline")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (marks the result invalid)")
    return ap.parse_args()


def reference_arm(args):
    # The reference is a Rust crate (Cargo.toml, build.rs, no setup.py / pyproject.toml): pip cannot
    # install it and there is no cargo / rustc in this image, so its own build cannot be run here.
    print(json.dumps({"impl": "reference", "metric": METRIC, "n_gpus": args.gpus,
                      "unavailable": "reference is a Rust crate: pip reports 'neither setup.py nor pyproject.toml "
                                     "found' and no cargo/rustc toolchain exists in this image"}))
    return 0


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while a region is timed."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, power, reasons = [], [], [], set()
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
                power.append(float(p[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            # under load = samples drawing real power; fall back to all of them
            load = [s for s, w in zip(sm, power) if w > 0.5 * max(power)] or sm
            load.sort()
            out.update(sm_mhz=load[len(load) // 2], sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       power_w_max=max(power))
        return out


# collectives per tensor-parallel degree, by measured ms/step on this benchmark
AUTO_COMM = {2: "sum_norm", 4: "sum_norm", 8: "sum_norm"}


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    import dataclasses

    import torch

    from loken_b200.models.config import get_config
    from loken_b200.parallel.comm import NcclComm, init_distributed
    from loken_b200.serve.engine import LLMEngine
    from loken_b200.utils import decode_bench

    # Libraries (NCCL's version banner among them) write to stdout; the contract is ONE JSON line
    # there, so everything but that line goes to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    rank, world, local = init_distributed()
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run",
                  file=sys.stderr)
        return 2
    dev = torch.device("cuda", local)
    cfg = get_config(args.model)
    if args.layers:
        cfg = dataclasses.replace(cfg, n_layers=args.layers)
    comm = None
    comm_name = "none"
    if world > 1:
        mode = args.comm
        if mode == "auto":
            mode = AUTO_COMM.get(world, "nccl")
        if mode in ("fused", "push", "sum_norm"):
            from loken_b200.parallel.symm import SymmComm

            comm = SymmComm(dev, max_rows=max(args.batch, 256), hidden=cfg.hidden)
            comm.fused_gemm = mode == "fused"
            comm.fused_norm = mode == "sum_norm"
            comm_name = {"fused": "GEMM-epilogue all-reduce over peer memory",
                         "push": "peer-memory all-reduce kernel",
                         "sum_norm": "one peer-memory kernel per layer boundary: reduce-scatter + residual + RMSNorm + "
                                     "e4m3 quantise + all-gather, residual stream sharded by rows"}[mode]
        else:
            comm = NcclComm()
            comm_name = "nccl"
    max_ctx = args.prompt_len + args.steps * 2 + args.warmup * 2 + 64
    max_ctx = (max_ctx + 255) // 256 * 256
    eng = LLMEngine(cfg, device=dev, tp_rank=rank, tp_size=world, comm=comm, max_seqs=max(args.batch, 1),
                    max_prefill_tokens=8192, max_ctx=max_ctx, seed=0,
                    num_blocks=args.batch * (max_ctx // 16) + 256, lookahead=0)
    sampler = ClockSampler(local) if rank == 0 else None
    r = decode_bench.run(eng, batch=args.batch, prompt_len=args.prompt_len, steps=args.steps, warmup=args.warmup,
                         world=world, rank=rank, clock_sampler=sampler)
    if rank == 0:
        base = None   # the reference publishes no number for this configuration
        line = {
            "metric": METRIC, "value": round(r["tok_s"], 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(r["device_ms"] / args.steps, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": base, "dtype": "fp8 (e4m3 block-scaled) weights+activations, bf16 residual/attention",
            "data": "synthetic: random-init N(0,0.02) weights, uniform random prompt token ids",
            "impl": "ours",
            "config": {"model": cfg.name + "-shaped" + (f" ({cfg.n_layers} layers, DEBUG)" if args.layers else ""),
                       "global_batch": args.batch, "seq_len": args.prompt_len, "context_at_timing": r["context_len"],
                       "parallelism": f"tp{world}", "tp_collectives": comm_name, "kv_cache": "q8 paged, block 16",
                       "sampling": "temperature 0.7 top-p 0.9 on device",
                       "l2": "inputs larger than L2: every step streams the rank's whole weight shard "
                             f"({cfg.param_count() / world / 1e9:.1f} GB) and the batch's KV cache",
                       "decode_graph": f"batch bucket {r['batch_padded']}, kv splits {r['nsplit']}"},
            "e2e": {"value": round(r["e2e_tok_s"], 2), "unit": "tok/s", "ms_per_step": round(r["e2e_ms"] / args.steps, 4),
                    "h2d_bytes_per_step": int(r["h2d_bytes_per_step"]), "d2h_bytes_per_step": int(r["d2h_bytes_per_step"]),
                    "gpu_launches": r["e2e_gpu_launches"]},
            "gpu_launches": r["gpu_launches"],
            "clocks": r["clocks"],
            "ttft_p50_s": round(r["ttft_p50_s"], 4), "prefill_s": round(r["prefill_s"], 4),
        }
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        import gc
        import torch.distributed as dist

        # Leave in step: drop the engine (its CUDA graphs hold captured collectives), wait for the
        # device, meet the other ranks, unmap peer memory.  The process group is not destroyed:
        # tearing NCCL down after graph capture has been seen to block, and the process is about to
        # exit anyway.
        import threading

        bail = threading.Timer(45.0, os._exit, [0])   # the result is printed; never hang on the way out
        bail.daemon = True
        bail.start()
        del eng
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        if hasattr(comm, "close"):
            comm.close()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
