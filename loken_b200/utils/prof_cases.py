"""Small fixed workloads for profiling one kernel at a time.

    python -m loken_b200.utils.prof_cases gemm_fp8 --m 64            # 57344 x 8192 block-fp8 GEMM, 3 launches
    python -m loken_b200.utils.prof_cases gemm_bf16 --m 64
    python -m loken_b200.utils.prof_cases gemm_q8_0 --m 64            # dequant-fused GEMM over GGUF blocks
    python -m loken_b200.utils.prof_cases decode_step --layers 4 --batch 64 --ctx 1024 [--tp 8]
    python -m loken_b200.utils.prof_cases attn_decode --batch 64 --ctx 1024
    python -m loken_b200.utils.prof_cases sampler --batch 64
    python -m loken_b200.utils.prof_cases attn_prefill --seqs 8 --ctx 2048
    python -m loken_b200.utils.prof_cases add_rmsnorm --batch 64      # also glu, rope_kv, embed
    python -m loken_b200.utils.prof_cases moe --batch 128 --fmt mxfp4
    python -m loken_b200.utils.prof_cases gemm_q4_k --m 1             # up to 8 rows: the dp4a GEMV
    python -m loken_b200.utils.prof_cases gemv_timeline --fmt q4_k --n 28672 --k 4096

Each case warms up, then runs the measured launches between cudaProfilerStart/Stop, so a
profiler started with `--profile-from-start off` sees only those.  Inputs are larger than the L2
cache; a case holds a few GB at most.  `--tp N` shapes the decode step like one rank of an N-way
tensor-parallel group (collectives left out).
"""
from __future__ import annotations

import argparse
import dataclasses

import torch


def _bracket(fn, n: int = 3):
    """Mean device time of `fn` in ms over n launches replayed from a CUDA graph (so host launch
    cost does not set a floor under short kernels); the replay sits between
    cudaProfilerStart/Stop."""
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(g):
        for _ in range(n):
            fn()
    g.replay()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    g.replay()
    e.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return s.elapsed_time(e) / n


def _bracket_eager(fn, n: int = 1):
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(n):
        fn()
    e.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return s.elapsed_time(e) / n


def gemm_case(kind: str, M: int, N: int, K: int, swap_max_m: int = -1, bn: int = 0, ksplits: int = 0):
    from ..ops import gemm, rows

    if swap_max_m >= 0:
        gemm.FP8_SWAP_MAX_M = swap_max_m
    gemm.FP8_BN_OVERRIDE = bn
    gemm.SPLIT_OVERRIDE = ksplits

    w = torch.randn(N, K, device="cuda") * 0.02
    x = torch.randn(M, K, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    if kind in ("q8_0", "q4_k", "q6_k", "mxfp4"):
        from ..ops import quant

        wq = quant.quantize_weight_torch(w, kind)        # encoded on the device: seconds, not minutes
        del w
        fn = lambda: quant.linear_gguf(x, wq, out=out)
        nbytes = wq.nbytes()
    elif kind == "fp8":
        wq = gemm.quantize_weight_fp8(w)
        del w
        xq = rows.quant_fp8(x)
        fn = lambda: gemm.linear_fp8(xq, wq, out=out)
        nbytes = N * K
    else:
        wb = w.bfloat16()
        del w
        fn = lambda: gemm.linear_bf16(x, wb, out=out)
        nbytes = 2 * N * K
    for _ in range(3):
        fn()
    ms = _bracket(fn)
    print(f"gemm_{kind} M={M} N={N} K={K}: {ms * 1e3:.1f} us/launch, {nbytes / ms / 1e6:.0f} GB/s weights, "
          f"{2 * M * N * K / ms / 1e9:.1f} TFLOP/s")


def gemm_sweep_case(M: int, shapes, variants):
    """Block-fp8 GEMMs of the given (N, K) shapes at M tokens, each under every variant
    "name[:max_m[:mt[:rem_mt[:splits]]]]" ("fold" = the per-K-block fold kernel; "mx" = the block-scaled MMA
    with its plan left to the cost model or forced).  Weights rotate through copies that together exceed
    the L2, so every launch streams from HBM; times are CUDA-graph replays."""
    from ..ops import gemm, rows

    for (N, K) in shapes:
        copies = max(2, (300 << 20) // (N * K) + 1)
        ws = [gemm.quantize_weight_fp8(torch.randn(N, K, device="cuda") * 0.02) for _ in range(copies)]
        x = torch.randn(M, K, device="cuda").bfloat16()
        xq = rows.quant_fp8(x)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ref = None
        for v in variants:
            f = v.split(":")
            nums = [int(t) for t in f[1:]] + [0] * 4
            gemm.SPLIT_OVERRIDE = nums[0] if f[0] == "fold" else 0        # "fold:S": S K-splits of every tile
            gemm.FP8_MX_MAX_M = 0 if f[0] == "fold" else (nums[0] or 1 << 20)
            gemm.FP8_MX_WIDE_MAX_M = gemm.FP8_MX_MAX_M
            gemm.FP8_MX_PLAN = (nums[1], nums[2], nums[3])
            for w in ws:                       # "mxt": the same weights read tile-major
                w.tiled = None
                if f[0] == "mxt":
                    w.tile_major()

            def fn():
                for w in ws:
                    gemm.linear_fp8(xq, w, out=out)

            for _ in range(2):
                fn()
            got = out.float().clone()
            if ref is None:
                ref = got
            err = ((got - ref).abs().max() / ref.abs().max()).item()
            ms = _bracket(fn, 2) / copies
            note = ""
            if f[0] != "fold":
                # one more launch with the kernel's own wait counters: median over the CTAs, in microseconds
                # at the clock the SM ran (clock64 counts SM cycles; 1.9 GHz assumed for the printout)
                prof = torch.zeros(296, 8, dtype=torch.int64, device="cuda")
                gemm.FP8_MX_PROF = prof
                gemm.linear_fp8(xq, ws[0], out=out)
                torch.cuda.synchronize()
                gemm.FP8_MX_PROF = None
                live = prof[:148][prof[:148, 4] > 0]
                ex = prof[148:][prof[:148, 4] > 0].float().median(dim=0).values / 1900.0
                med = live[:, :4].float().median(dim=0).values / 1900.0
                t0 = int(live[:, 4].min())
                loop_end = (live[:, 5] - t0).float() / 1e3
                epi_end = (live[:, 6] - t0).float() / 1e3
                mma_done = (live[:, 2] - t0).float() / 1e3
                accw = live[:, 7].float().median() / 1900.0
                note = (f"; epilogue: tensor-memory loads {ex[0]:.2f}, staging {ex[1]:.2f}, barrier {ex[2]:.2f}, global stores {ex[3]:.2f}, waits for accumulators {accw:.1f}; per CTA (us at 1.9 GHz): loop {med[3]:.1f}, MMA thread waits for operands {med[1]:.1f}, "
                        f"for an accumulator {med[2]:.1f}; producer waits for a free stage {med[0]:.1f}; global timer (us "
                        f"after the first CTA's start): last start {float((live[:, 4] - t0).max()) / 1e3:.1f}, last unit's MMAs issued "
                        f"{loop_end.median():.1f} median / {loop_end.max():.1f} last, completed {mma_done.median():.1f} / "
                        f"{mma_done.max():.1f}, epilogues end "
                        f"{epi_end.median():.1f} median / {epi_end.max():.1f} last")
            print(f"gemm_fp8 M={M} N={N} K={K} {v}: {ms * 1e3:.1f} us/launch, {N * K / ms / 1e6:.0f} GB/s weights, "
                  f"diff vs first variant {err:.2e}{note}")
        del ws


def decode_step_case(layers: int, batch: int, ctx: int, tp: int, model: str):
    from ..models.config import get_config
    from ..serve.engine import LLMEngine
    from ..serve.params import SamplingParams

    cfg = dataclasses.replace(get_config(model), n_layers=layers)
    eng = LLMEngine(cfg, tp_rank=0, tp_size=tp, max_seqs=batch, max_prefill_tokens=8192, max_ctx=ctx + 256,
                    num_blocks=batch * ((ctx + 256) // 16) + 64, use_graphs=False)
    g = torch.Generator().manual_seed(0)
    sp = SamplingParams(temperature=0.7, top_k=0, top_p=0.9, ignore_eos=True, seed=1)
    ids = [eng.add_request(torch.randint(0, cfg.vocab, (ctx,), generator=g).tolist(), sp) for _ in range(batch)]
    while any(len(eng.seqs[i].output) == 0 for i in ids):
        eng.step()
    for _ in range(2):
        eng.step()
    ms = _bracket_eager(eng.step, 1)
    print(f"decode_step {model} layers={layers} batch={batch} ctx={ctx} tp={tp}: {ms:.3f} ms (eager, host included)")


def attn_decode_case(batch: int, ctx: int, n_q: int, n_kv: int, splits: int = 0):
    from ..ops import attention, rows

    hd, bs = 128, 16
    nb = (ctx + bs - 1) // bs
    cache = rows.KVCacheLayer(batch * nb * bs, n_kv, hd, "cuda", q8=True)
    cache.k.copy_(torch.randint(-127, 128, cache.k.shape, device="cuda").to(torch.int8))
    cache.v.copy_(torch.randint(-127, 128, cache.v.shape, device="cuda").to(torch.int8))
    cache.k_scale.fill_(0.01)
    cache.v_scale.fill_(0.01)
    bt = torch.arange(batch * nb, device="cuda", dtype=torch.int32).view(batch, nb)
    q = torch.randn(batch, n_q, hd, device="cuda").bfloat16()
    lens = torch.full((batch,), ctx, device="cuda", dtype=torch.int32)
    ns = splits or attention.pick_decode_splits(batch, n_kv, ctx)
    fn = lambda: attention.decode(q, cache, bt, lens, block_size=bs, nsplit=ns)
    for _ in range(3):
        fn()
    ms = _bracket(fn)
    nbytes = batch * ctx * n_kv * (hd + hd // 16) * 2
    print(f"attn_decode batch={batch} ctx={ctx} n_q={n_q} n_kv={n_kv} splits={ns}: {ms * 1e3:.1f} us, "
          f"{nbytes / ms / 1e6:.0f} GB/s of KV")


def sampler_case(batch: int, vocab: int):
    from ..ops import sampling

    logits = torch.randn(batch, vocab, device="cuda")
    t = torch.full((batch,), 0.7, device="cuda")
    u = torch.rand(batch, device="cuda")
    tk = torch.zeros(batch, dtype=torch.int32, device="cuda")
    tp = torch.full((batch,), 0.9, device="cuda")
    mp = torch.zeros(batch, device="cuda")
    fn = lambda: sampling.sample(logits, t, u, top_k=tk, top_p=tp, min_p=mp)
    for _ in range(3):
        fn()
    ms = _bracket(fn)
    print(f"sampler batch={batch} vocab={vocab}: {ms * 1e3:.1f} us, {batch * vocab * 4 / ms / 1e6:.0f} GB/s of logits")


def gemv_timeline_case(fmt: str, N: int, K: int):
    """Six back-to-back one-row GEMVs over six copies of a GGUF matrix (launched eagerly with programmatic
    dependent launch, as in a decode step) with the streaming kernel's own time stamps: when each CTA entered,
    when its wait for the kernel before ended, when the activations were staged, when the first stage of
    weights had landed, when it finished, and when its producer issued the first and the last copy.  Printed
    for the last two launches as min..max over CTAs, in us from the first entry."""
    from ..ops import quant

    dev = torch.device("cuda")
    ws = [quant.quantize_weight_torch(torch.randn(N, K, device=dev) * 0.05, fmt) for _ in range(6)]
    x = (torch.randn(1, K, device=dev) * 0.5).bfloat16()
    out = torch.empty(1, N, dtype=torch.bfloat16, device=dev)
    profs = [torch.zeros(300, 8, dtype=torch.int64, device=dev) for _ in range(2)]
    torch.cuda.profiler.start()
    for _ in range(3):
        for i in range(6):
            quant.linear_gguf(x, ws[i], out=out, front=quant.GemvFront(prof=profs[i % 2]))
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    a, b = profs[0].cpu(), profs[1].cpu()
    a, b = a[a[:, 0] > 0], b[b[:, 0] > 0]
    if len(a) == 0:
        print(f"gemv_timeline {fmt} {N}x{K}: the streaming form did not take this shape")
        return
    t0 = int(a[:, 0].min())
    names = ("entry", "wait ended", "staged", "first stage", "end", "first copy", "last copy")
    print(f"gemv_timeline {fmt} {N}x{K}: {len(a)} CTAs, {ws[0].nbytes() / 1e6:.1f} MB")
    for label, t in (("launch 5", a), ("launch 6", b)):
        cols = [((t[:, i] - t0).float() / 1000) for i in range(7)]
        print(f"  {label}: " + "  ".join(f"{n} {c.min():.1f}..{c.max():.1f}" for n, c in zip(names, cols)) + " us")


def attn_prefill_case(n_seqs: int, ctx: int, n_q: int, n_kv: int):
    """Variable-length flash prefill over keys gathered from the q8 paged cache (kv_gather +
    attn_prefill_kernel), `n_seqs` prompts of `ctx` tokens."""
    from ..ops import attention, rows

    hd, bs = 128, 16
    nb = (ctx + bs - 1) // bs
    cache = rows.KVCacheLayer(n_seqs * nb * bs, n_kv, hd, "cuda", q8=True)
    cache.k.copy_(torch.randint(-127, 128, cache.k.shape, device="cuda").to(torch.int8))
    cache.v.copy_(torch.randint(-127, 128, cache.v.shape, device="cuda").to(torch.int8))
    cache.k_scale.fill_(0.01)
    cache.v_scale.fill_(0.01)
    bt = torch.arange(n_seqs * nb, device="cuda", dtype=torch.int32).view(n_seqs, nb)
    plan = attention.plan_prefill([ctx] * n_seqs, [ctx] * n_seqs, n_q // n_kv, "cuda")
    q = torch.randn(n_seqs * ctx, n_q, hd, device="cuda").bfloat16()
    out = torch.empty(n_seqs * ctx, n_q * hd, device="cuda", dtype=torch.bfloat16)
    kbuf, vtbuf = attention.kv_gather(cache, bt, plan, bs)

    def fn():
        attention.kv_gather(cache, bt, plan, bs, kbuf, vtbuf)
        attention.prefill(q, kbuf, vtbuf, plan, out=out)

    for _ in range(3):
        fn()
    ms = _bracket(fn)
    flops = 4.0 * n_seqs * n_q * hd * ctx * ctx / 2
    print(f"attn_prefill seqs={n_seqs} ctx={ctx} n_q={n_q} n_kv={n_kv}: {ms * 1e3:.1f} us (gather + attention), "
          f"{flops / ms / 1e9:.1f} TFLOP/s causal")


def rows_case(which: str, T: int, H: int, I: int):
    """The row kernels of a decode step at `T` rows: add_rmsnorm (+ e4m3 quantise), glu (+ quantise),
    rope_kv (q/k norm + RoPE + q8 paged KV write), embed.  Buffers rotate through more than the L2."""
    from ..ops import rows

    nrot = max(1, (160 << 20) // max(1, T * max(H, 2 * I) * 2))
    if which == "add_rmsnorm":
        xs = [torch.randn(T, H, device="cuda").bfloat16() for _ in range(nrot)]
        d = torch.randn(T, H, device="cuda").bfloat16()
        w = torch.ones(H, device="cuda")
        o8 = rows.alloc_fp8_act(T, H, "cuda")
        it = [0]

        def fn():
            it[0] = (it[0] + 1) % nrot
            rows.add_rmsnorm(xs[it[0]], w, 1e-5, delta=d, out_fp8=o8, rows=T)
        nbytes = T * H * (2 + 2 + 2 + 1)
    elif which == "glu":
        gs = [torch.randn(T, 2 * I, device="cuda").bfloat16() for _ in range(nrot)]
        o8 = rows.alloc_fp8_act(T, I, "cuda")
        it = [0]

        def fn():
            it[0] = (it[0] + 1) % nrot
            rows.glu(gs[it[0]], out_fp8=o8, rows=T)
        nbytes = T * I * (4 + 1)
    elif which == "rope_kv":
        n_q, n_kv, hd = 64, 8, 128
        qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, device="cuda").bfloat16()
        cache = rows.KVCacheLayer(T * 64, n_kv, hd, "cuda", q8=True)
        pos = torch.arange(T, device="cuda", dtype=torch.int32)
        slots = (torch.arange(T, device="cuda", dtype=torch.int32) * 61) % (T * 64)
        inv = 1.0 / (5e5 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
        qo = torch.empty(T, n_q, hd, device="cuda", dtype=torch.bfloat16)
        fn = lambda: rows.rope_kv(qkv, pos, slots, cache, n_q, inv, pairing=0, q_out=qo, rows=T)
        nbytes = T * (n_q + 2 * n_kv) * hd * 2 + T * n_q * hd * 2 + T * 2 * n_kv * hd
    else:
        V = 128256
        table = torch.randn(V, H, device="cuda").bfloat16()
        tok = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
        out = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
        fn = lambda: rows.embed(tok, table, out=out)
        nbytes = T * H * 4
    for _ in range(3):
        fn()
    ms = _bracket(fn)
    print(f"{which} T={T} H={H} I={I}: {ms * 1e3:.2f} us, {nbytes / ms / 1e6:.0f} GB/s")


def moe_case(T: int, fmt: str, experts: int, top_k: int, H: int, I: int):
    """One gpt-oss-shaped mixture layer on one GPU: router GEMM, lk_moe_route, lk_moe_plan,
    lk_moe_permute, grouped gate_up GEMM, clamped GLU, grouped down GEMM, lk_moe_combine."""
    from ..models.config import get_config
    from ..models.moe import MoeRunner, random_moe

    cfg = dataclasses.replace(get_config("gpt-oss-120b"), n_experts=experts, top_k=top_k, hidden=H,
                              expert_intermediate=I, weight_format=fmt, n_layers=1)
    gen = torch.Generator(device="cuda").manual_seed(0)
    moe = random_moe(cfg, gen, "cuda", 0.02)

    class _W:
        pass
    w = _W()
    w.embed = torch.zeros(1, device="cuda")
    lay = _W()
    lay.moe = moe
    w.layers = [lay]
    run = MoeRunner(cfg, w, T)
    h = torch.randn(T, H, device="cuda").bfloat16()
    out = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    fn = lambda: run.forward(0, moe, h, out, T)
    for _ in range(3):
        fn()
    ms = _bracket(fn)
    wb = (moe.gate_up.nbytes() + moe.down.nbytes()) if fmt != "bf16" else (moe.gate_up.numel() + moe.down.numel()) * 2
    print(f"moe T={T} fmt={fmt} experts={experts} top_k={top_k} H={H} I={I}: {ms * 1e3:.1f} us per layer, "
          f"expert weights {wb / 1e6:.0f} MB ({wb / ms / 1e6:.0f} GB/s if all were read)")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm_sweep", "gemm_fp8", "gemm_bf16", "gemm_q8_0", "gemm_q4_k", "gemm_q6_k", "gemm_mxfp4",
                                    "decode_step", "attn_decode", "sampler", "attn_prefill", "add_rmsnorm", "glu",
                                    "rope_kv", "embed", "moe", "gemv_timeline"])
    ap.add_argument("--m", type=int, default=64)
    ap.add_argument("--n", type=int, default=57344)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--model", default="llama-3.3-70b")
    ap.add_argument("--n-q", type=int, default=64)
    ap.add_argument("--n-kv", type=int, default=8)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--seqs", type=int, default=8, help="attn_prefill: number of prompts")
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--inter", type=int, default=28672)
    ap.add_argument("--fmt", default="mxfp4", help="moe: expert weight format (mxfp4 | bf16 | q8_0 | q4_k)")
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--swap-max-m", type=int, default=-1, help="fp8 GEMM: largest M run with weights on the MMA M side")
    ap.add_argument("--gemm-splits", type=int, default=0, help="K splits of a GEMM with fewer tiles than SMs (0 = the library's choice)")
    ap.add_argument("--bn", type=int, default=0, help="fp8 GEMM: N-tile width of the tokens-on-M form (0 = the library's choice)")
    ap.add_argument("--splits", type=int, default=0, help="kv splits of the decode kernel (0 = the library's choice)")
    ap.add_argument("--shapes", default="57344x8192,8192x28672,10240x8192,8192x8192", help="gemm_sweep: N x K list")
    ap.add_argument("--variants", default="fold,mx", help="gemm_sweep: name[:max_m[:mt[:rem_mt[:splits]]]] list")
    a = ap.parse_args(argv)
    if a.case == "gemm_sweep":
        gemm_sweep_case(a.m, [tuple(int(t) for t in sh.split("x")) for sh in a.shapes.split(",")], a.variants.split(","))
    elif a.case == "gemv_timeline":
        gemv_timeline_case(a.fmt if a.fmt != "mxfp4" else "q4_k", a.n, a.k)
    elif a.case.startswith("gemm_"):
        gemm_case(a.case[5:], a.m, a.n, a.k, a.swap_max_m, a.bn, a.gemm_splits)
    elif a.case == "decode_step":
        decode_step_case(a.layers, a.batch, a.ctx, a.tp, a.model)
    elif a.case == "attn_decode":
        attn_decode_case(a.batch, a.ctx, a.n_q, a.n_kv, a.splits)
    elif a.case == "attn_prefill":
        attn_prefill_case(a.seqs, a.ctx, a.n_q, a.n_kv)
    elif a.case in ("add_rmsnorm", "glu", "rope_kv", "embed"):
        rows_case(a.case, a.batch, a.hidden, a.inter)
    elif a.case == "moe":
        moe_case(a.batch, a.fmt, a.experts, a.top_k, a.hidden if a.hidden != 8192 else 2880,
                 a.inter if a.inter != 28672 else 2880)
    else:
        sampler_case(a.batch, a.vocab)


if __name__ == "__main__":
    main()
