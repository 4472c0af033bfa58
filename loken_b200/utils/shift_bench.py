"""What a context shift costs against the cold prefill it avoids.

    python -m loken_b200.utils.shift_bench --shape qwen3-8b --window 4096 --past 500

A sequence fills its window (`--window` cached positions of a random-init model of the shape, Q4_K_M), then
`LLMEngine.context_shift` drops `--past` positions behind the kept head: the survivors are copied into fresh
blocks and every key is turned back by that many positions (`lk_kv_shift`), layer by layer.  Printed: the
device time of that shift, of decoding on afterwards, and of the cold prefill of a window-sized prompt, which
is what a runtime without the shift pays when a conversation outgrows its window (the reference measures
the same pair: `docs/STATUS.md:101-106`, 1256 ms cold against 156 ms on its own card for this shape).
"""
from __future__ import annotations

import argparse
import dataclasses
import json

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="qwen3-8b")
    ap.add_argument("--weight-format", default="q4_k_m")
    ap.add_argument("--window", type=int, default=4096)
    ap.add_argument("--past", type=int, default=500)
    ap.add_argument("--keep", type=int, default=4)
    a = ap.parse_args(argv)
    from ..models.config import get_config
    from ..serve.engine import LLMEngine
    from ..serve.params import SamplingParams

    cfg = dataclasses.replace(get_config(a.shape), weight_format=a.weight_format)
    eng = LLMEngine(cfg, max_seqs=8, max_prefill_tokens=8192, max_ctx=a.window + 256,
                    num_blocks=3 * (a.window // 16) + 128, seed=0)
    g = torch.Generator().manual_seed(0)
    sp = SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True, context_shift=True, num_keep=a.keep)

    def timed(fn):
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        out = fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e), out

    def fill():
        sid = eng.add_request(torch.randint(0, cfg.vocab, (a.window - 1,), generator=g).tolist(), sp)
        while len(eng.seqs[sid].output) == 0:
            eng.step()
        return sid

    fill()                                             # warm-up: kernels loaded, buffers grown
    cold_ms, sid = timed(fill)
    eng.step()                                         # one decode step, so the sequence is decoding
    shift_ms, dropped = timed(lambda: eng.context_shift(sid, n_keep=a.keep, n_discard=a.past))
    step_ms, _ = timed(lambda: [eng.step() for _ in range(8)])
    print(json.dumps({"shape": cfg.name, "weight_format": cfg.weight_format, "window": a.window, "dropped": dropped,
                      "cold_prefill_ms": round(cold_ms, 2), "shift_ms": round(shift_ms, 2),
                      "decode_ms_per_step_after": round(step_ms / 8, 3),
                      "status": int(eng.runner.wsp.read_status()), "shifts": eng.stats.context_shifts}))


if __name__ == "__main__":
    main()
