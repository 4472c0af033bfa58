"""Where a decode step's time goes, layer by layer, for a model shape at several batch sizes.

    python -m loken_b200.utils.layer_bench --model llama-3.3-70b --layers 4 --batch 1,8,64 --ctx 1024

Builds the engine with the first `--layers` layers of the shape (random-init weights), reads `--ctx`
prompt tokens per sequence so the cache is as long as in service, then times the embedding, every
layer and the head with CUDA events (`DecoderModel.profile_layers`, the same pass `GET /api/layer_perf`
runs) and prints one JSON line per batch size: the stages, the mean layer, and the step this predicts
for the whole model.  The reference's counterpart is its layer bench (`benches/` and `/api/layer_perf`).
"""
from __future__ import annotations

import argparse
import dataclasses
import json

import torch


def layer_times(model: str, layers: int, batch: int, ctx: int, weight_format=None) -> dict:
    from ..models.config import get_config
    from ..serve.engine import LLMEngine
    from ..serve.params import SamplingParams

    full = get_config(model)
    cfg = dataclasses.replace(full, n_layers=min(layers, full.n_layers))
    if weight_format:
        cfg = dataclasses.replace(cfg, weight_format=weight_format)
    eng = LLMEngine(cfg, max_seqs=max(batch, 8), max_prefill_tokens=8192, max_ctx=ctx + 256,
                    num_blocks=batch * ((ctx + 256) // 16) + 64, use_graphs=False)
    g = torch.Generator().manual_seed(0)
    sp = SamplingParams(temperature=0.7, top_k=0, top_p=0.9, ignore_eos=True, seed=1, max_tokens=4096)
    ids = [eng.add_request(torch.randint(0, cfg.vocab, (ctx,), generator=g).tolist(), sp) for _ in range(batch)]
    while any(len(eng.seqs[i].output) == 0 for i in ids):
        eng.step()
    # one decode step's inputs, staged the way the runner stages them, then the profiling pass over them
    r = eng.runner
    seqs = [eng.seqs[i] for i in ids]
    for s in seqs:                            # the slot of the token a decode step would write
        short = s.total_len - eng.alloc.length(s.seq_id)
        if short > 0 and not eng.alloc.append(s.seq_id, short):
            raise MemoryError("no cache block for the profiled step")
    B, nsplit = r._stage_decode(seqs, eng.alloc)
    inp = r._decode_inputs(B, nsplit)
    r.model.profile_layers(inp)
    stages = r.model.profile_layers(inp)
    per_layer = [s["ms"] for s in stages if s["stage"].startswith("layer")]
    other = sum(s["ms"] for s in stages if not s["stage"].startswith("layer"))
    mean = sum(per_layer) / max(1, len(per_layer))
    del eng
    torch.cuda.empty_cache()
    return {"model": model, "weight_format": cfg.weight_format, "batch": batch, "ctx": ctx, "layers_timed": len(per_layer),
            "layer_ms_mean": round(mean, 4), "layer_ms_min": round(min(per_layer), 4), "layer_ms_max": round(max(per_layer), 4),
            "embed_and_head_ms": round(other, 4),
            "whole_model_step_ms_predicted": round(mean * full.n_layers + other, 3),
            "note": "eager launches with an event after every stage: kernels do not overlap as they do in the decode graph",
            "stages": stages}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.3-70b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", default="1,8,64")
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--weight-format")
    a = ap.parse_args(argv)
    for b in [int(x) for x in a.batch.split(",")]:
        print(json.dumps(layer_times(a.model, a.layers, b, a.ctx, a.weight_format)))


if __name__ == "__main__":
    main()
