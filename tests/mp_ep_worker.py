"""Child process of the expert-parallel test: a tiny gpt-oss-shaped mixture model (sinks, sliding
window, clamped SwiGLU, expert biases) at EP = TP = world against the degree-1 ENGINE on the same
GPU.  Two ways to run the mixture layers at degree N: "replicated" (every rank holds every token,
computes its own experts' pairs, partial rows are summed by an all-reduce) and "dispatch" (the
residual stream is sharded by rows; pairs travel to the experts' ranks and back over peer memory).
bf16 experts must reproduce degree 1 to cosine >= 0.9995 at nine positions in ten (one more bf16 rounding
per partial sum; a flipped near-tie expert choice may move single positions further) with greedy tokens
equal up to near-ties; MXFP4 experts (e4m3 activations on the block-scaled tensor-core path) to the
format's own noise."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from loken_b200.models.config import tiny  # noqa: E402
from loken_b200.models.weights import random_weights  # noqa: E402
from loken_b200.parallel.comm import init_distributed  # noqa: E402
from loken_b200.parallel.symm import SymmComm  # noqa: E402
from loken_b200.serve.engine import LLMEngine  # noqa: E402
from loken_b200.serve.params import SamplingParams  # noqa: E402


def run(eng, prompts, sp):
    ids = [eng.add_request(p, sp) for p in prompts]
    steps = []
    while eng.has_work():
        eng.step()
        lg = eng.runner.last_logits
        steps.append(lg.float().clone() if lg is not None else None)
    return [eng.seqs[i].output for i in ids], steps


def main():
    out_path = sys.argv[1]
    fmt = sys.argv[2] if len(sys.argv) > 2 else "bf16"
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    cfg = tiny("gpt-oss", weight_format=fmt, n_experts=8, top_k=2, hidden=256, expert_intermediate=256, n_q=8, n_kv=8,
               head_dim=64, vocab=512, n_layers=3)
    if fmt == "bf16":
        cfg.kv_format = "bf16"      # the tight bound needs every rounding step shared by both degrees: no int8 cache
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (19, 40, 7, 33, 12)]
    sp = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, max_tokens=5)
    kw = dict(num_blocks=64, max_seqs=8, max_prefill_tokens=256, max_ctx=256)
    rep = {"world": world, "format": fmt}
    w1 = random_weights(cfg, dev, seed=5, std=0.05)
    e1 = LLMEngine(cfg, weights=w1, device=dev, **kw)
    ref_tokens, ref_logits = run(e1, prompts, sp)
    del e1
    for name in ("replicated", "dispatch"):
        comm = SymmComm(dev, max_rows=256, hidden=cfg.hidden, top_k=cfg.top_k)
        comm.fused_norm = name == "dispatch"
        w = random_weights(cfg, dev, seed=5, std=0.05, tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world)
        eng = LLMEngine(cfg, weights=w, device=dev, tp_rank=rank, tp_size=world, comm=comm, **kw)
        toks, logits = run(eng, prompts, sp)
        cos_min, ok, cosines = 1.0, True, []
        alive = [True] * len(prompts)
        for a, b in zip(logits, ref_logits):
            if a is None or b is None or a.shape != b.shape:
                ok = False
                break
            for i in range(len(prompts)):
                if not alive[i]:
                    continue
                cosines.append(torch.nn.functional.cosine_similarity(a[i], b[i], dim=0).item())
                cos_min = min(cos_min, cosines[-1])
                if int(a[i].argmax()) != int(b[i].argmax()):
                    top2 = torch.topk(b[i], 2).values
                    ok &= bool((top2[0] - top2[1]) < 0.01 * b[i].abs().max())
                    alive[i] = False
        # a mixture model has discrete choices inside: a rounding-order difference can flip an expert that was
        # a near-tie at one position, which moves that position's logits by far more than rounding does.  So the
        # rounding bound holds for nine positions in ten, and the worst position stays within one flipped expert.
        cosines.sort()
        cos_p10 = cosines[len(cosines) // 10] if cosines else 0.0
        rep[f"logits_cos_p10_{name}"] = cos_p10
        passed = (ok and cos_p10 >= 0.9995 and cos_min >= 0.98) if fmt == "bf16" else (cos_p10 >= 0.99 and cos_min >= 0.9)
        flag = torch.tensor([int(passed)], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        rep[f"match_{name}"] = bool(flag.item())
        rep[f"tokens_equal_{name}"] = toks == ref_tokens
        rep[f"logits_cos_min_{name}"] = cos_min
        rep[f"status_{name}"] = eng.runner.wsp.read_status()
        rep[f"sharded_steps_{name}"] = int(eng.runner.model.sharded_steps)
        del eng
        torch.cuda.synchronize()
        dist.barrier()
        comm.close()
    if rank == 0:
        json.dump(rep, open(out_path, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
