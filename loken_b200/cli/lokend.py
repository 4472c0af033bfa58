"""`lokend serve`: load the configured model(s) and serve the HTTP API.

    python -m loken_b200.cli.lokend serve --config loken.toml
    python -m loken_b200.cli.lokend serve --model model.gguf --port 8080 --tp 8

With tensor parallelism the command is started once per GPU by torch.distributed.run; rank 0
serves HTTP and the other ranks follow its engine steps (`parallel/follower.py`).  Start-up
order follows the reference's `src/bin/lokend.rs:64-560`: config, device probe, model load,
optional drafter, routes.
"""
from __future__ import annotations

import argparse
import sys

from ..config import load_config


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="lokend")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve", help="serve the HTTP API")
    s.add_argument("--config", help="TOML configuration file")
    s.add_argument("--model", help="GGUF path or built-in shape name (overrides [inference] model)")
    s.add_argument("--model-id")
    s.add_argument("--host")
    s.add_argument("--port", type=int)
    s.add_argument("--tp", type=int)
    s.add_argument("--max-seqs", type=int)
    s.add_argument("--max-ctx", type=int)
    s.add_argument("--draft-model")
    s.add_argument("--draft-k", type=int)
    s.add_argument("--keep-alive", help="how long a model stays on the device after its last request (5m, 300s, 1h, a bare "
                                        "number is seconds; -1 keeps it for ever); OLLAMA_KEEP_ALIVE is read too")
    s.add_argument("--lora", help="PEFT adapter directory merged into a bf16 / block-fp8 checkpoint at load")
    s.add_argument("--tp-sum", choices=["boundary", "push", "fused", "nccl"],
                   help="how tensor-parallel layers are summed (boundary = one kernel per layer boundary: "
                        "reduce-scatter + residual + norm + all-gather)")
    s.add_argument("--expert-slots", type=int,
                   help="mixture models larger than the card: experts per layer kept resident, the rest streamed from host memory")
    s.add_argument("--requant", choices=["fp8_block", "bf16"], help="re-encode float tensors at load")
    sub.add_parser("check-config", help="parse the configuration and print what was ignored").add_argument(
        "--config", required=True)
    return ap


def apply_flags(cfg, args):
    i, s = cfg.inference, cfg.server
    for name, target, attr in (("model", i, "model"), ("model_id", i, "model_id"), ("host", s, "host"),
                               ("port", s, "port"), ("tp", i, "tp"), ("max_seqs", i, "max_seqs"),
                               ("max_ctx", i, "max_ctx"), ("draft_model", i, "draft_model"),
                               ("draft_k", i, "draft_k"), ("lora", i, "lora"), ("tp_sum", i, "tp_sum"),
                               ("expert_slots", i, "expert_slots")):
        v = getattr(args, name, None)
        if v is not None:
            setattr(target, attr, v)
    if getattr(args, "keep_alive", None) is not None:
        from ..config import _parse_duration

        i.keep_alive_s = _parse_duration(args.keep_alive)
    return cfg.validate()


def serve(cfg, requant=None) -> int:
    from ..api.common import ModelRegistry
    from ..api.context import ServerSettings
    from ..api.server import serve as http_serve
    from ..engine.llm import LLM

    i, s = cfg.inference, cfg.server
    if not i.model:
        print("lokend: no model configured ([inference] model or --model)", file=sys.stderr)
        return 2
    import os as _os

    if not _os.path.exists(i.model):
        from ..store.catalogue import Catalogue as _Cat

        hit = _Cat(cfg.ollama_models_dir, cfg.huggingface_models_dir).resolve(i.model)
        if hit is not None:                   # `name:tag`, `owner/repo` or a GGUF's file name in a model store
            i.model_id = i.model_id or hit.name
            i.model = hit.path
    comm, rank, world = None, 0, 1
    if i.tp > 1:
        from ..parallel.comm import init_distributed
        from ..parallel.symm import SymmComm

        rank, world, local = init_distributed()
        if world != i.tp:
            print(f"lokend: tp = {i.tp} but {world} ranks were started", file=sys.stderr)
            return 2
        import torch

        from ..models.loader import peek_config

        shape = peek_config(i.model)          # the symmetric heap is sized from the model's own shape
        if i.tp_sum == "nccl":
            from ..parallel.comm import NcclComm

            comm = NcclComm()
        else:
            comm = SymmComm(torch.device("cuda", local), max_rows=max(i.max_seqs, 256), hidden=shape.hidden,
                            top_k=shape.top_k if shape.is_moe else 0)
            comm.fused_norm = i.tp_sum == "boundary"
            comm.fused_gemm = i.tp_sum == "fused"
    llm = LLM.load(i.model, model_id=i.model_id, requant=requant, kv_format=cfg.kv_format, tp_rank=rank,
                   tp_size=world, comm=comm, max_seqs=i.max_seqs, max_ctx=i.max_ctx,
                   max_prefill_tokens=i.max_prefill_tokens, lora=i.lora, expert_slots=i.expert_slots,
                   kv_disk_dir=i.kv_disk_dir if world == 1 else None, kv_disk_host_mb=i.kv_disk_host_mb,
                   kv_disk_max_gb=i.kv_disk_max_gb,
                   **({"draft": (i.draft_model, i.draft_k)} if (i.draft_model and world > 1) else {}))
    if i.draft_model and world == 1:
        from ..serve.speculative import attach_draft

        attach_draft(llm, i.draft_model, k=i.draft_k)
    for n in cfg.notes:
        print("lokend: config:", n, file=sys.stderr)
    if rank != 0:
        from ..parallel.follower import follow

        return follow(llm, llm.control_group, llm.watchdog)
    reg = ModelRegistry()
    reg.add(llm, default=True)
    from ..store.catalogue import Catalogue

    catalogue = Catalogue(cfg.ollama_models_dir, cfg.huggingface_models_dir)
    http_serve(reg, ServerSettings(host=s.host, port=s.port, api_keys=s.api_keys, require_auth=s.require_auth,
                                   allowed_origins=s.allowed_origins, rate_limit_rps=s.rate_limit_rps,
                                   rate_limit_burst=s.rate_limit_burst, max_body_bytes=s.max_body_mb << 20,
                                   request_timeout_s=s.request_timeout_s, gate_slots=i.max_seqs,
                                   prefill_peer=i.prefill_peer, route_requests=cfg.cluster.route_requests,
                                   keep_alive_s=(i.keep_alive_s if world == 1 else -1.0),
                                   resume_unverified=cfg.cluster.resume_unverified, node_id=cfg.cluster.node_id),
          cluster=cfg.cluster, catalogue=catalogue)
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    cfg = load_config(args.config)
    if args.cmd == "check-config":
        for n in cfg.notes:
            print(n)
        print("ok")
        return 0
    cfg = apply_flags(cfg, args)
    return serve(cfg, requant=args.requant)


if __name__ == "__main__":
    sys.exit(main())
