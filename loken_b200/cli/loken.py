"""`loken`: the client and model tool (`src/bin/loken.rs:33-172`).

    loken list | ps | show MODEL          talk to a running lokend
    loken generate MODEL PROMPT           one completion (streams to the terminal)
    loken chat MODEL                      interactive chat
    loken load PATH [--id NAME]           ask the server to load a model
    loken delete MODEL                    unload it
    loken validate FILE.gguf              check a GGUF file: header, tensor table, payload sizes
    loken convert --from in.gguf --format q4_k_m -o out.gguf [--calibration rec.json]     re-encode a model
    loken convert --shape NAME --format q8_0 -o out.gguf     write a random-init model file
    loken draft attach|detach|status
    loken pull NAME                       fetch a model into the daemon's stores (streams progress; resumable)
    loken swap PATH [--id NAME]           replace the resident model
    loken launch AGENT [-m MODEL] [--config] [-- ARGS]      run a coding agent against the daemon
    loken popular                         a few models to start with
    loken calibrate MODEL -n NAME -t FILE...   have the daemon record a calibration for `convert`
    loken draft-head SOURCE OUT           write a model's multi-token-prediction head (its `mtp.*` tensors) as a
                                          companion file the daemon can attach (`loken draft attach --method head`)
"""
from __future__ import annotations

import argparse
import json
import sys
import urllib.error
import urllib.request
from typing import Iterator, Optional


class Client:
    """Minimal HTTP client of the server's own API (the reference's `src/api/client.rs`)."""

    def __init__(self, base: str = "http://127.0.0.1:11434", api_key: Optional[str] = None, timeout: float = 600.0):
        self.base, self.key, self.timeout = base.rstrip("/"), api_key, timeout

    def _req(self, method: str, path: str, body=None):
        data = None if body is None else json.dumps(body).encode()
        req = urllib.request.Request(self.base + path, data=data, method=method)
        req.add_header("content-type", "application/json")
        if self.key:
            req.add_header("authorization", f"Bearer {self.key}")
        return urllib.request.urlopen(req, timeout=self.timeout)

    def json(self, method: str, path: str, body=None):
        try:
            with self._req(method, path, body) as r:
                return json.loads(r.read() or b"{}")
        except urllib.error.HTTPError as e:
            raise SystemExit(f"loken: {e.code} {e.read().decode(errors='replace')}")
        except urllib.error.URLError as e:
            raise SystemExit(f"loken: cannot reach {self.base}: {e.reason}")

    def ndjson(self, path: str, body) -> Iterator[dict]:
        try:
            with self._req("POST", path, body) as r:
                for line in r:
                    line = line.strip()
                    if line:
                        yield json.loads(line)
        except urllib.error.HTTPError as e:
            raise SystemExit(f"loken: {e.code} {e.read().decode(errors='replace')}")
        except urllib.error.URLError as e:
            raise SystemExit(f"loken: cannot reach {self.base}: {e.reason}")


def validate_gguf(path: str) -> dict:
    """Opens the file, walks the tensor table and checks that every payload has the size its type
    and shape imply and lies inside the file."""
    from ..formats import gguf as G

    r = G.GGUFReader(path)
    problems = []
    total = 0
    for name, t in r.tensors.items():
        try:
            bv, bb = G.block_info(t.ggml_type)
        except ValueError:
            problems.append(f"{name}: unknown tensor type {t.ggml_type}")
            continue
        n = 1
        for d in t.shape:
            n *= d
        if t.shape and t.shape[-1] % bv:
            problems.append(f"{name}: row of {t.shape[-1]} values is not a whole number of {bv}-value blocks")
        want = n // bv * bb
        if want != t.nbytes:
            problems.append(f"{name}: payload is {t.nbytes} bytes, shape and type imply {want}")
        total += t.nbytes
    arch = r.meta.get("general.architecture")
    if not arch:
        problems.append("general.architecture is missing")
    elif f"{arch}.block_count" not in r.meta:
        problems.append(f"{arch}.block_count is missing")
    out = {"file": path, "version": r.version, "tensors": len(r.tensors), "metadata_keys": len(r.meta),
           "payload_bytes": total, "architecture": arch, "problems": problems, "ok": not problems}
    r.close()
    return out


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="loken")
    ap.add_argument("--server", default="http://127.0.0.1:11434")
    ap.add_argument("--api-key")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("list")
    sub.add_parser("ps")
    sub.add_parser("show").add_argument("model")
    g = sub.add_parser("generate")
    g.add_argument("model")
    g.add_argument("prompt")
    g.add_argument("--max-tokens", type=int, default=256)
    g.add_argument("--temperature", type=float)
    c = sub.add_parser("chat")
    c.add_argument("model")
    c.add_argument("--system")
    ld = sub.add_parser("load")
    ld.add_argument("path")
    ld.add_argument("--id")
    sub.add_parser("delete").add_argument("model")
    sub.add_parser("validate").add_argument("file")
    sub.add_parser("repair").add_argument("file")
    cv = sub.add_parser("convert")
    cv.add_argument("--shape", help="built-in shape name, e.g. qwen3-1.7b: write a random-init model file")
    cv.add_argument("--from", dest="source", help="a GGUF file to re-encode in --format")
    cv.add_argument("--calibration", help="a calibration record (JSON) that lifts the most sensitive tensors one step")
    cv.add_argument("--format", default="q8_0", choices=["q8_0", "q4_k_m", "q4_k", "q6_k", "bf16", "f16", "mxfp4"])
    cv.add_argument("--layers", type=int, help="write only the first N layers")
    cv.add_argument("-o", "--output", required=True)
    cv.add_argument("--seed", type=int, default=0)
    d = sub.add_parser("draft")
    d.add_argument("action", choices=["attach", "detach", "status"])
    d.add_argument("--model")
    d.add_argument("--draft")
    d.add_argument("-k", type=int, default=4)
    d.add_argument("--method", default="model", choices=["model", "prompt_lookup", "head"],
                   help="head: --draft names a directory with an EAGLE or MTP head, or random:eagle / random:mtp")
    pl = sub.add_parser("pull")
    pl.add_argument("name", help="name:tag of an Ollama registry model, or owner/repo[:file] on the Hugging Face hub")
    pl.add_argument("--insecure", action="store_true")
    sw = sub.add_parser("swap")
    sw.add_argument("path")
    sw.add_argument("--id")
    la = sub.add_parser("launch")
    la.add_argument("agent", choices=["claude", "cline"])
    la.add_argument("-m", "--model")
    la.add_argument("--config", action="store_true", help="print or write the configuration and start nothing")
    la.add_argument("args", nargs="*", help="arguments handed to the agent, after --")
    sub.add_parser("popular")
    sub.add_parser("peers", help="the nodes this server sees: alive, suspicion, round trip, what each serves")
    ca = sub.add_parser("calibrate")
    ca.add_argument("model", help="the checkpoint: a path or a name in the model stores")
    ca.add_argument("-n", "--name", required=True, help="the record's name, which convert refers to")
    ca.add_argument("-t", "--text", required=True, nargs="+", help="text files to calibrate on, read here and sent")
    ca.add_argument("--excerpt", type=int, help="characters taken from each text")
    ca.add_argument("--tokens", type=int, help="tokens in all")
    pc = sub.add_parser("plan-cut", help="where to cut a layer stack over nodes; computed here, no server needed")
    pc.add_argument("spec", help="a JSON file: layers, layer_bytes, nodes, links, objective (see cluster/cut_plan.py)")
    dh = sub.add_parser("draft-head")
    dh.add_argument("source", help="a checkpoint directory (safetensors), a GGUF file that carries mtp.* tensors, or a hub "
                                   "repository (owner/name): then only the head's bytes are fetched, by ranged reads")
    dh.add_argument("output", help="OUT.gguf, or a directory for a safetensors companion")
    return ap


POPULAR = (
    ("Qwen/Qwen3-0.6B", "small enough for a laptop CPU"),
    ("Qwen/Qwen3-8B", "general purpose, one GPU with room to spare"),
    ("meta-llama/Llama-3.1-8B-Instruct", "the common baseline; Q4_K_M files are everywhere"),
    ("openai/gpt-oss-120b", "a mixture model in MXFP4: one B200, or eight with expert parallelism"),
    ("meta-llama/Llama-3.3-70B-Instruct", "block-fp8 on one B200, tensor-parallel for latency"),
)


def extract_draft_head(source: str, output: str) -> dict:
    """Collects a checkpoint's multi-token-prediction tensors (`mtp.*`, with or without a `model.` prefix) and
    writes them as a companion: OUT.gguf (tensor names without the prefix, `general.type = draft-head`) or a
    directory holding `head.safetensors`.  Both are what `serve/draft_head.py: load_draft_head` reads."""
    import glob
    import os

    import numpy as np

    tensors = {}
    if os.path.isdir(source):
        from safetensors import safe_open

        for f in sorted(glob.glob(os.path.join(source, "*.safetensors"))):
            with safe_open(f, framework="pt", device="cpu") as h:
                for k in h.keys():
                    name = k.removeprefix("model.")
                    if name.startswith("mtp."):
                        tensors[name[4:]] = h.get_tensor(k).float().numpy()
    else:
        from ..formats import gguf as G

        r = G.GGUFReader(source)
        try:
            for k, ti in r.tensors.items():
                if k.startswith("mtp."):
                    tensors[k[4:]] = ti.to_float()
        finally:
            r.close()
    if not tensors:
        raise ValueError(f"{source} carries no mtp.* tensors")
    if output.endswith(".gguf"):
        from ..formats import gguf as G

        w = G.GGUFWriter(output)
        w.add_meta("general.type", "draft-head")
        w.add_meta("general.name", os.path.basename(os.path.normpath(source)) + " (mtp)")
        for k, v in tensors.items():
            w.add_tensor(k, np.ascontiguousarray(v, dtype=np.float32), G.F32 if v.ndim < 2 else G.BF16)
        w.close()
    else:
        import torch
        from safetensors.torch import save_file

        os.makedirs(output, exist_ok=True)
        save_file({k: torch.from_numpy(np.ascontiguousarray(v)).bfloat16() if v.ndim >= 2 else torch.from_numpy(v.copy())
                   for k, v in tensors.items()}, os.path.join(output, "head.safetensors"))
    return {"source": source, "output": output, "tensors": len(tensors),
            "bytes": int(sum(v.size for v in tensors.values()) * 2)}


def main(argv=None, out=sys.stdout) -> int:
    args = build_parser().parse_args(argv)
    cl = Client(args.server, args.api_key)
    p = lambda *a: print(*a, file=out)
    if args.cmd == "list":
        for m in cl.json("GET", "/api/tags")["models"]:
            p(f"{m['name']:40s} {m['details']['parameter_size']:>8s} {m['details']['quantization_level']}")
    elif args.cmd == "ps":
        for m in cl.json("GET", "/api/ps")["models"]:
            p(f"{m['name']:40s} ctx {m.get('context_length')}")
    elif args.cmd == "show":
        p(json.dumps(cl.json("POST", "/api/show", {"model": args.model}), indent=1))
    elif args.cmd == "generate":
        opts = {"num_predict": args.max_tokens}
        if args.temperature is not None:
            opts["temperature"] = args.temperature
        for ev in cl.ndjson("/api/generate", {"model": args.model, "prompt": args.prompt, "options": opts}):
            out.write(ev.get("response", ""))
            out.flush()
        p()
    elif args.cmd == "chat":
        msgs = [{"role": "system", "content": args.system}] if args.system else []
        while True:
            try:
                line = input(">>> ")
            except EOFError:
                break
            if line.strip() in ("/bye", "/exit"):
                break
            msgs.append({"role": "user", "content": line})
            text = ""
            for ev in cl.ndjson("/api/chat", {"model": args.model, "messages": msgs}):
                piece = ev.get("message", {}).get("content", "")
                text += piece
                out.write(piece)
                out.flush()
            p()
            msgs.append({"role": "assistant", "content": text})
    elif args.cmd == "load":
        p(json.dumps(cl.json("POST", "/load", {"model": args.path, "id": args.id}), indent=1))
    elif args.cmd == "delete":
        p(json.dumps(cl.json("DELETE", f"/api/models/{args.model}")))
    elif args.cmd in ("validate", "repair"):
        rep = validate_gguf(args.file)
        p(json.dumps(rep, indent=1))
        if args.cmd == "repair" and not rep["ok"]:
            p("loken: nothing can be rebuilt from the file itself; fetch it again")
        return 0 if rep["ok"] else 1
    elif args.cmd == "convert":
        import dataclasses

        from ..models.config import get_config
        from ..models.loader import export_random_gguf

        if args.source:
            from ..formats.requant import requantize_gguf

            rep = requantize_gguf(args.source, args.output, args.format, calibration=args.calibration)
            p(json.dumps(rep, indent=1))
            return 0
        if not args.shape:
            p("loken convert: give --from FILE.gguf (re-encode a model) or --shape NAME (write a random-init one)")
            return 2
        cfg = dataclasses.replace(get_config(args.shape), weight_format=args.format)
        if args.layers:
            cfg = dataclasses.replace(cfg, n_layers=args.layers)
        export_random_gguf(args.output, cfg, seed=args.seed)
        p(f"wrote {args.output}")
    elif args.cmd == "popular":
        p("A few models to start with, by their Hugging Face ids:")
        for name, why in POPULAR:
            p(f"  {name}\n      {why}")
        p("`loken pull NAME` fetches one; any GGUF file or safetensors directory loads with `loken load PATH`.")
    elif args.cmd == "calibrate":
        texts = []
        for path in args.text:
            with open(path, encoding="utf-8", errors="replace") as f:
                texts.append(f.read())
        body = {"model": args.model, "name": args.name, "texts": texts}
        if args.excerpt:
            body["excerpt"] = args.excerpt
        if args.tokens:
            body["tokens"] = args.tokens
        last = None
        for ev in cl.ndjson("/api/calibrate", body):
            last = ev
            p(json.dumps(ev))
        return 0 if last is not None and "error" not in last else 1
    elif args.cmd == "peers":
        rep = cl.json("GET", "/api/cluster/peers")
        if not rep.get("clustered"):
            p("this server sees no other node ([cluster] peers or discovery join it to others)")
        for n in rep.get("peers", []):
            st = n.get("state") or {}
            rtt = "-" if n.get("rtt_ms") is None else f"{n['rtt_ms']:.1f} ms"
            p(f"{n['node_id']:20s} {'self ' if n['is_self'] else ('alive' if n['alive'] else 'gone ')} phi {n['phi']:5.2f}  rtt {rtt:>9s}  "
              f"{st.get('tok_per_s', 0.0):7.1f} tok/s  {', '.join(st.get('models', [])) or '-'}")
    elif args.cmd == "plan-cut":
        from ..cluster.cut_plan import plan_from_request

        try:
            with open(args.spec) as f:
                plan = plan_from_request(json.load(f))
        except (ValueError, KeyError, TypeError, OSError) as e:
            p(f"loken plan-cut: {e}")
            return 2
        if plan is None:
            p("loken plan-cut: no arrangement of these layers fits these nodes over these links")
            return 1
        for sgm in plan.segments:
            p(f"{sgm.node:20s} layers {sgm.lo:3d} .. {sgm.hi - 1:3d}  ({len(sgm)})")
        p(f"crossings {plan.crossing_ms:.3f} ms per token, objective {plan.total_ms:.3f}" + ("" if plan.exact else "  (fixed node order: not exact)"))
    elif args.cmd == "draft-head":
        try:
            import os

            if not os.path.exists(args.source) and args.source.count("/") == 1 and args.output.endswith(".gguf"):
                from ..store.download import fetch_draft_head

                p(json.dumps(fetch_draft_head(args.source, args.output, token=os.environ.get("HF_TOKEN")), indent=1))
            else:
                p(json.dumps(extract_draft_head(args.source, args.output), indent=1))
        except (ValueError, OSError) as e:
            p(f"loken draft-head: {e}")
            return 1
    elif args.cmd == "swap":
        p(json.dumps(cl.json("POST", "/api/swap", {"model": args.path, "id": args.id}), indent=1))
    elif args.cmd == "pull":
        # a pull is stalled when no progress line arrives for 8 times the longest gap seen so far
        import time

        last, longest, status = time.monotonic(), 5.0, None
        for ev in cl.ndjson("/api/pull", {"model": args.name, "insecure": args.insecure}):
            now = time.monotonic()
            longest, last = max(longest, now - last), now
            if ev.get("error"):
                p(f"loken: {ev['error']}")
                return 1
            if ev.get("total"):
                out.write(f"\r{ev.get('status', '')}: {100.0 * ev.get('completed', 0) / ev['total']:5.1f} %")
                out.flush()
            elif ev.get("status") != status:
                status = ev.get("status")
                p(f"\n{status}" if status else "")
        p()
    elif args.cmd == "launch":
        import os

        from . import launch as L

        loaded = [m["name"] for m in cl.json("GET", "/api/ps").get("models", [])]
        held = [m["name"] for m in cl.json("GET", "/api/tags").get("models", [])]
        try:
            model = L.pick_model(args.model, loaded, held)
            info = cl.json("POST", "/api/show", {"model": model}).get("model_info") or {}
            window = next((int(v) for k, v in info.items() if k.endswith(".context_length")), None)
            key = os.environ.get("LOKEN_API_KEY") or args.api_key or None
            return L.launch(args.agent, L.Launch(args.server, model, key, window), args.config, args.args, out)
        except ValueError as e:
            p(f"loken: {e}")
            return 1
    elif args.cmd == "draft":
        if args.action == "status":
            p(json.dumps(cl.json("GET", "/api/draft/status"), indent=1))
        elif args.action == "attach":
            p(json.dumps(cl.json("POST", "/api/draft/attach", {"model": args.model, "draft": args.draft, "k": args.k,
                                                               "method": args.method}), indent=1))
        else:
            p(json.dumps(cl.json("POST", "/api/draft/detach", {"model": args.model})))
    else:
        p(f"loken {args.cmd}: unknown command")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
