"""The HTTP server: one FastAPI app carrying the Ollama, OpenAI and Messages dialects plus the
operational routes, behind the cross-cutting layers the reference stacks on its router
(`src/api/handlers/mod.rs:3084-3165`): request id, API-key auth with per-key cache scope, token-
bucket rate limit, body limit, CORS, and errors in each dialect's own envelope.

    app = create_app(registry, ServerSettings(...));  uvicorn.run(app, host=..., port=...)
"""
from __future__ import annotations

import time
from typing import Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse

from . import anthropic, files, ollama, openai, pooling
from .common import ApiError, ModelRegistry, new_request_id
from .context import VERSION, ServerContext, ServerSettings

OPEN_PATHS = {"/", "/health", "/ping", "/version", "/api/version", "/metrics"}


def error_body(path: str, e: ApiError) -> dict:
    if path.startswith("/api/"):
        return {"error": e.message}
    if path.startswith("/v1/messages"):
        return {"type": "error", "error": {"type": e.kind, "message": e.message}}
    return {"error": {"message": e.message, "type": e.kind, "param": None, "code": e.code}}


def ops_router(ctx: ServerContext):
    from fastapi import APIRouter

    r = APIRouter()

    @r.get("/health")
    async def health():
        models = ctx.registry.list()
        ok = all(m.worker.healthy for m in models)
        body = {"status": "ok" if ok else "degraded", "models": [m.model_id for m in models],
                "uptime_s": round(time.time() - ctx.started, 1)}
        return JSONResponse(body, status_code=200 if ok else 503)

    @r.get("/ping")
    async def ping():
        return PlainTextResponse("pong")

    @r.get("/version")
    async def version():
        from ..version import stamp

        return dict(stamp(), version=VERSION)

    @r.post("/api/cluster/prefill")
    async def cluster_prefill(req: Request):
        # disaggregated prefill: this node reads the prompt and answers with its cache, which the
        # asking node imports and decodes from (`cluster/handover.py`)
        from fastapi.responses import Response
        from starlette.concurrency import run_in_threadpool

        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        ids = body.get("prompt_ids")
        if ids is None:
            ids = llm.prompt_ids(body.get("prompt"), body.get("messages"))
        if not ids:
            raise ApiError(400, "prompt, messages or prompt_ids is required")
        try:
            blob = await run_in_threadpool(llm.on_engine_thread, lambda eng: eng.export_prefix(list(ids)))
        except ValueError as e:
            raise ApiError(400, str(e))
        return Response(blob, media_type="application/octet-stream",
                        headers={"x-loken-tokens": str(len(ids))})

    @r.post("/api/cluster/import")
    async def cluster_import(req: Request, model: Optional[str] = None):
        from starlette.concurrency import run_in_threadpool

        blob = await req.body()
        llm = ctx.registry.get(model)
        try:
            n = await run_in_threadpool(llm.on_engine_thread, lambda eng: eng.import_prefix(blob))
        except (ValueError, MemoryError) as e:
            raise ApiError(400, str(e))
        return {"status": "imported", "tokens": n}

    def _describe() -> dict:
        models = ctx.registry.list()
        free = sum(m.engine.alloc.free_blocks() for m in models)
        return {"models": [m.model_id for m in models], "load": float(sum(len(m.worker.tickets) for m in models)),
                "tok_per_s": float(ctx.rate.rate), "prefill_tok_per_s": float(ctx.prefill_rate.rate),
                "free_kv_blocks": int(free), "layer_cost": dict(ctx.layer_cost),
                "card_bytes_free": int(_card_bytes_free())}

    def _card_bytes_free() -> int:
        try:
            import torch

            if not torch.cuda.is_available():
                return 0
            return int(sum(torch.cuda.mem_get_info(i)[0] for i in range(torch.cuda.device_count())))
        except Exception:
            return 0

    def _membership():
        if getattr(ctx, "membership", None) is None:
            import socket

            from ..cluster.membership import Membership

            ctx.membership = Membership(ctx.settings.node_id or socket.gethostname())
        return ctx.membership

    ctx.describe = _describe

    @r.get("/api/cluster/state")
    async def cluster_state():
        return dict(_membership().state(), **{"self_state": _describe()})

    @r.post("/api/cluster/gossip")
    async def cluster_gossip(req: Request):
        from ..cluster.gossip import fold

        m = _membership()
        body = await req.json()
        if not isinstance(body, dict) or not body.get("id"):
            raise ApiError(400, "a gossip payload names its sender (id)")
        fold(m, body)
        d = _describe()
        return m.gossip_payload(f"http://{ctx.settings.host}:{ctx.settings.port}", d["models"], d["load"],
                                d["tok_per_s"], d["free_kv_blocks"], d["layer_cost"], d["card_bytes_free"],
                                d["prefill_tok_per_s"])

    @r.get("/api/cluster/peers")
    async def cluster_peers():
        """Who this node sees (`docs/CLUSTER.md:44` of the reference): `clustered` and one record per peer."""
        m = _membership()
        st = m.state()
        me = {"node_id": m.self_id, "endpoint": f"http://{ctx.settings.host}:{ctx.settings.port}", "alive": True, "phi": 0.0,
              "rtt_ms": 0.0, "is_self": True, "state": _describe()}
        peers = [{"node_id": p["id"], "endpoint": p["addr"], "alive": p["alive"] and not p["excluded"], "phi": p["phi"],
                  "rtt_ms": p["rtt_ms"], "is_self": False,
                  "state": {k: p[k] for k in ("models", "load", "tok_per_s", "layer_cost", "card_bytes_free")}} for p in st["peers"]]
        return {"clustered": bool(peers), "peers": [me] + peers}

    @r.post("/api/cluster/prefix")
    async def cluster_prefix(req: Request):
        """How much of a prompt this node already holds in its prefix cache.  Only this node can answer: it
        tokenises for its own model and looks in its own cache.  A model that is not resident answers 0."""
        body = await req.json()
        name = body.get("model")
        if name and name not in ctx.registry.models and name not in ctx.registry.aliases:
            return {"cached_tokens": 0}          # by its exact name: the default model's cache says nothing about another model
        try:
            llm = ctx.registry.get(name)
        except ApiError:
            return {"cached_tokens": 0}
        prompt = body.get("prompt", "")
        ids = [int(t) for t in prompt] if isinstance(prompt, list) else llm.tokenize(str(prompt))
        if not ids:
            return {"cached_tokens": 0}
        # a cached prompt belongs to the key that wrote it: the answer covers the caller's own scope only
        scope = body.get("cache_salt") or (("key:" + req.state.api_key) if getattr(req.state, "api_key", None) else None)
        salt = 0
        if scope:
            from ..engine.llm import GenerationParams

            salt = llm._salt(GenerationParams(cache_salt=str(scope)))
        alloc = llm.engine.alloc
        return {"cached_tokens": len(alloc.match_prefix(ids, salt)[0]) * alloc.block_size, "prompt_tokens": len(ids)}

    @r.post("/api/cluster/measure")
    async def cluster_measure(req: Request):
        """What a layer of `model` costs on this node, measured now and published with the next gossip round:
        `card_ms` (one decode row through one layer on the device), `host_ms` (0: this build runs no layer of a
        device-resident model on the host) and `card_bytes` (one layer's weights and its share of the cache).  A
        head that plans a pipeline cut asks it of a peer that has no figure for the model yet."""
        from starlette.concurrency import run_in_threadpool

        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        rows = await run_in_threadpool(llm.on_engine_thread, lambda eng: eng.layer_perf(1))
        per_layer = [float(r["ms"]) for r in rows if str(r.get("stage", "")).startswith("layer")]
        if not per_layer:
            raise ApiError(500, "the engine reported no per-layer times")
        cfg = llm.cfg
        bits = {"bf16": 16.0, "fp8": 8.25, "q8_0": 8.5, "q6_k": 6.5625, "q4_k": 4.5, "q4_k_m": 4.85, "mxfp4": 4.25}.get(cfg.weight_format, 16.0)
        from ..cluster.cut_plan import layer_bytes_of

        cost = {"card_ms": sum(per_layer) / len(per_layer), "host_ms": 0.0,
                "card_bytes": int(layer_bytes_of(cfg, weight_bits=bits, kv_tokens=int(body.get("context", 0)))[0]),
                "layers": cfg.n_layers}
        ctx.layer_cost[llm.model_id] = cost
        return cost

    @r.get("/api/multi-device/status")
    async def multi_device_status():
        """How each resident model is spread over devices: parallel degrees, this rank's device, cache blocks."""
        out = []
        for m in ctx.registry.list():
            eng = getattr(m.engine, "_e", m.engine)
            w = getattr(eng, "weights", None)
            out.append({"model": m.model_id, "device": str(getattr(eng, "device", "cpu")),
                        "tp": int(getattr(w, "tp_size", 1) or 1), "tp_rank": int(getattr(w, "tp_rank", 0) or 0),
                        "ep": int(getattr(w, "ep_size", 1) or 1), "layers": m.cfg.n_layers,
                        "layer_range": list(getattr(w, "layer_range", None) or (0, m.cfg.n_layers)),
                        "kv_blocks": int(eng.alloc.num_blocks), "kv_blocks_free": int(eng.alloc.free_blocks()),
                        "kv_block_tokens": int(eng.alloc.block_size),
                        "disk_tier": eng.disk.stats() if getattr(eng, "disk", None) is not None else None})
        return {"models": out}

    @r.get("/api/distributed/stats")
    async def distributed_stats():
        from ..place.devices import list_devices

        devs = list_devices(nvml=getattr(ctx, "nvml", None))
        return {"devices": len(devs), "memory_total": sum(d.get("memory_total") or 0 for d in devs),
                "memory_free": sum(d.get("memory_free") or 0 for d in devs), "models": [m.model_id for m in ctx.registry.list()],
                "node": _membership().self_id, "peers_alive": len(_membership().alive())}

    @r.get("/api/distributed/recommend")
    async def distributed_recommend():
        """The largest model of the stores that fits what is free on this node's devices (weights plus a tenth
        for cache and workspaces)."""
        from ..place.devices import list_devices

        free = sum(d.get("memory_free") or 0 for d in list_devices(nvml=getattr(ctx, "nvml", None)))
        best = None
        if ctx.catalogue is not None:
            for e in ctx.catalogue.list():
                need = int(e.size * 1.1)
                if need <= free and (best is None or e.size > best.size):
                    best = e
        return {"memory_free": free, "model": best.name if best else None, "size": int(best.size) if best else 0}

    @r.post("/api/models/validate")
    async def models_validate(req: Request):
        """Checks a model's file: tensor table, payload sizes, required metadata (`loken validate`)."""
        from ..cli.loken import validate_gguf

        body = await req.json()
        path = _model_file(body)
        try:
            return validate_gguf(path)
        except (OSError, ValueError) as e:
            raise ApiError(400, f"cannot read {path}: {e}")

    @r.post("/api/models/repair")
    async def models_repair(req: Request):
        """Validates, and fetches the model again from where its store entry came from when the file is damaged
        (nothing can be rebuilt from a damaged file itself)."""
        from ..cli.loken import validate_gguf

        body = await req.json()
        path = _model_file(body)
        try:
            rep = validate_gguf(path)
        except (OSError, ValueError) as e:
            rep = {"file": path, "ok": False, "problems": [str(e)]}
        rep["repaired"] = False
        if not rep["ok"]:
            rep["action"] = f"fetch it again: POST /api/pull {{\"model\": \"{body.get('model', '')}\"}}"
        return rep

    def _model_file(body: dict) -> str:
        import os

        name = body.get("path") or body.get("model")
        if not name:
            raise ApiError(400, "model (a name in the stores) or path is required")
        if os.path.exists(str(name)):
            return str(name)
        if ctx.catalogue is not None:
            e = ctx.catalogue.find(str(name))
            if e is not None and e.path:
                return e.path
        try:
            m = ctx.registry.get(str(name))
            if m.path:
                return m.path
        except ApiError:
            pass
        raise ApiError(404, f"no file is known for {name}")

    @r.get("/api/distributed/devices")
    async def devices():
        from ..place.devices import list_devices

        return {"devices": list_devices(nvml=getattr(ctx, "nvml", None))}

    @r.get("/metrics")
    async def metrics():
        g = {}
        for m in ctx.registry.list():
            a = m.engine.alloc
            tag = m.model_id.replace('"', "")
            g[f'loken_kv_blocks_free{{model="{tag}"}}'] = a.free_blocks()
            g[f'loken_engine_steps_total{{model="{tag}"}}'] = m.engine.stats.steps
            g[f'loken_preemptions_total{{model="{tag}"}}'] = m.engine.stats.preemptions
            g[f'loken_requests_running{{model="{tag}"}}'] = len(m.worker.tickets)
        d = ctx.gate.depth()
        g["loken_gate_active"] = d["active"]
        g["loken_gate_queued"] = d["queued"]
        return PlainTextResponse(ctx.metrics.render(g), media_type="text/plain; version=0.0.4")

    @r.post("/reset_prefix_cache")
    async def reset_prefix_cache():
        from starlette.concurrency import run_in_threadpool

        # the allocator belongs to the engine thread: the drop runs there, between two steps
        n = 0
        for m in ctx.registry.list():
            n += int(await run_in_threadpool(m.on_engine_thread, lambda eng: eng.reset_prefix_cache()) or 0)
        return {"status": "ok", "blocks_dropped": n}

    @r.get("/api/inflight")
    async def inflight():
        return {"requests": [dict(v, id=k) for k, v in list(ctx.inflight.items())], "gate": ctx.gate.depth()}

    @r.get("/api/stage_perf")
    async def stage_perf():
        return {"stages": ctx.metrics.stage_table()}

    @r.get("/api/layer_perf")
    async def layer_perf(rows: int = 1):
        from starlette.concurrency import run_in_threadpool

        out = {}
        for m in ctx.registry.list():
            try:
                out[m.model_id] = await run_in_threadpool(m.on_engine_thread, lambda eng: eng.layer_perf(rows))
            except Exception as e:
                out[m.model_id] = {"error": f"{type(e).__name__}: {e}"}
        return out

    @r.get("/api/models")
    async def api_models():
        return {"models": [m.info() for m in ctx.registry.list()]}

    @r.post("/load")
    async def load(req: Request):
        from starlette.concurrency import run_in_threadpool

        from ..engine.llm import LLM

        body = await req.json()
        path = body.get("model") or body.get("path")
        if not path:
            raise ApiError(400, "model (a GGUF path or a built-in shape name) is required")
        kw = {k: body[k] for k in ("requant", "kv_format", "max_seqs", "max_ctx", "num_blocks", "lora") if k in body}
        cat = getattr(ctx, "catalogue", None)
        entry = cat.resolve(path) if cat is not None else None
        if entry is not None:
            # a store name (`name:tag`, `owner/repo`, a GGUF's file name): the files it resolves to
            body.setdefault("id", entry.name)
            path = entry.path
        loader = getattr(ctx, "loader", None) or LLM.load
        evicted = []
        while True:
            try:
                llm = await run_in_threadpool(lambda: loader(path, model_id=body.get("id"), **kw))
                break
            except (KeyError, FileNotFoundError, IOError, ValueError) as e:
                raise ApiError(400, f"cannot load {path}: {e}")
            except (MemoryError, RuntimeError) as e:
                # out of device memory: unload the model that has been idle longest and try again
                # (`recover.rs` retry_on_oom_for / `vram_manager.rs` evict_idle_llm)
                if not isinstance(e, MemoryError) and "out of memory" not in str(e).lower():
                    raise
                # the memory authority trims the allocator's cache, asks the registered reclaimers, and if
                # none of them released anything unloads the model idle longest (`place/vram.py`)
                from ..place.vram import authority

                va = authority()
                va.set_evictor(ctx.registry.evict_idle)
                try:
                    rep = va.give_way()
                    gone, gave = list(rep.evicted), bool(rep.evicted or rep.reclaimed)
                except Exception:
                    victim = ctx.registry.evict_idle()
                    gone, gave = ([victim] if victim else []), bool(victim)
                if not gave:
                    raise ApiError(507, f"cannot load {path}: out of device memory and no idle model to unload")
                evicted += gone
        ctx.registry.add(llm, default=bool(body.get("default")))
        return {"status": "loaded", "model": llm.info(), "evicted": evicted}

    def _calibration_dir() -> str:
        import os as _os

        cat = getattr(ctx, "catalogue", None)
        base = cat.ollama.dirs[0] if cat is not None and cat.ollama.dirs else _os.path.expanduser("~/.loken")
        return _os.path.join(base, "calibrations")

    def _ndjson_job(job, stream: bool):
        """Runs `job(emit)` in a worker thread; with `stream` every emitted dict is one NDJSON line as it
        happens, otherwise the last one is the JSON reply.  A failure is the last line, with `error`."""
        import json as _json
        import queue
        import threading

        from starlette.concurrency import iterate_in_threadpool
        from starlette.responses import JSONResponse, StreamingResponse

        q: "queue.Queue" = queue.Queue()

        def run():
            try:
                job(q.put)
            except Exception as e:              # the reason travels to the client, not to a log
                q.put({"error": f"{type(e).__name__}: {e}"})
            q.put(None)

        threading.Thread(target=run, daemon=True).start()

        def lines():
            while True:
                ev = q.get()
                if ev is None:
                    return
                yield ev

        if stream:
            return StreamingResponse(iterate_in_threadpool((_json.dumps(ev) + "\n").encode() for ev in lines()),
                                     media_type="application/x-ndjson")
        last = {}
        for ev in lines():
            last = ev
        return JSONResponse(last, status_code=400 if "error" in last else 200)

    @r.post("/api/calibrate")
    async def calibrate(req: Request):
        """Records what the matrices of a checkpoint see on the given `texts` as the calibration `name`:
        per tensor, the mean square of the activations it multiplies and of its own values (the fp32
        forward of `models/reference.py`).  `model` is a path or a store name; `tokens` bounds the pass
        (default 4096), `excerpt` the characters taken from each text, `rows` how many activation rows per
        tensor are kept beside the record for error-compensated conversion (default 64, 0 for none)."""
        from starlette.concurrency import run_in_threadpool

        body = await req.json()
        name, model, texts = body.get("name"), body.get("model"), body.get("texts") or []
        if not name or not model or not texts or not all(isinstance(t, str) for t in texts):
            raise ApiError(400, "name, model and texts (a list of strings) are required")
        if "/" in name or name.startswith("."):
            raise ApiError(400, "a calibration name is a plain file name")
        cat = getattr(ctx, "catalogue", None)
        entry = cat.resolve(model) if cat is not None else None
        path = entry.path if entry is not None else model
        excerpt, budget = int(body.get("excerpt") or 4000), int(body.get("tokens") or 4096)

        def job(emit):
            import os as _os

            import torch as _torch

            from ..formats.requant import calibrate as _cal, write_calibration
            from ..models.loader import load_gguf
            from ..text.tokenizer import from_gguf_meta

            emit({"status": "loading"})
            w, meta = load_gguf(path, _torch.device("cuda" if _torch.cuda.is_available() else "cpu"), requant="bf16")
            tk = from_gguf_meta(meta)
            lists = [tk.encode(t[:excerpt], True) for t in texts]
            emit({"status": "recording", "texts": len(lists), "tokens": min(budget, sum(len(x) for x in lists))})
            keep = int(body.get("rows", 64) or 0)
            kept = {} if keep > 0 else None
            stats = _cal(w, lists, max_tokens=budget, keep_rows=keep, rows_out=kept)
            out = _os.path.join(_calibration_dir(), name + ".json")
            rec = write_calibration(out, name, model, stats, len(lists), min(budget, sum(len(x) for x in lists)), rows=kept)
            emit({"status": "success", "calibration": name, "path": out, "tensors": len(rec["stats"]),
                  "rows": keep if kept else 0})

        return await run_in_threadpool(_ndjson_job, job, body.get("stream", True) is not False)

    @r.post("/api/convert")
    async def convert(req: Request):
        """Converts a checkpoint (`model`: a GGUF path or a store name) into the model `name` (`name:tag`) of
        the first Ollama store, re-encoded as `format` (q8_0, q4_k_m, q4_k, q6_k, mxfp4, bf16, f16); a
        `calibration` recorded by /api/calibrate lifts the most sensitive tensors one step.  `complete`
        finishes a conversion whose file was written but never registered."""
        import os as _os

        from starlette.concurrency import run_in_threadpool

        body = await req.json()
        name, model, fmt = body.get("name"), body.get("model"), (body.get("format") or "q4_k_m").lower()
        cat = getattr(ctx, "catalogue", None)
        if not name or (not model and not body.get("complete")):
            raise ApiError(400, "name (the model to create) and model (the checkpoint to convert) are required")
        if cat is None or not cat.ollama.dirs:
            raise ApiError(400, "no ollama_models_dir is configured to hold the converted model")
        from ..formats.requant import FORMATS

        if fmt not in FORMATS:
            raise ApiError(400, f"format must be one of {', '.join(FORMATS)}")
        work = _os.path.join(cat.ollama.dirs[0], "conversions")
        out = _os.path.join(work, name.replace("/", "_").replace(":", "_") + f".{fmt}.gguf")
        cal = body.get("calibration")
        cal_path = _os.path.join(_calibration_dir(), cal + ".json") if cal else None
        if cal_path and not _os.path.exists(cal_path):
            raise ApiError(404, f"no calibration named {cal}")
        entry = cat.resolve(model) if model else None
        src = entry.path if entry is not None else model

        def job(emit):
            from ..formats.requant import requantize_gguf

            _os.makedirs(work, exist_ok=True)
            if not (body.get("complete") and _os.path.exists(out)):
                if not src or not _os.path.isfile(src):
                    raise FileNotFoundError(f"{model}: not a GGUF file or a store name that resolves to one")
                emit({"status": "converting", "format": fmt})
                state = {"last": 0}

                def progress(tensor, done, total):
                    if done == total or done - state["last"] >= max(1, total // 50):
                        state["last"] = done
                        emit({"status": "converting", "completed": done, "total": total})

                rep = requantize_gguf(src, out, fmt, calibration=cal_path, progress=progress)
            else:
                rep = {"output": out, "format": fmt, "resumed": True}
            emit({"status": "registering"})
            e = cat.ollama.create(name, out)
            _os.remove(out)                       # the store holds the blob (hard link or copy)
            emit(dict(rep, status="success", model=e.name, size=e.size))

        return await run_in_threadpool(_ndjson_job, job, body.get("stream", True) is not False)

    @r.post("/api/pipeline/tail")
    async def pipeline_tail(req: Request):
        """Runs this node as one segment of a pipeline across nodes: layers `from` .. `to` of `model`,
        relaying to `next` ("host:port" of the following segment) unless this is the last one.  Answers
        the wire port the upstream segment (or the head) connects to.  A head calls this, not an
        operator.  A second call for the same model and range answers the segment that already runs."""
        from starlette.concurrency import run_in_threadpool

        body = await req.json()
        model, lo, hi = body.get("model"), body.get("from"), body.get("to")
        if not model or lo is None or hi is None or int(lo) < 0 or int(hi) <= int(lo):
            raise ApiError(400, "model, from and to (a non-empty layer range) are required")
        lo, hi = int(lo), int(hi)
        key = (model, lo, hi, body.get("next"))
        segs = ctx.__dict__.setdefault("segments", {})
        if key in segs:
            srv, run = segs[key]
            return {"status": "running", "port": srv.addr[1], "host": srv.addr[0], **run.status()}

        def start():
            import torch as _torch

            from ..cluster.pipeline import SegmentLink, SegmentServer
            from ..cluster.segment import SegmentRunner
            from ..models.loader import load_gguf, peek_config

            cat = getattr(ctx, "catalogue", None)
            entry = cat.resolve(model) if cat is not None else None
            path = entry.path if entry is not None else model
            shape = peek_config(path)
            if hi > shape.n_layers:
                raise ValueError(f"{model} has {shape.n_layers} layers; the range ends at {hi}")
            last = hi == shape.n_layers and not body.get("next")
            dev = _torch.device("cuda", _torch.cuda.current_device())
            import os as _os

            if _os.path.exists(path):
                w, _meta = load_gguf(path, dev, layer_range=(lo, hi), kv_format=body.get("kv_format"))
            else:
                from ..models.weights import random_weights

                w = random_weights(shape, dev, seed=int(body.get("seed", 0)), layer_range=(lo, hi))
            run = SegmentRunner(w.cfg, w, lo, hi, last=last, device=dev, max_ctx=int(body.get("max_ctx", 8192)),
                                max_requests=int(body.get("max_requests", 16)))
            nxt = None
            if body.get("next"):
                h, _, pt = str(body["next"]).rpartition(":")
                nxt = SegmentLink(h or "127.0.0.1", int(pt))
            srv = SegmentServer(run.run, cut=run.cut, host=body.get("listen", "0.0.0.0"), port=int(body.get("port", 0)),
                                next_hop=nxt).start()
            segs[key] = (srv, run)
            return srv, run

        try:
            srv, run = await run_in_threadpool(start)
        except (ValueError, FileNotFoundError, KeyError) as e:
            raise ApiError(400, f"cannot start the segment: {e}")
        return {"status": "started", "port": srv.addr[1], "host": srv.addr[0], **run.status()}

    @r.post("/api/cluster/generate")
    async def cluster_generate(req: Request):
        """Tokens for a peer that keeps the text layer of the request: the engine's step outputs as JSON lines
        (`cluster/forward.py`).  Never forwarded again: this route submits to this node's engine."""
        from fastapi.responses import StreamingResponse

        from ..cluster import forward

        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        try:
            ids = [int(t) for t in body["prompt"]]
            params = forward.params_from_wire(body.get("params") or {})
        except (KeyError, TypeError, ValueError) as e:
            raise ApiError(400, f"bad forwarded request: {e}")
        if not ids or len(ids) >= llm.engine.max_ctx:
            raise ApiError(400, "the forwarded prompt is empty or longer than the context window")
        gen = forward.serve_raw(llm, ids, params, node_id=_membership().self_id, timeout_s=ctx.settings.request_timeout_s)
        return StreamingResponse(gen, media_type="application/x-ndjson")

    def _plan_inputs(body: dict) -> dict:
        """A plan over this node and the peers it sees, from what each measured and published for `model`
        (`POST /api/cluster/measure`): a layer's time and bytes, the room on the cards, the timed round trips."""
        model = str(body["model"])
        mine = ctx.layer_cost.get(model)
        if mine is None:
            raise ApiError(409, f"this node has no layer cost for {model}: POST /api/cluster/measure first")
        m = _membership()
        nodes = [{"id": m.self_id, "bytes": body.get("self_bytes", _card_bytes_free()), "layer_ms": mine["card_ms"],
                  "host_ms": mine.get("host_ms", 0.0)}]
        links = []
        for p in m.alive():
            c = p.layer_cost.get(model)
            if c is None or p.rtt_ms is None:
                continue          # a peer that has not measured the model, or was never timed, takes no layers
            nodes.append({"id": p.node_id, "bytes": p.card_bytes_free, "layer_ms": c["card_ms"], "host_ms": c.get("host_ms", 0.0)})
            links.append({"from": m.self_id, "to": p.node_id, "ms": p.rtt_ms / 2.0})
        mine_links = list(links)
        for i, a in enumerate(mine_links):
            for b in mine_links[i + 1:]:
                # two peers were never timed against each other from here: priced as the way through this node
                links.append({"from": a["to"], "to": b["to"], "ms": a["ms"] + b["ms"]})
        return dict(body, nodes=nodes, links=links, layers=int(mine.get("layers", 0)), layer_bytes=int(mine["card_bytes"]),
                    objective=body.get("objective", "time"), first=m.self_id)

    @r.post("/api/cluster/plan")
    async def cluster_plan(req: Request):
        """Where to cut a layer stack over nodes (`cluster/cut_plan.py: plan_from_request` documents the body).
        Nodes that are not named take their link prices from what this node has measured about its peers.
        409 when no arrangement fits: the caller picks fewer layers, another format or one node."""
        from ..cluster.cut_plan import plan_from_request

        body = await req.json()
        if not body.get("nodes") and body.get("model"):
            body = _plan_inputs(body)
        try:
            plan = plan_from_request(body)
        except (ValueError, KeyError, TypeError) as e:
            raise ApiError(400, f"cannot plan: {e}")
        if plan is None:
            raise ApiError(409, "no arrangement of these layers fits these nodes over these links")
        return plan.to_json()

    @r.post("/api/layers/swap")
    async def layers_swap(req: Request):
        """Attach or detach adapters on a loaded model without reloading it.  `adapters` is the set the model
        should end up with: PEFT directories, each optionally with a `weight` (`[]` detaches everything).  The
        weights are rewritten in place (`models/lora.py: AdapterSet`), cached prompt rows computed under the
        old weights are dropped, and the call waits for nothing: it answers 409 while requests are in flight."""
        from starlette.concurrency import run_in_threadpool

        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        wanted = {}
        for a in body.get("adapters") or []:
            path, wt = (a, 1.0) if isinstance(a, str) else (a.get("path"), a.get("weight", 1.0))
            if not path:
                raise ApiError(400, "every adapter names its path")
            wanted[str(path)] = float(wt)

        def work(eng):
            from ..models.lora import AdapterSet

            e = getattr(eng, "_e", eng)
            if eng.has_work():
                raise RuntimeError("busy")
            mw = getattr(e, "weights", None)
            if mw is None:
                raise ValueError("this engine exposes no weights to adapt")
            if getattr(e, "adapters", None) is None:
                e.adapters = AdapterSet(mw)
            rep = e.adapters.apply(wanted)
            rep["prefix_blocks_dropped"] = int(e.alloc.reset_prefix_cache() or 0)
            if getattr(e, "disk", None) is not None:
                e.disk.rescope("|".join(f"{p}={w}" for p, w in sorted(wanted.items())))
            return rep

        try:
            return await run_in_threadpool(llm.on_engine_thread, work)
        except RuntimeError as e:
            if str(e) == "busy":
                raise ApiError(409, "requests are in flight on this model; swap adapters when it is idle")
            raise ApiError(500, str(e))
        except (ValueError, OSError, KeyError) as e:
            raise ApiError(400, f"cannot swap adapters: {e}")

    @r.post("/api/swap")
    async def swap(req: Request):
        """Replace the resident model: the named one (or every resident language model when none is
        named) is unloaded first, so the new model has the card to itself, then the new one is loaded as
        the default.  A load that fails leaves the server without the old model: the reply says so."""
        import json as _json

        body = await req.json()
        if not (body.get("model") or body.get("path")):
            raise ApiError(400, "model (what to load) is required")
        names = [body["replace"]] if body.get("replace") else [m.model_id for m in ctx.registry.list()]
        gone = [n for n in names if ctx.registry.remove(n)]
        from ..place.vram import authority

        authority().residency_epoch += len(gone)
        body["default"] = True

        class _Again:
            async def json(self_inner):
                return body

        try:
            out = await load(_Again())
        except ApiError as e:
            raise ApiError(e.status, f"{e.message} (unloaded: {_json.dumps(gone)})")
        out["status"] = "swapped"
        out["unloaded"] = gone
        return out

    @r.delete("/api/models/{model_id:path}")
    async def unload(model_id: str):
        if not ctx.registry.remove(model_id):
            raise ApiError(404, f"model '{model_id}' not found", "not_found_error")
        return {"status": "unloaded", "model": model_id}

    @r.get("/api/draft/status")
    async def draft_status():
        out = {}
        for m in ctx.registry.list():
            sp = getattr(m.engine, "spec", None)
            out[m.model_id] = sp.status() if sp is not None else {"attached": False}
        return out

    @r.post("/api/draft/attach")
    async def draft_attach(req: Request):
        from starlette.concurrency import run_in_threadpool

        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        from ..serve.speculative import attach_draft

        try:
            st = await run_in_threadpool(lambda: attach_draft(llm, body.get("draft"), k=int(body.get("k", 4)),
                                                              method=body.get("method", "model")))
        except (KeyError, ValueError, IOError) as e:
            raise ApiError(400, str(e))
        return st

    @r.post("/api/draft/detach")
    async def draft_detach(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        from ..serve.speculative import detach_draft

        return detach_draft(llm)

    return r


def create_app(registry: ModelRegistry, settings: Optional[ServerSettings] = None) -> FastAPI:
    ctx = ServerContext(registry, settings)
    app = FastAPI(title="loken_b200", version=VERSION, docs_url=None, redoc_url=None)
    app.state.ctx = ctx

    @app.middleware("http")
    async def layers(request: Request, call_next):
        path = request.url.path
        rid = request.headers.get("x-request-id") or new_request_id()
        try:
            cl = request.headers.get("content-length")
            # a model blob is streamed to disk, never held in memory: the body limit is for JSON bodies
            if cl and int(cl) > ctx.settings.max_body_bytes and not path.startswith("/api/blobs/"):
                raise ApiError(413, f"request body is limited to {ctx.settings.max_body_bytes} bytes")
            key = None
            if path not in OPEN_PATHS and request.method != "OPTIONS":
                key = ctx.auth.check(request.headers)
                ctx.limiter.check(key or (request.client.host if request.client else "anon"))
            request.state.api_key = key
            request.state.request_id = rid
            resp = await call_next(request)
        except ApiError as e:
            resp = _error_response(path, e)
        resp.headers.setdefault("x-request-id", rid)
        origin = request.headers.get("origin")
        allowed = ctx.settings.allowed_origins
        if origin and (not allowed or "*" in allowed or origin in allowed):
            resp.headers["access-control-allow-origin"] = origin if allowed and "*" not in allowed else "*"
            resp.headers["access-control-allow-headers"] = "authorization, content-type, x-api-key, x-request-id"
            resp.headers["access-control-allow-methods"] = "GET, POST, DELETE, OPTIONS"
        ctx.metrics.observe_http(path, resp.status_code)
        return resp

    def _error_response(path: str, e: ApiError) -> JSONResponse:
        headers = {}
        if e.retry_after is not None:
            headers["retry-after"] = str(max(1, int(e.retry_after + 0.999)))
        return JSONResponse(error_body(path, e), status_code=e.status, headers=headers)

    @app.exception_handler(ApiError)
    async def api_error(request: Request, e: ApiError):
        return _error_response(request.url.path, e)

    @app.exception_handler(ValueError)
    async def value_error(request: Request, e: ValueError):
        return _error_response(request.url.path, ApiError(400, str(e)))

    @app.exception_handler(Exception)
    async def any_error(request: Request, e: Exception):
        return _error_response(request.url.path, ApiError(500, f"{type(e).__name__}: {e}", "server_error"))

    @app.options("/{rest:path}")
    async def preflight(rest: str):
        return PlainTextResponse("")

    app.include_router(ollama.router(ctx))
    app.include_router(openai.router(ctx))
    app.include_router(anthropic.router(ctx))
    app.include_router(ops_router(ctx))
    app.include_router(files.router(ctx, lambda: app))
    app.include_router(pooling.router(ctx))

    @app.post("/invocations")
    async def invocations(request: Request):
        # SageMaker's single route: the body's shape says which API it is
        body = await request.json()
        target = ("/v1/chat/completions" if "messages" in body else "/v1/completions" if "prompt" in body
                  else "/v1/embeddings" if "input" in body else None)
        if target is None:
            raise ApiError(400, "the body needs messages, prompt or input")
        for route in app.router.routes:
            if getattr(route, "path", None) == target and "POST" in getattr(route, "methods", ()):
                return await route.endpoint(request)
        raise ApiError(404, f"{target} is not served")

    def _endpoint(path: str):
        for route in app.router.routes:
            if getattr(route, "path", None) == path and "POST" in getattr(route, "methods", ()):
                return route.endpoint
        raise ApiError(404, f"{path} is not served")

    @app.post("/v1/chat/completions/batch")
    async def chat_batch(request: Request):
        # `messages` is a list of conversations; each is answered as its own chat completion and comes
        # back as one choice, in order
        import json as _json

        body = await request.json()
        convs = body.get("messages")
        if not isinstance(convs, list) or not convs or not all(isinstance(c, list) for c in convs):
            raise ApiError(400, "messages must be a list of conversations")
        if body.get("stream") or body.get("tools") or int(body.get("n") or 1) > 1:
            raise ApiError(400, "a batch of conversations takes no stream, no tools and n = 1")
        chat = _endpoint("/v1/chat/completions")
        choices, usage, first = [], {"prompt_tokens": 0, "completion_tokens": 0, "total_tokens": 0}, None
        for i, conv in enumerate(convs):
            sub = dict(body, messages=conv)
            scope = dict(request.scope)
            one = Request(scope)
            one._json = sub                    # the handler reads the parsed body from the request
            one.state.api_key = getattr(request.state, "api_key", None)
            resp = await chat(one)
            j = _json.loads(resp.body)
            first = first or j
            ch = j["choices"][0]
            ch["index"] = i
            choices.append(ch)
            for k in usage:
                usage[k] += j.get("usage", {}).get(k, 0)
        return JSONResponse(dict(first, choices=choices, usage=usage))

    @app.post("/v1/moderations")
    async def moderations():
        raise ApiError(501, "no moderation classifier is configured on this server", "not_implemented")

    @app.post("/v1/forecast")
    async def forecast():
        raise ApiError(501, "no forecaster checkpoint is loaded on this server", "not_implemented")

    return app


def serve(registry: ModelRegistry, settings: Optional[ServerSettings] = None, cluster=None, catalogue=None):
    """`cluster`: the configuration's [cluster] section; with peers listed or discovery on, a gossip loop
    runs beside the server (`cluster/gossip.py`, `cluster/discovery.py`).  `catalogue`: the model stores (`store/catalogue.py`) behind
    listings, pulls, copies and deletes, and behind loads by name."""
    import uvicorn

    s = settings or ServerSettings()
    app = create_app(registry, s)
    app.state.ctx.catalogue = catalogue
    loop, disco = None, None
    if cluster is not None and (getattr(cluster, "peers", None) or getattr(cluster, "discovery", False)):
        import socket

        from ..cluster.gossip import GossipLoop
        from ..cluster.membership import Membership

        ctx = app.state.ctx
        node_id = cluster.node_id or socket.gethostname()
        me = cluster.listen or f"http://{s.host}:{s.port}"
        ctx.membership = Membership(node_id, suspect_phi=cluster.suspect_phi)
        loop = GossipLoop(ctx.membership, me, list(cluster.peers), ctx.describe,
                          interval_s=cluster.heartbeat_ms / 1000.0)
        if getattr(cluster, "discovery", False):
            # nodes heard on the multicast group join the gossip's address book beside the seeds
            from ..cluster.discovery import Announcement, Discovery

            try:
                disco = Discovery(Announcement(cluster.name, node_id, me),
                                  on_peer=lambda nid, ep: loop.addrs.setdefault(ep, ep)).start()
            except OSError as e:
                print(f"loken: multicast discovery is off ({e}); the seed list still applies", flush=True)
        loop.start()
    import threading

    stop_reaper = threading.Event()

    def reaper():
        # the keep-alive: checked a few times per period, never more often than every five seconds
        ka = app.state.ctx.settings.keep_alive_s
        period = max(5.0, (ka if ka and ka > 0 else 60.0) / 4.0)
        while not stop_reaper.wait(period):
            try:
                app.state.ctx.reap_idle()
            except Exception as e:
                print(f"loken: keep-alive check failed: {e}", flush=True)

    if s.keep_alive_s is not None and s.keep_alive_s >= 0:
        threading.Thread(target=reaper, name="keep-alive", daemon=True).start()
    try:
        uvicorn.run(app, host=s.host, port=s.port, log_level="info")
    finally:
        stop_reaper.set()
        if loop is not None:
            loop.stop()
        if disco is not None:
            disco.stop()
