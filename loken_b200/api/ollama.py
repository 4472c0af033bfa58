"""Ollama-compatible routes: /api/version, /api/tags, /api/show, /api/ps, /api/chat, /api/generate
(`src/api/handlers/mod.rs:2864-2935`, `docs/API.md:12-31`).  Streams are newline-delimited JSON
objects; the last one carries `done: true`, the done reason and the timing / count fields in
nanoseconds."""
from __future__ import annotations

import datetime
import json
import time
from typing import Iterator

from fastapi import APIRouter, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse
from starlette.concurrency import iterate_in_threadpool, run_in_threadpool

from ..text.chat import parse_tool_calls
from ..text.stream import split_thinking
from .common import ApiError, check_messages, new_request_id, params_from_ollama
from .context import VERSION, ServerContext


def _now() -> str:
    return datetime.datetime.now(datetime.timezone.utc).strftime("%Y-%m-%dT%H:%M:%S.%fZ")


def _details(llm) -> dict:
    cfg = llm.cfg
    n = cfg.param_count()
    size = f"{n / 1e9:.1f}B" if n >= 1e9 else f"{n / 1e6:.0f}M"
    return {"format": "gguf", "family": cfg.arch, "families": [cfg.arch], "parameter_size": size,
            "quantization_level": cfg.weight_format.upper()}


def _default_opener():
    from ..store.download import requests_opener

    return requests_opener


def router(ctx: ServerContext) -> APIRouter:
    r = APIRouter()

    @r.get("/")
    async def root():
        return PlainTextResponse("Ollama is running")

    @r.get("/api/version")
    async def version():
        return {"version": VERSION}

    def _catalogue():
        return getattr(ctx, "catalogue", None)

    @r.get("/api/tags")
    async def tags():
        """Loaded models, then what the model stores hold (Ollama manifests, the Hugging Face cache,
        bare GGUF files), each listed once; then the models resident on the peers this node sees, each
        under its `node` (`docs/CLUSTER.md:57` of the reference)."""
        out, seen = [], set()
        for m in ctx.registry.list():
            seen.add(m.model_id)
            out.append({"name": m.model_id, "model": m.model_id,
                        "modified_at": datetime.datetime.fromtimestamp(m.loaded_at, datetime.timezone.utc).isoformat(),
                        "size": int(m.cfg.param_count()), "digest": "", "details": _details(m)})
        cat = _catalogue()
        for e in (cat.list() if cat is not None else []):
            if e.name in seen:
                continue
            out.append({"name": e.name, "model": e.name, "size": int(e.size), "digest": e.digest.split(":")[-1],
                        "modified_at": datetime.datetime.fromtimestamp(e.modified or 0, datetime.timezone.utc).isoformat(),
                        "details": {"format": "gguf" if e.source != "huggingface" else "safetensors",
                                    "family": "", "parameter_size": "", "quantization_level": ""}})
        m = getattr(ctx, "membership", None)
        for p in (m.alive() if m is not None else []):
            for name in p.models:
                out.append({"name": name, "model": name, "node": p.node_id, "endpoint": p.addr, "size": 0, "digest": "",
                            "details": {"format": "", "family": "", "parameter_size": "", "quantization_level": ""}})
        return {"models": out}

    @r.post("/api/show")
    async def show(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model") or body.get("name"))
        cfg = llm.cfg
        a = cfg.arch
        info = {"general.architecture": a, "general.parameter_count": cfg.param_count(),
                f"{a}.context_length": cfg.context_length, f"{a}.embedding_length": cfg.hidden,
                f"{a}.block_count": cfg.n_layers, f"{a}.attention.head_count": cfg.n_q,
                f"{a}.attention.head_count_kv": cfg.n_kv}
        caps = ["completion"]
        if llm.tokenizer.chat_template and "tools" in llm.tokenizer.chat_template:
            caps.append("tools")
        return {"modelfile": f"FROM {llm.path or llm.model_id}\n", "parameters": "", "template":
                llm.tokenizer.chat_template or "", "details": _details(llm), "model_info": info,
                "capabilities": caps}

    @r.get("/api/ps")
    async def ps():
        out = []
        for m in ctx.registry.list():
            out.append({"name": m.model_id, "model": m.model_id, "size": int(m.cfg.param_count()),
                        "details": _details(m), "size_vram": int(m.cfg.param_count()),
                        "expires_at": "0001-01-01T00:00:00Z", "context_length": m.engine.max_ctx})
        return {"models": out}

    def _final(llm, t0, t_first, n_in, n_out, reason, cached: int = 0) -> dict:
        now = time.perf_counter()
        return {"prompt_eval_cached_count": int(cached), "done": True, "done_reason": "length" if reason == "length" else "stop",
                "total_duration": int((now - t0) * 1e9), "load_duration": 0, "prompt_eval_count": n_in,
                "prompt_eval_duration": int(((t_first or now) - t0) * 1e9), "eval_count": n_out,
                "eval_duration": int((now - (t_first or now)) * 1e9)}

    def _run(llm, ids, params, rid, scope, stream: bool, wrap, tools=None):
        """Common body of chat / generate.  `wrap(text, thinking, calls)` makes the dialect's payload."""
        t0 = time.perf_counter()

        if stream:
            def gen() -> Iterator[bytes]:
                t_first, n_out, reason, held = None, 0, None, ""
                for ev in ctx.run(llm, ids, params, request_id=rid, scope=scope):
                    if ev.error:
                        yield (json.dumps({"error": ev.error}) + "\n").encode()
                        return
                    if t_first is None and ev.token_ids:
                        t_first = time.perf_counter()
                    n_out += len(ev.token_ids)
                    reason = ev.finish_reason or reason
                    if tools:
                        held += ev.text          # tool calls need the whole answer; emitted with `done`
                        continue
                    if ev.text:
                        yield (json.dumps({"model": llm.model_id, "created_at": _now(), **wrap(ev.text, "", []),
                                           "done": False}, ensure_ascii=False) + "\n").encode()
                last = {"model": llm.model_id, "created_at": _now()}
                if tools:
                    thinking, answer = split_thinking(held)
                    answer, calls = parse_tool_calls(answer)
                    last.update(wrap(answer, thinking, calls))
                else:
                    last.update(wrap("", "", []))
                last.update(_final(llm, t0, t_first, len(ids), n_out, reason))
                yield (json.dumps(last, ensure_ascii=False) + "\n").encode()

            return StreamingResponse(iterate_in_threadpool(gen()), media_type="application/x-ndjson",
                                     headers={"x-request-id": rid})

        def run_all():
            text, t_first, n_out, reason = "", None, 0, None
            for ev in ctx.run(llm, ids, params, request_id=rid, scope=scope):
                if ev.error:
                    raise ApiError(500, ev.error, "server_error")
                if t_first is None and ev.token_ids:
                    t_first = time.perf_counter()
                text += ev.text
                n_out += len(ev.token_ids)
                reason = ev.finish_reason or reason
            thinking, answer = split_thinking(text)
            calls = []
            if tools:
                answer, calls = parse_tool_calls(answer)
            out = {"model": llm.model_id, "created_at": _now(), **wrap(answer, thinking, calls)}
            out.update(_final(llm, t0, t_first, len(ids), n_out, reason))
            return out

        return run_all

    @r.post("/api/chat")
    async def chat(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        check_messages(body.get("messages"))
        params = params_from_ollama(body.get("options"), body, llm)
        tools = body.get("tools")
        ids = await run_in_threadpool(llm.prompt_ids, None, body["messages"], tools, params)
        rid = new_request_id("ollama")

        def wrap(text, thinking, calls):
            msg = {"role": "assistant", "content": text}
            if thinking:
                msg["thinking"] = thinking
            if calls:
                msg["tool_calls"] = [{"function": {"name": c["function"]["name"],
                                                   "arguments": json.loads(c["function"]["arguments"] or "{}")}}
                                     for c in calls]
            return {"message": msg}

        res = _run(llm, ids, params, rid, getattr(req.state, "api_key", None), body.get("stream", True), wrap, tools)
        if isinstance(res, StreamingResponse):
            return res
        return JSONResponse(await run_in_threadpool(res), headers={"x-request-id": rid})

    @r.post("/api/generate")
    async def generate(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        params = params_from_ollama(body.get("options"), body, llm)
        prompt = body.get("prompt", "")
        if not prompt and not body.get("raw"):
            # an empty prompt is a load / keep-alive probe
            return {"model": llm.model_id, "created_at": _now(), "response": "", "done": True, "done_reason": "load"}
        if body.get("raw"):
            ids = llm.prompt_ids(prompt, params=params)
        else:
            msgs = []
            if body.get("system"):
                msgs.append({"role": "system", "content": body["system"]})
            msgs.append({"role": "user", "content": prompt})
            ids = await run_in_threadpool(llm.prompt_ids, None, msgs, None, params)
        rid = new_request_id("ollama")

        def wrap(text, thinking, calls):
            out = {"response": text}
            if thinking:
                out["thinking"] = thinking
            return out

        res = _run(llm, ids, params, rid, getattr(req.state, "api_key", None), body.get("stream", True), wrap)
        if isinstance(res, StreamingResponse):
            return res
        return JSONResponse(await run_in_threadpool(res), headers={"x-request-id": rid})

    @r.post("/api/embed")
    async def embed(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        inp = body.get("input")
        items = inp if isinstance(inp, list) else [inp]
        t0 = time.perf_counter()
        out, total = [], 0
        for it in items:
            vec, n = await run_in_threadpool(llm.embed, str(it))
            out.append(vec)
            total += n
        return {"model": llm.model_id, "embeddings": out, "total_duration": int((time.perf_counter() - t0) * 1e9),
                "prompt_eval_count": total}

    @r.post("/api/embeddings")
    async def embeddings_legacy(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        vec, _ = await run_in_threadpool(llm.embed, str(body.get("prompt", "")))
        return {"embedding": vec}

    @r.post("/api/push")
    async def push():
        raise ApiError(403, "pushing models is not supported")

    @r.post("/api/copy")
    async def copy(req: Request):
        body = await req.json()
        src, dst = body.get("source"), body.get("destination")
        if not src or not dst:
            raise ApiError(400, "source and destination are required")
        cat = _catalogue()
        if cat is not None and cat.ollama.find(src) is not None:
            cat.ollama.copy(src, dst)            # stays in the directory of its source, beside the blobs it shares
            return JSONResponse({}, status_code=200)
        ctx.registry.alias(src, dst)
        return JSONResponse({}, status_code=200)

    @r.delete("/api/delete")
    async def delete(req: Request):
        body = await req.json()
        name = body.get("model") or body.get("name")
        if not name:
            raise ApiError(400, "model is required")
        dropped = ctx.registry.drop(name)
        cat = _catalogue()
        removed = cat.delete(name) if cat is not None else 0         # every copy, in every store directory
        if not dropped and not removed:
            raise ApiError(404, f"model '{name}' not found")
        return JSONResponse({}, status_code=200)

    @r.post("/api/create")
    async def create(req: Request):
        # a new name for a loaded model; sampling defaults of a Modelfile are not stored
        body = await req.json()
        name, base = body.get("model") or body.get("name"), body.get("from")
        if not name or not (base or body.get("files")):
            raise ApiError(400, "model, and from (a model here) or files (uploaded blobs), are required")
        if body.get("adapters"):
            raise ApiError(400, "adapters are merged at load (POST /load with lora); a model is not created from them")
        cat = _catalogue()
        files = body.get("files") or {}
        if files:
            # a model from a blob uploaded through /api/blobs: `files` maps a file name to its digest
            if cat is None:
                raise ApiError(400, "no model store is configured to build a model in")
            ggufs = [(fn, dg) for fn, dg in files.items() if str(fn).endswith(".gguf")] or list(files.items())
            bp = _find_blob(cat, str(ggufs[0][1]))
            if bp is None:
                raise ApiError(400, f"blob {ggufs[0][1]} was not uploaded (HEAD /api/blobs/<digest> says so)")
            cat.ollama.create(name, bp, template=body.get("template"), system=body.get("system"),
                              params=body.get("parameters") or None, license=body.get("license"))
            return {"status": "success"}
        src = cat.resolve(base) if cat is not None else None
        if src is not None and src.source in ("ollama", "gguf"):
            # a new manifest over the same weights blob, with its own template / system prompt / parameters
            cat.ollama.create(name, src.path, template=body.get("template") or src.template,
                              system=body.get("system") or src.system,
                              params=body.get("parameters") or src.params or None, license=src.license)
            return {"status": "success"}
        ctx.registry.alias(base, name)
        return {"status": "success"}

    def _find_blob(cat, digest: str):
        import os

        from ..store.catalogue import blob_path

        for store in cat.ollama.dirs:
            bp = blob_path(store, digest)
            if os.path.exists(bp):
                return bp
        return None

    def _check_digest(digest: str) -> str:
        import re

        if not re.fullmatch(r"sha256:[0-9a-f]{64}", digest or ""):
            raise ApiError(400, "a blob is named sha256:<64 hex digits>")
        return digest

    @r.head("/api/blobs/{digest}")
    async def blob_head(digest: str):
        """200 when the blob is in a store, 404 when it has to be uploaded."""
        from fastapi import Response

        cat = _catalogue()
        found = cat is not None and _find_blob(cat, _check_digest(digest)) is not None
        return Response(status_code=200 if found else 404)

    @r.post("/api/blobs/{digest}")
    async def blob_post(digest: str, req: Request):
        """Uploads a blob: streamed to a partial file in the first store, hashed as it arrives, kept only when
        the hash is the name it was sent under.  201 when stored, 200 when it was there already."""
        import hashlib
        import os

        from fastapi import Response

        from ..store.catalogue import blob_path

        cat = _catalogue()
        if cat is None or not cat.ollama.dirs:
            raise ApiError(400, "no model store is configured to keep blobs in")
        _check_digest(digest)
        if _find_blob(cat, digest) is not None:
            return Response(status_code=200)
        store = cat.ollama.dirs[0]
        os.makedirs(os.path.join(store, "blobs"), exist_ok=True)
        bp = blob_path(store, digest)
        tmp = bp + f".upload-{os.getpid()}"
        h = hashlib.sha256()
        try:
            with open(tmp, "wb") as f:
                async for chunk in req.stream():
                    h.update(chunk)
                    f.write(chunk)
            if "sha256:" + h.hexdigest() != digest:
                raise ApiError(400, "the uploaded bytes do not have the digest they were sent under")
            os.replace(tmp, bp)
        finally:
            if os.path.exists(tmp):
                os.remove(tmp)
        return Response(status_code=201)

    @r.post("/api/pull")
    async def pull(req: Request):
        # no registry is reachable from this server: a pull succeeds only for what is already here
        body = await req.json()
        name = body.get("model") or body.get("name")
        if not name:
            raise ApiError(400, "model is required")
        known = {m.model_id for m in ctx.registry.list()} | set(ctx.registry.aliases)
        cat = _catalogue()
        if name in known or (cat is not None and cat.resolve(name) is not None):
            return {"status": "success"}
        if cat is None:
            raise ApiError(404, f"model '{name}' is not on this server and no model store is configured; "
                                f"load a local file with POST /load")
        from ..store.download import pull_ollama

        def fetch_all():
            return [s for s in pull_ollama(cat.ollama, name, opener=getattr(ctx, "opener", None) or _default_opener())]

        try:
            states = await run_in_threadpool(fetch_all)
        except (IOError, OSError) as e:
            raise ApiError(502, f"pull of '{name}' failed: {e}")
        if body.get("stream", True) is False:
            return {"status": "success"}
        body_text = "".join(json.dumps(s) + "\n" for s in states)
        return PlainTextResponse(body_text, media_type="application/x-ndjson")

    return r
