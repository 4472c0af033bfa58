"""OpenAI-compatible routes: /v1/chat/completions, /v1/completions, /v1/models, /tokenize,
/detokenize (surface of `src/api/handlers/openai/`, `docs/API.md:32-55`, with the vLLM request
extensions of `docs/API.md:120-160`).  Streaming is server-sent events ending in `data: [DONE]`;
`stream_options.include_usage` adds a final usage chunk; reasoning goes to `reasoning_content`,
tool calls are parsed out of the text into `tool_calls`.
"""
from __future__ import annotations

import json
import base64
import struct
import time
from typing import Iterator, List

from fastapi import APIRouter, Request
from fastapi.responses import JSONResponse, StreamingResponse
from starlette.concurrency import iterate_in_threadpool, run_in_threadpool

from ..text.chat import parse_tool_calls
from ..text.stream import ThinkingSplitter, split_thinking
from .common import ApiError, Usage, check_messages, new_request_id, params_from_openai, prefill_comment
from .context import ServerContext


TOOL_MARKERS = ("<tool_call>", "[TOOL_CALLS]", "<|python_tag|>", "<|start|>", "<|channel|>")
MAX_MARKER = max(len(m) for m in TOOL_MARKERS)


def _sse(obj) -> bytes:
    return b"data: " + json.dumps(obj, ensure_ascii=False).encode() + b"\n\n"


def _lp_chat(llm, toks: List[int], lps, as_ids: bool = False) -> dict:
    """`as_ids` (`return_tokens_as_token_ids`): each token is written `token_id:<id>`, which survives tokens
    that are not valid text on their own."""
    name = (lambda i: f"token_id:{i}") if as_ids else (lambda i: llm.detokenize([i], skip_special=False))
    content = []
    for t, (lp, top) in zip(toks, lps or []):
        piece = llm.detokenize([t], skip_special=False)
        content.append({"token": name(t), "logprob": lp, "bytes": list(piece.encode()),
                        "top_logprobs": [{"token": name(i), "logprob": l,
                                          "bytes": list(llm.detokenize([i], skip_special=False).encode())}
                                         for i, l in top]})
    return {"content": content}


def _lp_text(llm, toks: List[int], lps, as_ids: bool = False) -> dict:
    name = (lambda i: f"token_id:{i}") if as_ids else (lambda i: llm.detokenize([i], skip_special=False))
    return {"tokens": [name(t) for t in toks], "token_logprobs": [lp for lp, _ in (lps or [])],
            "top_logprobs": [{name(i): l for i, l in top} for _, top in (lps or [])],
            "text_offset": []}


def _beam_request(body: dict, params, chat: bool):
    """Validates a `use_beam_search` request and returns (n, length_penalty, early_stopping)."""
    if body.get("stream"):
        raise ApiError(400, "beam search does not stream")
    if body.get("prompt_embeds") is not None:
        raise ApiError(400, "beam search does not take prompt_embeds")
    n = int(body.get("n") or 1)
    if body.get("best_of") and int(body["best_of"]) > n:
        raise ApiError(400, "beam search takes best_of up to n")
    if getattr(params, "grammar", None) is not None or body.get("response_format") or body.get("structured_outputs"):
        raise ApiError(400, "beam search does not take a structured output")
    if chat and body.get("tool_choice") == "required":
        raise ApiError(400, "beam search does not take a required tool call")
    if not 1 <= n <= 10:
        raise ApiError(400, "beam search takes n in 1..10")
    es = body.get("early_stopping", False)
    if es not in (True, False, "never"):
        raise ApiError(400, "early_stopping must be true, false or \"never\"")
    return n, float(body.get("length_penalty", 1.0)), es


def _beam_choices(llm, ids, params, body: dict, chat: bool):
    from ..serve.beam import run_beam_search

    n, lp, es = _beam_request(body, params, chat)
    beams = run_beam_search(llm, ids, n, params.max_tokens, lp, es, params.ignore_eos, params.stop_token_ids)
    eos = set(getattr(llm.engine, "eos", ()) or ()) | set(params.stop_token_ids)
    choices, n_out = [], 0
    for i, b in enumerate(beams):
        body_toks = b.tokens[:-1] if (b.finished_by == "stop" and b.tokens and b.tokens[-1] in eos) else b.tokens
        text = llm.detokenize(body_toks, params.skip_special_tokens)
        reason = "stop" if b.finished_by == "stop" else "length"
        ch = ({"index": i, "message": {"role": "assistant", "content": text}, "finish_reason": reason} if chat
              else {"index": i, "text": text, "finish_reason": reason})
        if params.logprobs:
            ch["logprobs"] = {"tokens": [llm.detokenize([t], False) for t in b.tokens], "token_logprobs": b.logprobs,
                              "cumulative_logprob": b.cum_logprob}
        choices.append(ch)
        n_out += len(b.tokens)
    return choices, n_out



def router(ctx: ServerContext) -> APIRouter:
    r = APIRouter()

    def model_card(llm) -> dict:
        return {"id": llm.model_id, "object": "model", "created": int(llm.loaded_at), "owned_by": "loken",
                "max_model_len": llm.engine.max_ctx, "root": llm.path or llm.model_id}

    @r.get("/v1/models")
    async def models():
        return {"object": "list", "data": [model_card(m) for m in ctx.registry.list()]}

    @r.get("/v1/models/{model_id:path}")
    async def model(model_id: str):
        return model_card(ctx.registry.get(model_id))

    @r.post("/tokenize")
    @r.post("/v1/tokenize")
    async def tokenize(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        if "messages" in body:
            check_messages(body["messages"])
            ids = llm.prompt_ids(messages=body["messages"], tools=body.get("tools"),
                                 add_generation_prompt=body.get("add_generation_prompt", True))
        else:
            ids = llm.tokenize(str(body.get("prompt", "")), add_special=body.get("add_special_tokens", True))
        out = {"count": len(ids), "max_model_len": llm.engine.max_ctx, "tokens": ids}
        if body.get("return_token_strs"):
            out["token_strs"] = [llm.detokenize([t], skip_special=False) for t in ids]
        return out

    @r.post("/detokenize")
    @r.post("/v1/detokenize")
    async def detokenize(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        return {"prompt": llm.detokenize([int(t) for t in body.get("tokens", [])], skip_special=False)}

    @r.post("/v1/embeddings")
    async def embeddings(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        inp = body.get("input")
        if inp is None:
            raise ApiError(400, "input is required")
        items = inp if isinstance(inp, list) and inp and not isinstance(inp[0], int) else [inp]
        pooling = body.get("pooling", "last")
        if pooling not in ("last", "mean"):
            raise ApiError(400, "pooling must be 'last' or 'mean'")
        fmt = body.get("encoding_format", "float")
        if fmt not in ("float", "base64"):
            raise ApiError(400, "encoding_format must be 'float' or 'base64'")
        data, total = [], 0
        for i, it in enumerate(items):
            vec, n = await run_in_threadpool(llm.embed, it, pooling)
            dims = body.get("dimensions")
            if dims:
                vec = vec[:int(dims)]
            if fmt == "base64":
                vec = base64.b64encode(struct.pack(f"<{len(vec)}f", *vec)).decode()
            data.append({"object": "embedding", "index": i, "embedding": vec})
            total += n
        return {"object": "list", "model": llm.model_id, "data": data,
                "usage": {"prompt_tokens": total, "total_tokens": total}}

    # ------------------------------------------------------------------ chat completions
    @r.post("/v1/chat/completions")
    async def chat(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        check_messages(body.get("messages"))
        params = params_from_openai(body, llm, chat=True)
        tools = body.get("tools") if body.get("tool_choice") != "none" else None
        kw = dict(body.get("chat_template_kwargs") or {})
        if body.get("documents") is not None:
            kw["documents"] = body["documents"]           # a variable of the model's template (retrieval-style templates read it)
        ids = await run_in_threadpool(
            llm.prompt_ids, None, body["messages"], tools, params,
            add_generation_prompt=body.get("add_generation_prompt", True),
            continue_final_message=body.get("continue_final_message", False), **kw)
        rid = new_request_id("chatcmpl")
        created = int(time.time())
        scope = getattr(req.state, "api_key", None)
        priority = body.get("priority", "interactive") if isinstance(body.get("priority"), str) else "interactive"
        include_reasoning = body.get("include_reasoning", True)

        if body.get("use_beam_search"):
            _beam_request(body, params, chat=True)
            choices, n_out = await run_in_threadpool(_beam_choices, llm, ids, params, body, True)
            return JSONResponse({"id": rid, "object": "chat.completion", "created": created, "model": llm.model_id,
                                 "choices": choices, "usage": Usage(len(ids), n_out).openai()},
                                headers={"x-request-id": rid})

        if body.get("stream"):
            include_usage = bool((body.get("stream_options") or {}).get("include_usage"))

            def gen() -> Iterator[bytes]:
                base = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": llm.model_id}
                yield _sse({**base, "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""},
                                                 "finish_reason": None}]})
                split = ThinkingSplitter()
                n_out, held, reason = 0, "", None
                tool_mode, sent_any = False, False
                figs, cached = None, 0
                try:
                    for ev in ctx.run(llm, ids, params, priority=priority, request_id=rid, scope=scope):
                        if ev.error:
                            yield _sse({"error": {"message": ev.error, "type": "server_error"}})
                            break
                        if ev.progress is not None:
                            yield prefill_comment(ev.progress)
                            continue
                        if ev.finished:
                            figs, cached = ev.figures, ev.cached_tokens
                        n_out += len(ev.token_ids)
                        for kind, text in split.push(ev.text) + (split.flush() if ev.finished else []):
                            if kind == "reasoning":
                                if include_reasoning:
                                    yield _sse({**base, "choices": [{"index": 0, "delta": {"reasoning_content": text},
                                                                     "finish_reason": None}]})
                                continue
                            if tools:
                                # buffer from the first call marker on; the calls are parsed at the end
                                held += text
                                if not tool_mode:
                                    cut = min([i for i in (held.find(m) for m in TOOL_MARKERS) if i >= 0] or [-1])
                                    if cut >= 0:
                                        tool_mode = True
                                        text, held = held[:cut], held[cut:]
                                    elif not sent_any and held.lstrip().startswith("{"):
                                        tool_mode = True
                                        text = ""
                                    else:
                                        keep = 0          # a tail that may still grow into a marker stays back
                                        for n in range(min(len(held), MAX_MARKER - 1), 0, -1):
                                            if any(m.startswith(held[-n:]) for m in TOOL_MARKERS):
                                                keep = n
                                                break
                                        text, held = held[:len(held) - keep], held[len(held) - keep:]
                                else:
                                    text = ""
                            sent_any = sent_any or bool(text.strip())
                            if text:
                                delta = {"content": text}
                                ch = {"index": 0, "delta": delta, "finish_reason": None}
                                if ev.logprobs and params.logprobs:
                                    ch["logprobs"] = _lp_chat(llm, ev.token_ids, ev.logprobs, bool(body.get("return_tokens_as_token_ids")))
                                yield _sse({**base, "choices": [ch]})
                        if ev.finished:
                            reason = ev.finish_reason
                    calls = []
                    if tools and held:
                        rest, calls = parse_tool_calls(held)
                        if calls:
                            yield _sse({**base, "choices": [{"index": 0, "finish_reason": None, "delta": {
                                "tool_calls": [dict(c, index=i) for i, c in enumerate(calls)]}}]})
                        elif rest:
                            yield _sse({**base, "choices": [{"index": 0, "delta": {"content": rest},
                                                             "finish_reason": None}]})
                    fin = "tool_calls" if calls else ("length" if reason == "length" else "stop")
                    yield _sse({**base, "choices": [{"index": 0, "delta": {}, "finish_reason": fin}]})
                    if include_usage:
                        yield _sse({**base, "choices": [],
                                    "usage": Usage(len(ids), n_out, cached, figures=figs).openai()})
                    yield b"data: [DONE]\n\n"
                except ApiError as e:
                    yield _sse({"error": {"message": e.message, "type": e.kind, "code": e.code}})

            return StreamingResponse(iterate_in_threadpool(gen()), media_type="text/event-stream",
                                     headers={"x-request-id": rid, "cache-control": "no-cache"})

        def run_all():
            from ..utils.figures import sum_figures

            choices = []
            total_out = 0
            fig_parts, cached = [], 0
            for idx in range(params.n):
                text, toks, lps, reason = "", [], [], None
                p = params
                if params.n > 1 and params.seed is not None:
                    import dataclasses

                    p = dataclasses.replace(params, seed=params.seed + idx)
                for ev in ctx.run(llm, ids, p, priority=priority, request_id=f"{rid}-{idx}", scope=scope):
                    if ev.error:
                        raise ApiError(500, ev.error, "server_error")
                    text += ev.text
                    toks += ev.token_ids
                    lps += ev.logprobs or []
                    reason = ev.finish_reason or reason
                    if ev.finished and ev.figures:
                        fig_parts.append(ev.figures)
                        cached = ev.cached_tokens
                reasoning, answer = split_thinking(text)
                calls = []
                if tools:
                    answer, calls = parse_tool_calls(answer)
                msg = {"role": "assistant", "content": answer if (answer or not calls) else None}
                if reasoning and include_reasoning:
                    msg["reasoning_content"] = reasoning
                if calls:
                    msg["tool_calls"] = calls
                ch = {"index": idx, "message": msg,
                      "finish_reason": "tool_calls" if calls else ("length" if reason == "length" else "stop")}
                if params.logprobs:
                    ch["logprobs"] = _lp_chat(llm, toks, lps, bool(body.get("return_tokens_as_token_ids")))
                choices.append(ch)
                total_out += len(toks)
            return {"id": rid, "object": "chat.completion", "created": created, "model": llm.model_id,
                    "choices": choices,
                    "usage": Usage(len(ids), total_out, cached, figures=sum_figures(fig_parts)).openai()}

        out = await run_in_threadpool(run_all)
        return JSONResponse(out, headers={"x-request-id": rid})

    # ------------------------------------------------------------------ text completions
    @r.post("/v1/completions")
    async def completions(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        params = params_from_openai(body, llm, chat=False)
        prompt = body.get("prompt", "")
        prompts = prompt if isinstance(prompt, list) and prompt and not isinstance(prompt[0], int) else [prompt]
        if body.get("suffix"):
            raise ApiError(400, "suffix (fill-in-the-middle) needs a model with FIM tokens")
        if body.get("prompt_embeds") is not None:
            # the prompt as embedding rows (loken's container, a torch.save archive read without unpickling,
            # or bare f32): one prompt per payload, answered in order
            from ..engine.llm import EmbedsPrompt
            from ..text.prompt_embeds import decode_request

            if body.get("use_beam_search"):
                raise ApiError(400, "beam search takes a text prompt, not prompt_embeds")
            try:
                arrays = decode_request(body["prompt_embeds"], llm.cfg.hidden, llm.engine.max_ctx)
            except ValueError as e:
                raise ApiError(400, str(e))
            id_lists = [EmbedsPrompt(a) for a in arrays]
            prompts = [None] * len(id_lists)
            params.echo = False
        else:
            id_lists = [llm.prompt_ids(p, params=params) for p in prompts]
        rid = new_request_id("cmpl")
        created = int(time.time())
        scope = getattr(req.state, "api_key", None)

        if body.get("use_beam_search"):
            _beam_request(body, params, chat=False)
            if len(id_lists) != 1:
                raise ApiError(400, "beam search takes one prompt")
            choices, n_out = await run_in_threadpool(_beam_choices, llm, id_lists[0], params, body, False)
            return JSONResponse({"id": rid, "object": "text_completion", "created": created, "model": llm.model_id,
                                 "choices": choices, "usage": Usage(len(id_lists[0]), n_out).openai()},
                                headers={"x-request-id": rid})

        if body.get("stream"):
            if len(id_lists) != 1:
                raise ApiError(400, "streaming takes one prompt")
            ids = id_lists[0]

            def gen():
                base = {"id": rid, "object": "text_completion", "created": created, "model": llm.model_id}
                n_out, reason, figs, cached = 0, None, None, 0
                if params.echo and isinstance(prompts[0], str):
                    yield _sse({**base, "choices": [{"index": 0, "text": prompts[0], "finish_reason": None}]})
                for ev in ctx.run(llm, ids, params, request_id=rid, scope=scope):
                    if ev.error:
                        yield _sse({"error": {"message": ev.error, "type": "server_error"}})
                        break
                    n_out += len(ev.token_ids)
                    reason = ev.finish_reason or reason
                    figs, cached = ev.figures or figs, max(cached, int(ev.cached_tokens or 0))
                    if ev.text or ev.finished:
                        ch = {"index": 0, "text": ev.text,
                              "finish_reason": None if not ev.finished else ("length" if reason == "length" else "stop")}
                        if params.logprobs and ev.logprobs:
                            ch["logprobs"] = _lp_text(llm, ev.token_ids, ev.logprobs, bool(body.get("return_tokens_as_token_ids")))
                        yield _sse({**base, "choices": [ch]})
                if (body.get("stream_options") or {}).get("include_usage"):
                    yield _sse({**base, "choices": [], "usage": Usage(len(ids), n_out, cached, figures=figs).openai()})
                yield b"data: [DONE]\n\n"

            return StreamingResponse(iterate_in_threadpool(gen()), media_type="text/event-stream",
                                     headers={"x-request-id": rid})

        def run_all():
            from ..utils.figures import sum_figures

            choices, n_in, n_out = [], 0, 0
            fig_parts, cached = [], 0
            for pi, ids in enumerate(id_lists):
                for k in range(params.n):
                    text, toks, lps, reason = "", [], [], None
                    for ev in ctx.run(llm, ids, params, request_id=f"{rid}-{pi}-{k}", scope=scope):
                        if ev.error:
                            raise ApiError(500, ev.error, "server_error")
                        text += ev.text
                        toks += ev.token_ids
                        lps += ev.logprobs or []
                        reason = ev.finish_reason or reason
                        cached = max(cached, int(ev.cached_tokens or 0))
                        if ev.figures:
                            fig_parts.append(ev.figures)
                    if params.echo and isinstance(prompts[pi], str):
                        text = prompts[pi] + text
                    ch = {"index": len(choices), "text": text,
                          "finish_reason": "length" if reason == "length" else "stop"}
                    if params.logprobs:
                        ch["logprobs"] = _lp_text(llm, toks, lps, bool(body.get("return_tokens_as_token_ids")))
                    choices.append(ch)
                    n_out += len(toks)
                n_in += len(ids)
            return {"id": rid, "object": "text_completion", "created": created, "model": llm.model_id,
                    "choices": choices, "usage": Usage(n_in, n_out, cached, figures=sum_figures(fig_parts)).openai()}

        return JSONResponse(await run_in_threadpool(run_all), headers={"x-request-id": rid})

    # ------------------------------------------------------------------ responses
    responses_store = {}

    def _responses_messages(body: dict):
        msgs = []
        if body.get("instructions"):
            msgs.append({"role": "system", "content": body["instructions"]})
        inp = body.get("input")
        if isinstance(inp, str):
            msgs.append({"role": "user", "content": inp})
        else:
            for it in inp or []:
                if it.get("type", "message") != "message":
                    continue
                c = it.get("content")
                if isinstance(c, list):
                    c = "".join(p_.get("text", "") for p_ in c if isinstance(p_, dict))
                msgs.append({"role": it.get("role", "user"), "content": c or ""})
        return msgs

    @r.post("/v1/responses")
    async def responses(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        msgs = _responses_messages(body)
        check_messages(msgs)
        b2 = dict(body)
        if body.get("max_output_tokens") is not None:
            b2["max_tokens"] = body["max_output_tokens"]
        fmt = (body.get("text") or {}).get("format") or {}
        if fmt.get("type") == "json_schema":
            b2["response_format"] = {"type": "json_schema", "json_schema": {"schema": fmt.get("schema", {})}}
        elif fmt.get("type") == "json_object":
            b2["response_format"] = {"type": "json_object"}
        params = params_from_openai(b2, llm, chat=True)
        ids = await run_in_threadpool(llm.prompt_ids, None, msgs, None, params)
        rid = new_request_id("resp")
        created = int(time.time())
        scope = getattr(req.state, "api_key", None)

        def envelope(status, text, n_out, reasoning=""):
            out = []
            if reasoning:
                out.append({"type": "reasoning", "id": "rs_" + rid[5:], "summary": [{"type": "summary_text",
                                                                                    "text": reasoning}]})
            out.append({"type": "message", "id": "msg_" + rid[5:], "role": "assistant", "status": status,
                        "content": [{"type": "output_text", "text": text, "annotations": []}]})
            return {"id": rid, "object": "response", "created_at": created, "model": llm.model_id, "status": status,
                    "output": out, "output_text": text,
                    "usage": {"input_tokens": len(ids), "output_tokens": n_out, "total_tokens": len(ids) + n_out}}

        if body.get("stream"):
            def gen():
                def ev(name, data):
                    return f"event: {name}\ndata: {json.dumps(dict(data, type=name), ensure_ascii=False)}\n\n".encode()

                yield ev("response.created", {"response": envelope("in_progress", "", 0)})
                split = ThinkingSplitter()
                text, n_out = "", 0
                for e in ctx.run(llm, ids, params, request_id=rid, scope=scope):
                    if e.error:
                        yield ev("error", {"message": e.error})
                        return
                    n_out += len(e.token_ids)
                    for kind, piece in split.push(e.text) + (split.flush() if e.finished else []):
                        if kind == "content" and piece:
                            text += piece
                            yield ev("response.output_text.delta", {"item_id": "msg_" + rid[5:], "output_index": 0,
                                                                    "content_index": 0, "delta": piece})
                yield ev("response.output_text.done", {"item_id": "msg_" + rid[5:], "output_index": 0,
                                                       "content_index": 0, "text": text})
                final = envelope("completed", text, n_out)
                responses_store[rid] = final
                yield ev("response.completed", {"response": final})

            return StreamingResponse(iterate_in_threadpool(gen()), media_type="text/event-stream",
                                     headers={"x-request-id": rid})

        def run_all():
            text, n_out = "", 0
            for e in ctx.run(llm, ids, params, request_id=rid, scope=scope):
                if e.error:
                    raise ApiError(500, e.error, "server_error")
                text += e.text
                n_out += len(e.token_ids)
            reasoning, answer = split_thinking(text)
            return envelope("completed", answer, n_out, reasoning)

        out = await run_in_threadpool(run_all)
        if body.get("store", True):
            responses_store[rid] = out
            while len(responses_store) > 1024:
                responses_store.pop(next(iter(responses_store)))
        return JSONResponse(out, headers={"x-request-id": rid})

    @r.get("/v1/responses/{rid}")
    async def get_response(rid: str):
        if rid not in responses_store:
            raise ApiError(404, f"response '{rid}' not found", "not_found_error")
        return responses_store[rid]

    @r.delete("/v1/responses/{rid}")
    async def delete_response(rid: str):
        if responses_store.pop(rid, None) is None:
            raise ApiError(404, f"response '{rid}' not found", "not_found_error")
        return {"id": rid, "object": "response", "deleted": True}

    return r
