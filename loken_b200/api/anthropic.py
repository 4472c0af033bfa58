"""Messages routes: /v1/messages and /v1/messages/count_tokens (`src/api/anthropic.rs`,
`src/api/handlers/anthropic_api.rs`).  Streaming follows the named-event protocol:
message_start, content_block_start / _delta / _stop per block (thinking, text, tool_use),
message_delta with the stop reason and usage, message_stop."""
from __future__ import annotations

import json
import uuid
from typing import Iterator, List

from fastapi import APIRouter, Request
from fastapi.responses import JSONResponse, StreamingResponse
from starlette.concurrency import iterate_in_threadpool, run_in_threadpool

from ..text.chat import parse_tool_calls
from ..text.stream import ThinkingSplitter, split_thinking
from .common import ApiError, check_messages, new_request_id, params_from_messages
from .context import ServerContext


def _to_chat(body: dict) -> List[dict]:
    """Messages-shaped input (system string or blocks; content blocks incl. tool_use / tool_result)
    -> plain chat messages."""
    msgs = []
    sys_ = body.get("system")
    if sys_:
        if isinstance(sys_, list):
            sys_ = "".join(b.get("text", "") for b in sys_ if isinstance(b, dict))
        msgs.append({"role": "system", "content": sys_})
    for m in body.get("messages", []):
        c = m.get("content")
        if isinstance(c, str):
            msgs.append({"role": m["role"], "content": c})
            continue
        text, calls = "", []
        for b in c or []:
            t = b.get("type")
            if t == "text":
                text += b.get("text", "")
            elif t == "tool_use":
                calls.append({"id": b.get("id"), "type": "function",
                              "function": {"name": b.get("name"), "arguments": json.dumps(b.get("input", {}))}})
            elif t == "tool_result":
                rc = b.get("content")
                if isinstance(rc, list):
                    rc = "".join(x.get("text", "") for x in rc if isinstance(x, dict))
                msgs.append({"role": "tool", "content": rc or "", "tool_call_id": b.get("tool_use_id")})
        if text or calls:
            mm = {"role": m["role"], "content": text}
            if calls:
                mm["tool_calls"] = calls
            msgs.append(mm)
    return msgs


def _tools(body: dict):
    tools = body.get("tools")
    if not tools:
        return None
    return [{"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""),
                                              "parameters": t.get("input_schema", {})}} for t in tools]


def _ev(name: str, data: dict) -> bytes:
    return f"event: {name}\ndata: {json.dumps(data, ensure_ascii=False)}\n\n".encode()


def _stop_reason(reason, calls, hit_stop_seq: bool) -> str:
    if calls:
        return "tool_use"
    if reason == "length":
        return "max_tokens"
    return "stop_sequence" if hit_stop_seq else "end_turn"


def router(ctx: ServerContext) -> APIRouter:
    r = APIRouter()

    @r.post("/v1/messages/count_tokens")
    async def count_tokens(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        msgs = _to_chat(body)
        check_messages(msgs)
        ids = await run_in_threadpool(llm.prompt_ids, None, msgs, _tools(body), None)
        return {"input_tokens": len(ids)}

    @r.post("/v1/messages")
    async def messages(req: Request):
        body = await req.json()
        llm = ctx.registry.get(body.get("model"))
        msgs = _to_chat(body)
        check_messages(msgs)
        params = params_from_messages(body, llm)
        tools = _tools(body)
        ids = await run_in_threadpool(llm.prompt_ids, None, msgs, tools, params)
        rid = "msg_" + uuid.uuid4().hex[:24]
        scope = getattr(req.state, "api_key", None)
        want_thinking = (body.get("thinking") or {}).get("type") == "enabled"

        if body.get("stream"):
            def gen() -> Iterator[bytes]:
                yield _ev("message_start", {"type": "message_start", "message": {
                    "id": rid, "type": "message", "role": "assistant", "model": llm.model_id, "content": [],
                    "stop_reason": None, "stop_sequence": None,
                    "usage": {"input_tokens": len(ids), "output_tokens": 0}}})
                split = ThinkingSplitter()
                block, kind_open = -1, None
                n_out, reason, held = 0, None, ""

                def open_block(kind):
                    nonlocal block, kind_open
                    out = b""
                    if kind_open is not None:
                        out += _ev("content_block_stop", {"type": "content_block_stop", "index": block})
                    block += 1
                    kind_open = kind
                    cb = {"type": "thinking", "thinking": ""} if kind == "thinking" else {"type": "text", "text": ""}
                    return out + _ev("content_block_start", {"type": "content_block_start", "index": block,
                                                             "content_block": cb})

                figs, cached = None, 0
                for ev in ctx.run(llm, ids, params, request_id=rid, scope=scope):
                    if ev.error:
                        yield _ev("error", {"type": "error", "error": {"type": "api_error", "message": ev.error}})
                        return
                    if ev.progress is not None:
                        from .common import prefill_comment

                        yield prefill_comment(ev.progress)
                        continue
                    if ev.finished:
                        figs, cached = ev.figures, ev.cached_tokens
                    n_out += len(ev.token_ids)
                    reason = ev.finish_reason or reason
                    for kind, text in split.push(ev.text) + (split.flush() if ev.finished else []):
                        if kind == "reasoning":
                            if not want_thinking:
                                continue
                            if kind_open != "thinking":
                                yield open_block("thinking")
                            yield _ev("content_block_delta", {"type": "content_block_delta", "index": block,
                                                              "delta": {"type": "thinking_delta", "thinking": text}})
                        elif tools:
                            held += text
                        else:
                            if kind_open != "text":
                                yield open_block("text")
                            yield _ev("content_block_delta", {"type": "content_block_delta", "index": block,
                                                              "delta": {"type": "text_delta", "text": text}})
                calls = []
                if tools:
                    rest, calls = parse_tool_calls(held)
                    if rest:
                        yield open_block("text")
                        yield _ev("content_block_delta", {"type": "content_block_delta", "index": block,
                                                          "delta": {"type": "text_delta", "text": rest}})
                    for c in calls:
                        if kind_open is not None:
                            yield _ev("content_block_stop", {"type": "content_block_stop", "index": block})
                        block += 1
                        kind_open = "tool_use"
                        yield _ev("content_block_start", {"type": "content_block_start", "index": block,
                                                          "content_block": {"type": "tool_use", "id": c["id"],
                                                                            "name": c["function"]["name"], "input": {}}})
                        yield _ev("content_block_delta", {"type": "content_block_delta", "index": block, "delta": {
                            "type": "input_json_delta", "partial_json": c["function"]["arguments"]}})
                if kind_open is not None:
                    yield _ev("content_block_stop", {"type": "content_block_stop", "index": block})
                yield _ev("message_delta", {"type": "message_delta", "delta": {
                    "stop_reason": _stop_reason(reason, calls, False), "stop_sequence": None},
                    "usage": {"output_tokens": n_out, "cache_read_input_tokens": cached,
                              **({"loken": figs} if figs else {})}})
                yield _ev("message_stop", {"type": "message_stop"})

            return StreamingResponse(iterate_in_threadpool(gen()), media_type="text/event-stream",
                                     headers={"x-request-id": rid})

        def run_all():
            text, n_out, reason = "", 0, None
            figs, cached = None, 0
            for ev in ctx.run(llm, ids, params, request_id=rid, scope=scope):
                if ev.error:
                    raise ApiError(500, ev.error, "api_error")
                if ev.finished:
                    figs, cached = ev.figures, ev.cached_tokens
                text += ev.text
                n_out += len(ev.token_ids)
                reason = ev.finish_reason or reason
            thinking, answer = split_thinking(text)
            calls = []
            if tools:
                answer, calls = parse_tool_calls(answer)
            content = []
            if thinking and want_thinking:
                content.append({"type": "thinking", "thinking": thinking})
            if answer or not calls:
                content.append({"type": "text", "text": answer})
            for c in calls:
                content.append({"type": "tool_use", "id": c["id"], "name": c["function"]["name"],
                                "input": json.loads(c["function"]["arguments"] or "{}")})
            return {"id": rid, "type": "message", "role": "assistant", "model": llm.model_id, "content": content,
                    "stop_reason": _stop_reason(reason, calls, False), "stop_sequence": None,
                    "usage": {"input_tokens": len(ids), "output_tokens": n_out, "cache_read_input_tokens": cached,
                              **({"loken": figs} if figs else {})}}

        return JSONResponse(await run_in_threadpool(run_all), headers={"x-request-id": rid})

    return r
