"""`LLM`: a loaded model a program can talk to — weights, tokenizer, chat template, the
continuous-batching engine and the worker thread that drives it.

    llm = LLM.load("model.gguf")                    # or LLM.load("llama-3.1-8b") for random-init weights
    print(llm.generate("Hello", GenerationParams(max_tokens=32)).text)
    for ev in llm.stream(messages=[{"role": "user", "content": "hi"}]): print(ev.text, end="")

Every request, streamed or not, goes through the worker thread's engine loop, so overlapping
callers batch together (the reference routes overlapping requests to its batch worker the same
way, `src/inference/engine/llm_engine/batching.rs:29-290`, `serve/continuous_serve.rs:1526-1707`).
Three consecutive failed steps stop the worker, as there.
"""
from __future__ import annotations

import os
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Sequence, Union

import torch

from ..models.config import ModelConfig, get_config
from ..serve.engine import LLMEngine, StepOutput
from ..serve.params import SamplingParams
from ..text.chat import parse_tool_calls, render_chat
from ..text.stream import StopTracker, StreamDetokenizer, split_thinking
from ..text.tokenizer import BaseTokenizer, ByteTokenizer, from_gguf_meta


@dataclass
class GenerationParams(SamplingParams):
    """Sampling parameters plus the text-level options of a request."""
    skip_special_tokens: bool = True
    echo: bool = False
    thinking_token_budget: Optional[int] = None
    truncate_prompt_tokens: Optional[int] = None   # -1: the model's window
    truncation_side: str = "left"                  # left keeps the last tokens, right the first
    cache_salt: Optional[str] = None


@dataclass
class StreamEvent:
    text: str = ""
    token_ids: List[int] = field(default_factory=list)
    finished: bool = False
    finish_reason: Optional[str] = None
    logprobs: Optional[List[tuple]] = None
    error: Optional[str] = None
    progress: Optional[tuple] = None     # (prompt tokens read, prompt tokens to read) while a prompt is read
    figures: Optional[dict] = None       # the request's `loken` figures, on the last event
    cached_tokens: int = 0               # prompt tokens served from the prefix cache, on the last event


@dataclass
class Completion:
    text: str
    token_ids: List[int]
    finish_reason: Optional[str]
    prompt_tokens: int
    completion_tokens: int
    cached_tokens: int = 0
    ttft_s: Optional[float] = None
    total_s: float = 0.0
    logprobs: Optional[List[tuple]] = None
    reasoning: str = ""
    tool_calls: List[dict] = field(default_factory=list)
    figures: Optional[dict] = None


class EmbedsPrompt(list):
    """A prompt given as embedding rows: placeholder token ids (one per row) carrying the rows."""

    def __init__(self, embeds):
        super().__init__([0] * int(embeds.shape[0]))
        self.embeds = embeds


class _Ticket:
    def __init__(self, prompt_ids, params, salt):
        self.prompt_ids, self.params, self.salt = prompt_ids, params, salt
        self.events: "queue.Queue[StepOutput | Exception | None]" = queue.Queue()
        self.seq_id: Optional[int] = None
        self.t0 = time.perf_counter()
        self.on_event = None         # optional callable(event) invoked from the worker thread
        from ..utils.figures import RequestFigures

        self.fig = RequestFigures(arrival=self.t0)


class EngineWorker(threading.Thread):
    """Owns the engine: admits tickets, runs `step()` while there is work, routes each step's
    outputs to the ticket they belong to."""

    def __init__(self, engine: LLMEngine, max_strikes: int = 3):
        super().__init__(daemon=True, name="loken-engine")
        self.engine = engine
        self.inbox: "queue.Queue" = queue.Queue()
        self.wake = threading.Event()
        self.stop_flag = False
        self.tickets: Dict[int, _Ticket] = {}
        self.max_strikes = max_strikes
        self.healthy = True
        self.last_error: Optional[str] = None
        self.busy_s = 0.0
        self.steps = 0
        from ..utils.figures import EnergyLedger

        dev = getattr(engine, "device", None)
        self.ledger = (EnergyLedger.default(dev.index or 0) if dev is not None and dev.type == "cuda"
                       else EnergyLedger())

    def submit(self, t: _Ticket):
        if not self.healthy:
            raise RuntimeError(f"engine worker stopped after repeated step failures: {self.last_error}")
        self.inbox.put(("add", t))
        self.wake.set()

    def abort(self, t: _Ticket):
        self.inbox.put(("abort", t))
        self.wake.set()

    def shutdown(self):
        self.stop_flag = True
        self.wake.set()

    def _deliver(self, t: _Ticket, ev):
        t.events.put(ev)
        if t.on_event is not None:
            try:
                t.on_event(ev)
            except Exception:
                pass

    def _drain_inbox(self):
        while True:
            try:
                op, t = self.inbox.get_nowait()
            except queue.Empty:
                return
            if op == "add":
                try:
                    t.seq_id = self.engine.add_request(t.prompt_ids, t.params, salt=t.salt)
                    self.tickets[t.seq_id] = t
                    t.fig.prompt_total = len(t.prompt_ids)
                    self.ledger.open(t.fig)
                except Exception as e:          # bad request: report to its caller only
                    self._deliver(t, e)
            elif op == "abort" and t.seq_id is not None:
                self.engine.abort(t.seq_id)
            elif op == "call":
                # a function to run on the engine thread between steps (embeddings, cache resets)
                try:
                    t.events.put(t.prompt_ids(self.engine))
                except Exception as e:
                    t.events.put(e)

    def run(self):
        if self.engine.device.type == "cuda":
            torch.cuda.set_device(self.engine.device)
        while not self.stop_flag:
            self._drain_inbox()
            if not self.engine.has_work() and not self.engine.cancelled:
                self.wake.wait(timeout=0.05)
                self.wake.clear()
                continue
            t0 = time.perf_counter()
            try:
                outs = self.engine.step()
            except Exception as e:
                self.last_error = f"{type(e).__name__}: {e}"
                for sid, t in list(self.tickets.items()):
                    seq = self.engine.seqs.get(sid)
                    if seq is not None and seq.state == "finished":
                        self._deliver(t, RuntimeError(self.last_error))
                        self._forget(sid)
                if self.engine.stats.consecutive_errors >= self.max_strikes:
                    self.healthy = False
                    for sid, t in list(self.tickets.items()):
                        self._deliver(t, RuntimeError(self.last_error))
                        self._forget(sid)
                    return
                continue
            now = time.perf_counter()
            self.busy_s += now - t0
            self.steps += 1
            self._note_progress(t0, now)
            for o in outs:
                t = self.tickets.get(o.seq_id)
                if t is None:
                    continue
                self.ledger.note_tokens(t.fig, len(o.new_tokens))
                if o.finished:
                    self._close_figures(t, o.seq_id, now)
                    o.figures = t.fig.to_json()
                    o.cached_tokens = getattr(self.engine.seqs.get(o.seq_id), "cached_tokens", 0)
                self._deliver(t, o)
                if o.finished:
                    self._forget(o.seq_id)

    def _note_progress(self, step_start: float, now: float):
        """After a step: which requests have started their prompt, how far each prompt has been read,
        who produced a first token (request figures and the `loken-prefill` progress lines)."""
        for sid, t in self.tickets.items():
            seq = self.engine.seqs.get(sid)
            if seq is None:
                continue
            f = t.fig
            state = getattr(seq, "state", "running")
            if f.prefill_start is None and state != "waiting":
                f.prefill_start = step_start
            cached = getattr(seq, "cached_tokens", 0)
            n_prompt = len(getattr(seq, "prompt", t.prompt_ids))
            computed = getattr(seq, "computed", n_prompt)
            total = max(0, n_prompt - cached)
            done = max(0, min(computed, n_prompt) - cached)
            self.ledger.note_tokens(f, max(0, done - f.prompt_done))
            f.prompt_total, f.prompt_done = total, done
            if f.first_token is None and getattr(seq, "output", None):
                f.first_token = now

    def _close_figures(self, t: "_Ticket", sid: int, now: float):
        f = t.fig
        seq = self.engine.seqs.get(sid)
        if f.prefill_start is None:
            f.prefill_start = now
        f.end = now
        alloc = getattr(self.engine, "alloc", None)
        if seq is not None and alloc is not None and hasattr(alloc, "num_blocks"):
            f.kv_used = len(getattr(seq, "prompt", [])) + len(getattr(seq, "output", []))
            f.kv_capacity = alloc.num_blocks * alloc.block_size
        if seq is not None:
            f.accepted_drafts = getattr(seq, "accepted_drafts", 0)
            f.rejected_drafts = getattr(seq, "rejected_drafts", 0)
        self.ledger.close(f)

    def _forget(self, sid: int):
        self.tickets.pop(sid, None)
        self.engine.seqs.pop(sid, None)
        self.engine.rngs.pop(sid, None)


class LLM:
    def __init__(self, engine: LLMEngine, tokenizer: BaseTokenizer, model_id: str, meta: Optional[dict] = None,
                 path: Optional[str] = None):
        self.engine = engine
        self.tokenizer = tokenizer
        self.model_id = model_id
        self.meta = meta or {}
        self.path = path
        self.cfg: ModelConfig = engine.cfg
        self.loaded_at = time.time()
        ends = set(tokenizer.end_token_ids())
        engine.eos.update(ends)          # in place: `engine` may be a lock-step wrapper
        engine.runner.end_ids = sorted(engine.eos)
        self.control_group = None
        self.watchdog = None
        from ..text.grammar import GrammarSession

        factory = lambda spec: GrammarSession(tokenizer, spec[0], spec[1])
        try:
            setattr(getattr(engine, "_e", engine), "grammar_factory", factory)
        except AttributeError:
            pass
        self.worker = EngineWorker(engine)
        self.worker.start()
        self.requests_served = 0
        self._digest: Optional[str] = None

    @property
    def weights_digest(self) -> str:
        """What identifies the bytes this model runs on, for a peer that wants to continue one of its answers
        (`serve/replay.py`): a fingerprint of the file or checkpoint directory, computed on first use; empty
        when nothing is known (then no other node may resume this node's answers, nor this node theirs)."""
        if self._digest is None:
            from ..serve.replay import path_fingerprint

            try:
                self._digest = path_fingerprint(self.path) if self.path else ""
            except OSError:
                self._digest = ""
        return self._digest

    # ---- construction ----
    @classmethod
    def load(cls, model: str, *, device=None, model_id: Optional[str] = None, requant: Optional[str] = None,
             kv_format: Optional[str] = None, seed: int = 0, tp_rank: int = 0, tp_size: int = 1, comm=None,
             lora=None, **engine_kw) -> "LLM":
        """`model` is a Hugging Face checkpoint directory, a GGUF path or the name of a built-in shape
        (random-init weights).  `lora`: a PEFT adapter directory, or a list of directories or
        (directory, weight) pairs, merged into a bf16 / block-fp8 checkpoint as it loads."""
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        # what a reload after a keep-alive needs to bring the same model back (one rank only)
        kept = {k: v for k, v in dict(engine_kw, requant=requant, kv_format=kv_format, lora=lora).items()
                if v is not None and isinstance(v, (int, float, str, bool, list, tuple))} if tp_size == 1 else {}
        group = None
        watchdog = None
        draft = engine_kw.pop("draft", None)       # (model, k): a drafter attached on every rank before wrapping
        slots = int(engine_kw.pop("expert_slots", 0) or 0)
        if slots > 0:
            # a mixture model larger than the card: `slots` experts per layer stay resident, the rest stream
            # from pinned host memory as the router asks for them (models/expert_tier.py)
            from ..models.expert_tier import TieredMoeRunner

            engine_kw["moe_runner_factory"] = lambda c, w, cap, cm: TieredMoeRunner(c, w, cap, cm, slots=slots)
        if tp_size > 1:
            import torch.distributed as dist

            from ..parallel.follower import LockstepEngine, control_group
            from ..parallel.watchdog import RankWatchdog

            group = control_group()          # collective: every rank creates it here
            store = getattr(dist.distributed_c10d, "_get_default_store", lambda: None)()
            if store is not None:
                watchdog = RankWatchdog(store, tp_rank, tp_size, interval_s=1.0, timeout_s=15.0).start()

        def wrap(eng):
            if draft is not None:
                from ..serve.speculative import attach_draft_engine

                attach_draft_engine(eng, draft[0], k=draft[1], tp_rank=tp_rank, tp_size=tp_size, comm=comm)
            return LockstepEngine(eng, group, watchdog) if tp_size > 1 and tp_rank == 0 else eng

        if os.path.isdir(model) and os.path.exists(os.path.join(model, "config.json")):
            # a Hugging Face checkpoint directory (bf16 or block-fp8 safetensors + tokenizer.json)
            from ..models.loader_hf import load_hf
            from ..text.tokenizer import HFTokenizer

            w, hf = load_hf(model, dev, tp_rank=tp_rank, tp_size=tp_size, requant=requant, kv_format=kv_format)
            if lora:
                from ..models.lora import load_lora, merge_lora

                for item in ([lora] if isinstance(lora, (str, tuple)) else list(lora)):
                    path, wt = item if isinstance(item, tuple) else (item, 1.0)
                    merge_lora(w, load_lora(path), float(wt))
            tk_path = os.path.join(model, "tokenizer.json")
            if os.path.exists(tk_path):
                import tokenizers

                eos = hf.get("eos_token_id")
                eos_ids = eos if isinstance(eos, list) else ([eos] if eos is not None else [])
                tmpl = None
                tc_path = os.path.join(model, "tokenizer_config.json")
                if os.path.exists(tc_path):
                    import json as _json

                    tmpl = _json.load(open(tc_path)).get("chat_template")
                tk = HFTokenizer(tokenizers.Tokenizer.from_file(tk_path), hf.get("bos_token_id"),
                                 eos_ids[0] if eos_ids else None, eos_ids, False, tmpl)
            else:
                tk = ByteTokenizer(w.cfg.vocab)
            eng = LLMEngine(w.cfg, weights=w, device=dev, tp_rank=tp_rank, tp_size=tp_size, comm=comm, **engine_kw)
            llm = cls(wrap(eng), tk, model_id or os.path.basename(os.path.normpath(model)), hf, path=model)
            llm.load_kwargs = kept
            llm.control_group, llm.watchdog = group, watchdog
            return llm
        if lora:
            raise ValueError("adapters merge into a Hugging Face checkpoint directory (bf16 or block-fp8)")
        if os.path.exists(model):
            from ..models.loader import load_gguf

            w, meta = load_gguf(model, dev, tp_rank=tp_rank, tp_size=tp_size, ep_rank=tp_rank, ep_size=tp_size,
                                requant=requant, kv_format=kv_format)
            tk = from_gguf_meta(meta)
            eng = LLMEngine(w.cfg, weights=w, device=dev, tp_rank=tp_rank, tp_size=tp_size, comm=comm, **engine_kw)
            name = model_id or os.path.splitext(os.path.basename(model))[0]
            llm = cls(wrap(eng), tk, name, meta, path=model)
            llm.load_kwargs = kept
            llm.control_group, llm.watchdog = group, watchdog
            return llm
        cfg = get_config(model)
        if kv_format:
            cfg.kv_format = kv_format
        eng = LLMEngine(cfg, device=dev, seed=seed, tp_rank=tp_rank, tp_size=tp_size, comm=comm, **engine_kw)
        llm = cls(wrap(eng), ByteTokenizer(cfg.vocab), model_id or model, {"general.architecture": cfg.arch})
        llm.control_group, llm.watchdog = group, watchdog
        llm._digest = f"init:{model}:{cfg.weight_format}:{cfg.n_layers}:{seed}"      # random weights are a function of these
        return llm

    def close(self):
        self.worker.shutdown()
        self.worker.join(timeout=5)

    # ---- text <-> tokens ----
    def tokenize(self, text: str, add_special: bool = True) -> List[int]:
        return self.tokenizer.encode(text, add_special)

    def detokenize(self, ids: Sequence[int], skip_special: bool = True) -> str:
        return self.tokenizer.decode(ids, skip_special)

    def render(self, messages: Sequence[dict], tools=None, add_generation_prompt: bool = True,
               continue_final_message: bool = False, **template_kwargs) -> str:
        tk = self.tokenizer
        bos = tk.decode([tk.bos_id], skip_special=False) if tk.bos_id is not None else ""
        eos = tk.decode([tk.eos_id], skip_special=False) if tk.eos_id is not None else ""
        return render_chat(messages, tk.chat_template, tools=tools, add_generation_prompt=add_generation_prompt,
                           continue_final_message=continue_final_message, bos_token=bos, eos_token=eos,
                           **template_kwargs)

    def prompt_ids(self, prompt: Union[str, Sequence[int], None] = None, messages: Optional[Sequence[dict]] = None,
                   tools=None, params: Optional[GenerationParams] = None, **render_kw) -> List[int]:
        if messages is not None:
            text = self.render(messages, tools=tools, **render_kw)
            ids = self.tokenizer.encode(text, add_special=not text.startswith("<|begin_of_text|>"))
        elif isinstance(prompt, str):
            ids = self.tokenizer.encode(prompt, add_special=True)
        else:
            ids = [int(t) for t in (prompt or [])]
        if params is not None and params.truncate_prompt_tokens:
            keep = params.truncate_prompt_tokens
            if keep < 0:
                keep = max(1, self.engine.max_ctx - 1 - int(params.max_tokens or 1))
            ids = ids[:keep] if params.truncation_side == "right" else ids[-keep:]
        bad = [t for t in ids if not (0 <= t < self.cfg.vocab)]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside the model's vocabulary of {self.cfg.vocab}")
        return ids

    # ---- generation ----
    def _salt(self, params: GenerationParams) -> int:
        if not params.cache_salt:
            return 0
        h = 0xcbf29ce484222325
        for b in params.cache_salt.encode():
            h = ((h ^ b) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
        return h

    def submit(self, ids: List[int], params: GenerationParams, on_event=None) -> _Ticket:
        t = _Ticket(ids, params, self._salt(params))
        t.on_event = on_event
        self.worker.submit(t)
        self.requests_served += 1
        return t

    def abort(self, ticket: _Ticket):
        cancel = getattr(ticket, "cancel", None)       # a request a peer is answering (`cluster/forward.py`)
        if cancel is not None:
            cancel()
            return
        self.worker.abort(ticket)

    def on_engine_thread(self, fn, timeout_s: float = 120.0):
        """Runs fn(engine) on the worker thread between steps and returns its result."""
        t = _Ticket(fn, None, 0)
        self.worker.inbox.put(("call", t))
        self.worker.wake.set()
        out = t.events.get(timeout=timeout_s)
        if isinstance(out, Exception):
            raise out
        return out

    def embed(self, text_or_ids, pooling: str = "last") -> List[float]:
        ids = self.tokenize(text_or_ids) if isinstance(text_or_ids, str) else [int(t) for t in text_or_ids]
        if not ids:
            raise ValueError("nothing to embed")
        v = self.on_engine_thread(lambda eng: eng.embed(ids, pooling))
        return [float(x) for x in v.tolist()], len(ids)

    def stream(self, prompt=None, params: Optional[GenerationParams] = None, *, messages=None, tools=None,
               timeout_s: float = 600.0, **render_kw) -> Iterator[StreamEvent]:
        """Yields text deltas as tokens arrive; stop sequences end the stream and are cut from the
        text unless `include_stop_str_in_output`."""
        params = params or GenerationParams()
        ids = self.prompt_ids(prompt, messages, tools, params, **render_kw)
        ticket = self.submit(ids, params)
        yield from self.events_of(ticket, params, timeout_s)

    def events_of(self, ticket: _Ticket, params: GenerationParams, timeout_s: float = 600.0
                  ) -> Iterator[StreamEvent]:
        detok = StreamDetokenizer(self.tokenizer, params.skip_special_tokens)
        stops = StopTracker(params.stop, params.include_stop_str_in_output)
        # Thinking budget (`src/api/thinking_budget.rs:1-8`): once the reasoning block has used its
        # tokens, the request is ended, the closing tag is appended and generation restarts from
        # there (the prefix cache holds everything already computed).
        budget = params.thinking_token_budget
        open_tag, close_tag = "<think>", "</think>"
        n_think, inside, seen_text, all_tokens = 0, False, "", []
        deadline = time.monotonic() + timeout_s
        got_token = False
        try:
            while True:
                try:
                    # until the first token arrives the wait wakes every 250 ms to report how far the prompt
                    # has been read (`docs/API.md:499-514` of the reference: `: loken-prefill` comment lines)
                    ev = ticket.events.get(timeout=timeout_s if got_token else 0.25)
                except queue.Empty:
                    if not got_token and time.monotonic() < deadline:
                        f = ticket.fig
                        if f.prompt_total > 0:
                            yield StreamEvent(progress=(int(f.prompt_done), int(f.prompt_total)))
                        continue
                    self.abort(ticket)
                    yield StreamEvent(finished=True, finish_reason="timeout", error="generation timed out")
                    return
                got_token = True
                if isinstance(ev, Exception):
                    yield StreamEvent(finished=True, finish_reason="error", error=str(ev))
                    return
                text = ""
                for tok in ev.new_tokens:
                    if tok in self.engine.eos and not params.ignore_eos and ev.finished and tok == ev.new_tokens[-1]:
                        continue              # the end token itself is not text
                    text += detok.push(tok)
                if ev.finished:
                    text += detok.flush()
                out, hit = stops.push(text)
                if hit:
                    self.abort(ticket)
                    yield StreamEvent(out, list(ev.new_tokens), True, "stop", ev.logprobs,
                                      figures=self._figures_now(ticket, ev), cached_tokens=self._cached(ticket, ev))
                    return
                if budget is not None and not ev.finished:
                    all_tokens += list(ev.new_tokens)
                    seen_text += text
                    inside = seen_text.rfind(open_tag) > seen_text.rfind(close_tag)
                    if inside:
                        n_think += len(ev.new_tokens)
                    if inside and n_think >= budget:
                        # end this pass and continue after a forced closing tag
                        self.abort(ticket)
                        yield StreamEvent(out + stops.flush() + close_tag, list(ev.new_tokens), False, None, ev.logprobs)
                        closing = self.tokenizer.encode(close_tag, add_special=False)
                        import dataclasses

                        left = None if params.max_tokens is None else max(1, params.max_tokens - len(all_tokens))
                        p2 = dataclasses.replace(params, thinking_token_budget=None, max_tokens=left)
                        t2 = self.submit(list(ticket.prompt_ids) + all_tokens + closing, p2)
                        yield from self.events_of(t2, p2, timeout_s)
                        return
                if ev.finished:
                    out += stops.flush()
                    yield StreamEvent(out, list(ev.new_tokens), True, ev.finish_reason, ev.logprobs,
                                      figures=self._figures_now(ticket, ev), cached_tokens=self._cached(ticket, ev))
                    return
                yield StreamEvent(out, list(ev.new_tokens), False, None, ev.logprobs)
        finally:
            if ticket.seq_id is not None and ticket.seq_id in self.worker.tickets:
                self.abort(ticket)

    @staticmethod
    def _figures_now(ticket: _Ticket, ev) -> dict:
        """The request's figures: what the worker closed at the last token, or (a stop string ended the
        request here, before the engine's own end) a closing made now."""
        figs = getattr(ev, "figures", None)
        if figs is not None:
            return figs
        f = ticket.fig
        if f.end is None:
            f.end = time.perf_counter()
        return f.to_json()

    @staticmethod
    def _cached(ticket: _Ticket, ev) -> int:
        return int(getattr(ev, "cached_tokens", 0) or 0)

    def generate(self, prompt=None, params: Optional[GenerationParams] = None, *, messages=None, tools=None,
                 **render_kw) -> Completion:
        params = params or GenerationParams()
        ids = self.prompt_ids(prompt, messages, tools, params, **render_kw)
        t0 = time.perf_counter()
        ticket = self.submit(ids, params)
        text, toks, reason, lps, ttft = "", [], None, [], None
        for ev in self.events_of(ticket, params):
            if ev.error:
                raise RuntimeError(ev.error)
            if ttft is None and ev.token_ids:
                ttft = time.perf_counter() - t0
            text += ev.text
            toks += ev.token_ids
            if ev.logprobs:
                lps += ev.logprobs
            reason = ev.finish_reason
        reasoning, answer = split_thinking(text)
        rest, calls = parse_tool_calls(answer) if tools else (answer, [])
        if params.echo and isinstance(prompt, str):
            rest = prompt + rest
        return Completion(rest, toks, "tool_calls" if calls else reason, len(ids), len(toks), 0, ttft,
                          time.perf_counter() - t0, lps or None, reasoning, calls)

    # ---- introspection for the API layer ----
    def info(self) -> dict:
        cfg = self.cfg
        return {"id": self.model_id, "architecture": cfg.arch, "parameters": cfg.param_count(),
                "context_length": cfg.context_length, "quantization": cfg.weight_format, "kv_cache": cfg.kv_format,
                "layers": cfg.n_layers, "hidden": cfg.hidden, "heads": cfg.n_q, "kv_heads": cfg.n_kv,
                "experts": cfg.n_experts, "vocab": cfg.vocab, "path": self.path, "loaded_at": self.loaded_at}
