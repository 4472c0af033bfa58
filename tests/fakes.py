"""A CPU stand-in for LLMEngine with the same surface, so the text layer, the worker thread and
the HTTP dialects can be tested without a GPU.  Each request "generates" the bytes of a scripted
reply, one token per step, then the end token."""
import time
import types
from typing import Dict, List, Optional

import torch

from loken_b200.models.config import tiny
from loken_b200.serve.engine import EngineStats, StepOutput
from loken_b200.serve.kv_manager import PagedKvAllocator
from loken_b200.serve.params import SamplingParams


class FakeSeq:
    def __init__(self, sid, prompt, params, reply):
        self.seq_id, self.prompt, self.params = sid, list(prompt), params
        self.output: List[int] = []
        self.reply = reply
        self.state = "running"
        self.finish_reason = None


class FakeEngine:
    def __init__(self, reply: str = "Hello from the fake engine.", max_ctx: int = 512, fail_steps: int = 0,
                 step_delay: float = 0.0):
        self.cfg = tiny("llama")
        self.cfg.vocab = 260
        self.device = torch.device("cpu")
        self.max_ctx = max_ctx
        self.eos = {257}
        self.runner = types.SimpleNamespace(end_ids=[257], model=None)
        # the real allocator: the ops routes are tested against the API the engine really has
        self.alloc = PagedKvAllocator(100, 16)
        self.seqs: Dict[int, FakeSeq] = {}
        self.rngs: Dict[int, object] = {}
        self.cancelled = set()
        self.stats = EngineStats()
        self.next_id = 0
        self.reply = reply
        self.fail_steps = fail_steps
        self.step_delay = step_delay
        self.prompts: List[List[int]] = []
        self.params_seen: list = []
        self.embeds: list = []

    def add_request(self, prompt, params: Optional[SamplingParams] = None, salt: int = 0) -> int:
        params = (params or SamplingParams()).validate()
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        sid = self.next_id
        self.next_id += 1
        self.seqs[sid] = FakeSeq(sid, prompt, params, list(self.reply.encode()) + [257])
        self.prompts.append(list(prompt))
        self.params_seen.append(params)
        self.embeds.append(getattr(prompt, "embeds", None))
        return sid

    def abort(self, sid):
        self.cancelled.add(sid)

    def reset_prefix_cache(self) -> int:
        return int(self.alloc.reset_prefix_cache() or 0)

    def layer_perf(self, n_tokens=1):
        return [{"stage": "embed", "ms": 0.01}, {"stage": "layer 0", "ms": 0.1}, {"stage": "head", "ms": 0.02}]

    def embed(self, tokens, pooling="last"):
        v = torch.zeros(8)
        v[len(tokens) % 8] = 1.0
        return v

    def has_work(self):
        return any(s.state == "running" for s in self.seqs.values())

    def step(self):
        if self.step_delay:
            time.sleep(self.step_delay)
        outs = []
        for sid in list(self.cancelled):
            s = self.seqs.get(sid)
            if s is not None and s.state == "running":
                s.state = "finished"
                outs.append(StepOutput(sid, [], True, "cancelled"))
        self.cancelled.clear()
        if self.fail_steps > 0:
            self.fail_steps -= 1
            self.stats.step_errors += 1
            self.stats.consecutive_errors += 1
            for s in self.seqs.values():
                if s.state == "running":
                    s.state = "finished"
            raise RuntimeError("injected step failure")
        self.stats.consecutive_errors = 0
        self.stats.steps += 1
        for s in list(self.seqs.values()):
            if s.state != "running":
                continue
            # a resumed request continues the script where its first part stopped
            at = getattr(s.params, "resume_position", 0) + len(s.output)
            tok = s.reply[min(at, len(s.reply) - 1)]
            s.output.append(tok)
            o = StepOutput(s.seq_id, [tok])
            if s.params.logprobs:
                o.logprobs = [(-0.5, [(tok, -0.5), (32, -1.5)][:s.params.top_logprobs])]
            if tok == 257 and not s.params.ignore_eos:
                o.finished, o.finish_reason = True, "stop"
            elif s.params.max_tokens is not None and len(s.output) >= s.params.max_tokens:
                o.finished, o.finish_reason = True, "length"
            elif at + 1 >= len(s.reply):
                o.finished, o.finish_reason = True, "length"
            if o.finished:
                s.state = "finished"
            outs.append(o)
        return outs


def fake_llm(reply: str = "Hello from the fake engine.", model_id: str = "fake-model", **kw):
    from loken_b200.engine.llm import LLM
    from loken_b200.text.tokenizer import ByteTokenizer

    return LLM(FakeEngine(reply, **kw), ByteTokenizer(260), model_id)
