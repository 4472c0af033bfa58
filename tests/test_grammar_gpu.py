"""Structured outputs end to end on a random-init model: whatever the logits say, the sampled
text stays inside the requested language."""
import json
import re

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def llm():
    from loken_b200.engine.llm import LLM

    m = LLM.load("tiny-llama", max_seqs=8, max_ctx=512, num_blocks=128, max_prefill_tokens=256)
    yield m
    m.close()


@pytest.mark.parametrize("temperature", [0.0, 1.0])
def test_regex_and_choice(llm, temperature):
    from loken_b200.engine.llm import GenerationParams

    for seed in range(3):
        p = GenerationParams(temperature=temperature, top_k=0, top_p=1.0, max_tokens=16, seed=seed,
                             grammar=("regex", "(yes|no|maybe) [0-9]{3}"))
        out = llm.generate("answer:", p)
        assert re.fullmatch(r"(yes|no|maybe) [0-9]{3}", out.text), out.text
        assert out.finish_reason == "stop"
    p = GenerationParams(temperature=temperature, max_tokens=16, seed=1, grammar=("choice", ["alpha", "beta"]))
    assert llm.generate("pick:", p).text in ("alpha", "beta")


def test_json_schema_and_unconstrained_neighbours(llm):
    from loken_b200.engine.llm import GenerationParams

    # bounded values and fixed whitespace: a random model cannot wander off into endless digits or spaces
    schema = {"type": "object", "properties": {"n": {"enum": [1, 22, 333]}, "ok": {"type": "boolean"}},
              "required": ["n", "ok"], "additionalProperties": False, "x-guidance": {"whitespace_flexible": False}}
    pj = GenerationParams(temperature=0.8, top_k=0, top_p=1.0, max_tokens=96, seed=3, grammar=("json_schema", schema))
    pf = GenerationParams(temperature=0.8, top_k=0, top_p=1.0, max_tokens=12, seed=4, ignore_eos=True)
    # a constrained and a free request in the same batch: only the first is masked
    t1 = llm.submit(llm.prompt_ids("json:"), pj)
    t2 = llm.submit(llm.prompt_ids("free:"), pf)
    text1 = "".join(ev.text for ev in llm.events_of(t1, pj))
    toks2 = [t for ev in llm.events_of(t2, pf) for t in ev.token_ids]
    obj = json.loads(text1)
    assert set(obj) == {"n", "ok"} and isinstance(obj["n"], int) and isinstance(obj["ok"], bool)
    assert len(toks2) == 12
    with pytest.raises(Exception):
        llm.generate("x", GenerationParams(grammar=("regex", "(unclosed")))
    assert llm.worker.healthy
    assert llm.engine.runner.wsp.read_status() == 0


def test_constrained_requests_under_speculation(llm):
    """Verify rows of a constrained request are masked for their own history: the text stays in the language,
    drafts that fit it are accepted, and the output equals plain constrained decoding."""
    from loken_b200.engine.llm import GenerationParams
    from loken_b200.serve.speculative import PromptLookupDrafter, Speculator

    forced = GenerationParams(temperature=0.0, max_tokens=40, grammar=("regex", "(ab ){6}ab"))
    schema = {"type": "object", "properties": {"n": {"enum": [1, 22, 333]}, "ok": {"type": "boolean"}},
              "required": ["n", "ok"], "additionalProperties": False, "x-guidance": {"whitespace_flexible": False}}
    sampled = GenerationParams(temperature=0.8, top_k=0, top_p=1.0, max_tokens=96, seed=3, grammar=("json_schema", schema))
    free = GenerationParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    plain = [llm.generate("ab ab ab ab ", forced).text, llm.generate("json:", sampled).text,
             llm.generate("ab ab ab ab ", free).token_ids]
    llm.on_engine_thread(lambda eng: eng.attach_speculator(Speculator(PromptLookupDrafter(), 4)))
    try:
        a = llm.generate("ab ab ab ab ", forced)
        assert a.text == "ab ab ab ab ab ab ab" == plain[0] and a.finish_reason == "stop"
        spec = llm.engine.spec
        assert spec.accepted > 0                    # the language leaves one choice per position, so the looked-up drafts fit
        b = llm.generate("json:", sampled)
        assert b.text == plain[1] and set(json.loads(b.text)) == {"n", "ok"}
        assert llm.generate("ab ab ab ab ", free).token_ids == plain[2]
    finally:
        llm.on_engine_thread(lambda eng: eng.detach_speculator())
    assert llm.worker.healthy and llm.engine.runner.wsp.read_status() == 0
