"""Draft heads (EAGLE / MTP form): the head's input maths on CPU, the safetensors layouts, and on the
GPU that drafting through a head never changes what is generated."""
import os

import pytest
import torch

from loken_b200.serve.draft_head import DraftHeadWeights, head_input


def test_head_input_is_fc_of_embedding_and_feature_with_the_mtp_norms():
    torch.manual_seed(0)
    H = 16
    fc = torch.randn(H, 2 * H).bfloat16()
    e, f = torch.randn(3, H).bfloat16(), torch.randn(3, H).bfloat16() * 5
    hw = DraftHeadWeights("eagle", fc, None, None)
    want = torch.cat([e.float(), f.float()], -1).bfloat16() @ fc.t()
    assert torch.equal(head_input(hw, e, f, 1e-5), want)
    hw = DraftHeadWeights("mtp", fc, torch.ones(H), None, torch.full((H,), 2.0), torch.ones(H))
    ne = e.float() * torch.rsqrt(e.float().pow(2).mean(-1, keepdim=True) + 1e-5) * 2.0
    nf = f.float() * torch.rsqrt(f.float().pow(2).mean(-1, keepdim=True) + 1e-5)
    want = ((torch.cat([ne, nf], -1).bfloat16() @ fc.t()).float() + 1.0).bfloat16()
    assert torch.equal(head_input(hw, e, f, 1e-5), want)


def _write_head(tmp_path, cfg, kind):
    from safetensors.torch import save_file

    H, hd = cfg.hidden, cfg.head_dim
    g = torch.Generator().manual_seed(1)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.05).bfloat16()
    t = {"layers.0.self_attn.q_proj.weight": r(cfg.n_q * hd, H), "layers.0.self_attn.k_proj.weight": r(cfg.n_kv * hd, H),
         "layers.0.self_attn.v_proj.weight": r(cfg.n_kv * hd, H), "layers.0.self_attn.o_proj.weight": r(H, cfg.n_q * hd),
         "layers.0.mlp.gate_proj.weight": r(cfg.intermediate, H), "layers.0.mlp.up_proj.weight": r(cfg.intermediate, H),
         "layers.0.mlp.down_proj.weight": r(H, cfg.intermediate),
         "layers.0.post_attention_layernorm.weight": torch.ones(H)}
    if kind == "eagle":
        t["fc.weight"], t["fc.bias"] = r(H, 2 * H), torch.zeros(H)
    else:
        t["model.eh_proj.weight"], t["model.enorm.weight"], t["model.hnorm.weight"] = r(H, 2 * H), torch.ones(H), torch.ones(H)
    d = tmp_path / kind
    os.makedirs(d, exist_ok=True)
    save_file(t, str(d / "model.safetensors"))
    return str(d)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["eagle", "mtp", "random:eagle"])
def test_generation_is_unchanged_by_a_draft_head(tmp_path, kind):
    from loken_b200.models.config import tiny
    from loken_b200.models.weights import random_weights
    from loken_b200.serve.engine import LLMEngine
    from loken_b200.serve.params import SamplingParams
    from loken_b200.serve.speculative import attach_draft_engine

    dev = torch.device("cuda")
    cfg = tiny("llama", head_dim=64, n_q=4, n_kv=2, n_layers=3)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (9, 30, 17)]
    sp = [SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True),
          SamplingParams(temperature=0.8, top_p=0.9, seed=5, max_tokens=24, ignore_eos=True),
          SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)]

    def run(with_head):
        w = random_weights(cfg, dev, seed=2, std=0.05)
        eng = LLMEngine(cfg, weights=w, device=dev, num_blocks=128, max_seqs=4, max_prefill_tokens=256, max_ctx=128,
                        lookahead=8)
        if with_head:
            src = kind if kind.startswith("random") else _write_head(tmp_path, cfg, kind)
            st = attach_draft_engine(eng, src, k=3, method="head")
            assert st["drafter"]["method"] == "head" and kind.split(":")[-1] in st["drafter"]["model"]
        ids = [eng.add_request(p, s) for p, s in zip(prompts, sp)]
        while eng.has_work():
            eng.step()
        assert eng.runner.wsp.read_status() == 0
        return [eng.seqs[i].output for i in ids], eng

    plain, _ = run(False)
    drafted, eng = run(True)
    assert drafted == plain                       # verification keeps the text exact, greedy and sampled alike
    st = eng.spec.status()
    assert st["accepted"] + st["rejected"] > 0    # the head did propose tokens
    assert not eng.spec.drafter.known             # finished sequences gave their head cache back
