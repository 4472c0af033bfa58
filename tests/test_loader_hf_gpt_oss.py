"""gpt-oss checkpoints in the Hugging Face layout: MXFP4 experts as `*_blocks` / `*_scales` with
interleaved gate / up rows, sinks, biases, layer types; round trip through the writer and the loader."""
import json

import torch

from loken_b200.models.config import tiny
from loken_b200.models.loader_hf import config_from_hf, load_hf, save_hf_gpt_oss
from loken_b200.models.reference import forward_ref
from loken_b200.models.weights import random_weights


def _tiny():
    return tiny("gpt-oss", weight_format="mxfp4", n_experts=4, top_k=2, hidden=128, expert_intermediate=64, n_q=4, n_kv=2,
                head_dim=32, vocab=256, n_layers=2)


def test_config_reads_the_family_facts():
    hf = {"architectures": ["GptOssForCausalLM"], "num_hidden_layers": 4, "hidden_size": 2880, "num_attention_heads": 64,
          "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 2880, "vocab_size": 201088,
          "rope_theta": 150000, "sliding_window": 128, "num_local_experts": 128, "num_experts_per_tok": 4,
          "layer_types": ["sliding_attention", "full_attention"] * 2, "quantization_config": {"quant_method": "mxfp4"},
          "rope_scaling": {"rope_type": "yarn", "factor": 32.0, "original_max_position_embeddings": 4096,
                           "beta_fast": 32.0, "beta_slow": 1.0}}
    c = config_from_hf(hf, "oss")
    assert c.arch == "gpt-oss" and c.is_moe and c.n_experts == 128 and c.top_k == 4 and c.expert_intermediate == 2880
    assert c.weight_format == "mxfp4" and c.sinks and c.attn_bias and c.expert_bias and c.glu_mode == 1
    assert c.rope_scaling.kind == "yarn" and c.rope_scaling.factor == 32.0 and c.rope_scaling.original_context == 4096
    assert [c.layer_window(i) for i in range(4)] == [128, 0, 128, 0]


def test_round_trip_keeps_every_plane_and_the_logits(tmp_path):
    cfg = _tiny()
    dev = torch.device("cpu")
    w = random_weights(cfg, dev, seed=4, std=0.05)
    d = str(tmp_path / "oss")
    save_hf_gpt_oss(d, cfg, w)
    assert json.load(open(d + "/config.json"))["quantization_config"]["quant_method"] == "mxfp4"
    w2, hf = load_hf(d, dev)
    assert w2.cfg.weight_format == "mxfp4" and w2.cfg.n_experts == 4 and w2.cfg.sliding_window == cfg.sliding_window
    for a, b in zip(w.layers, w2.layers):
        assert torch.equal(a.moe.gate_up.codes, b.moe.gate_up.codes) and torch.equal(a.moe.gate_up.scales, b.moe.gate_up.scales)
        assert torch.equal(a.moe.down.codes, b.moe.down.codes) and torch.equal(a.moe.down.scales, b.moe.down.scales)
        assert torch.equal(a.moe.gate_up_b, b.moe.gate_up_b) and torch.equal(a.moe.down_b, b.moe.down_b)
        assert torch.equal(a.moe.router_w, b.moe.router_w) and torch.equal(a.sinks, b.sinks)
        assert torch.equal(a.wqkv.weight, b.wqkv.weight) and torch.equal(a.wqkv.bias, b.wqkv.bias)
        assert a.window == b.window
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (21,), generator=g).tolist()
    assert torch.equal(forward_ref(w, prompt), forward_ref(w2, prompt))


def test_expert_ranges_follow_the_rank_and_other_formats_decode_the_nibbles(tmp_path):
    cfg = _tiny()
    dev = torch.device("cpu")
    w = random_weights(cfg, dev, seed=4, std=0.05)
    d = str(tmp_path / "oss")
    save_hf_gpt_oss(d, cfg, w)
    r1, _ = load_hf(d, dev, tp_rank=1, tp_size=2)
    m = r1.layers[0].moe
    I, H = cfg.expert_intermediate, cfg.hidden
    assert (m.e_lo, m.e_cnt) == (2, 2) and m.gate_up.rows == 2 * 2 * I
    assert torch.equal(m.gate_up.codes, w.layers[0].moe.gate_up.codes[2 * 2 * I:])
    bf, _ = load_hf(d, dev, requant="bf16")
    from loken_b200.ops.quant import dequantize_weight

    want = dequantize_weight(w.layers[0].moe.gate_up).float()
    got = bf.layers[0].moe.gate_up.float()
    assert bf.layers[0].moe.fmt == "bf16" and torch.allclose(got.reshape(want.shape), want, atol=1e-6)
