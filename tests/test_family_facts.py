"""Family facts that live in file metadata: Granite's multipliers in a GGUF, Phi-3's fused feed-forward tensor."""
import os

import numpy as np
import pytest
import torch

from loken_b200.models import loader
from loken_b200.models.config import tiny
from loken_b200.models.weights import dequant_linear
from loken_b200.ops import quant


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k", "q6_k"])
def test_scale_weight_multiplies_the_block_scales(fmt):
    torch.manual_seed(1)
    w = torch.randn(32, 512) * 0.05
    q = quant.quantize_weight(w, fmt)
    before = quant.dequantize_weight(q).clone()
    codes = q.codes.clone()
    quant.scale_weight_(q, 0.37)
    assert torch.equal(q.codes, codes)
    after = quant.dequantize_weight(q)
    assert (after - 0.37 * before).abs().max().item() <= 2e-3 * before.abs().max().item()     # fp16 scale fields


@pytest.mark.parametrize("fmt", ["bf16", "q8_0"])
def test_granite_multipliers_are_read_from_a_gguf(tmp_path, fmt):
    base = dict(weight_format=fmt, head_dim=64, n_q=4, n_kv=2, hidden=256, intermediate=512, vocab=300)
    plain, gran = tiny("llama", **base), tiny("llama", **base)
    gran.arch = "granite"
    pa, pb = os.path.join(tmp_path, "a.gguf"), os.path.join(tmp_path, "b.gguf")
    loader.export_random_gguf(pa, plain, seed=5, std=0.05)
    loader.export_random_gguf(pb, gran, seed=5, std=0.05, tokenizer_meta={
        "granite.residual_scale": 0.25, "granite.logit_scale": 4.0, "granite.embedding_scale": 6.0,
        "granite.attention.scale": 0.0625})
    wa, _ = loader.load_gguf(pa, torch.device("cpu"))
    wb, _ = loader.load_gguf(pb, torch.device("cpu"))
    c = wb.cfg
    assert (c.arch, c.embedding_scale, c.logit_scale, c.softmax_scale()) == ("granite", 6.0, 0.25, 0.0625)
    for la, lb in zip(wa.layers, wb.layers):
        for name in ("wo", "w_down"):
            a, b = dequant_linear(getattr(la, name)).float(), dequant_linear(getattr(lb, name)).float()
            assert (b - 0.25 * a).abs().max().item() <= 4e-3 * a.abs().max().item()
        for name in ("wqkv", "w_gate_up"):
            assert torch.equal(dequant_linear(getattr(la, name)), dequant_linear(getattr(lb, name)))


def test_phi3_fused_feed_forward_tensor(tmp_path):
    """A file without `ffn_gate` holds gate and up as the two halves of `ffn_up` (and q, k, v in `attn_qkv`)."""
    from loken_b200.formats import gguf as G

    cfg = tiny("llama", weight_format="bf16", head_dim=64, n_q=4, n_kv=2, hidden=256, intermediate=512, vocab=300)
    src = os.path.join(tmp_path, "split.gguf")
    loader.export_random_gguf(src, cfg, seed=7, std=0.05)
    r = G.GGUFReader(src)
    dst = os.path.join(tmp_path, "fused.gguf")
    w = G.GGUFWriter(dst)
    for k, v in r.meta.items():
        if not (isinstance(v, list) and not v):
            w.add_meta(k, v)
    for name, ti in r.tensors.items():
        if ".ffn_gate." in name or ".attn_k." in name or ".attn_v." in name:
            continue
        x = ti.to_float()
        if ".ffn_up." in name:
            x = np.concatenate([r.tensors[name.replace("ffn_up", "ffn_gate")].to_float(), x], 0)
        if ".attn_q." in name:
            x = np.concatenate([x, r.tensors[name.replace("attn_q", "attn_k")].to_float(),
                                r.tensors[name.replace("attn_q", "attn_v")].to_float()], 0)
            name = name.replace("attn_q", "attn_qkv")
        w.add_tensor(name, x.astype(np.float32), G.F32)
    w.close()
    r.close()
    a, _ = loader.load_gguf(src, torch.device("cpu"))
    b, _ = loader.load_gguf(dst, torch.device("cpu"))
    for la, lb in zip(a.layers, b.layers):
        for name in ("wqkv", "w_gate_up", "w_down", "wo"):
            assert torch.equal(dequant_linear(getattr(la, name)), dequant_linear(getattr(lb, name)))
