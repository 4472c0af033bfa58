"""LoRA adapters merged into the base weights (CPU tensors; no GPU needed)."""
import json

import pytest
import torch

from loken_b200.models.config import tiny
from loken_b200.models.lora import adapter_from_tensors, load_lora, merge_lora
from loken_b200.models.weights import dequant_linear, random_weights


def _adapter_tensors(cfg, r, layers, projs, seed=0):
    g = torch.Generator().manual_seed(seed)
    hd = cfg.head_dim
    dims = {"q_proj": (cfg.n_q * hd, cfg.hidden), "k_proj": (cfg.n_kv * hd, cfg.hidden),
            "v_proj": (cfg.n_kv * hd, cfg.hidden), "o_proj": (cfg.hidden, cfg.n_q * hd),
            "gate_proj": (cfg.intermediate, cfg.hidden), "up_proj": (cfg.intermediate, cfg.hidden),
            "down_proj": (cfg.hidden, cfg.intermediate)}
    t = {}
    for il in layers:
        for p in projs:
            out, inn = dims[p]
            blk = "self_attn" if p in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            base = f"base_model.model.model.layers.{il}.{blk}.{p}"
            t[base + ".lora_A.weight"] = torch.randn(r, inn, generator=g) * 0.1
            t[base + ".lora_B.weight"] = torch.randn(out, r, generator=g) * 0.1
    return t


@pytest.mark.parametrize("fmt,tol", [("bf16", 2e-2), ("fp8_block", 8e-2)])
def test_merge_adds_scaled_BA_to_the_targeted_rows_only(fmt, tol):
    kw = dict(head_dim=128, n_q=4, n_kv=2, hidden=512, intermediate=1024) if fmt == "fp8_block" else {}
    cfg = tiny("llama", weight_format=fmt, **kw)
    mw = random_weights(cfg, torch.device("cpu"), seed=2, std=0.05)
    before = {n: dequant_linear(getattr(mw.layers[1], n)).clone() for n in ("wqkv", "wo", "w_gate_up", "w_down")}
    untouched = dequant_linear(mw.layers[0].wqkv).clone()
    r, alpha = 4, 8.0
    t = _adapter_tensors(cfg, r, [1], ["q_proj", "v_proj", "up_proj", "down_proj"])
    ad = adapter_from_tensors(t, r, alpha)
    assert merge_lora(mw, ad, weight=0.5) == 4
    hd, q, kv, I = cfg.head_dim, cfg.n_q * cfg.head_dim, cfg.n_kv * cfg.head_dim, cfg.intermediate
    pre = "base_model.model.model.layers.1."
    delta = lambda blk, p: 0.5 * (alpha / r) * (t[pre + f"{blk}.{p}.lora_B.weight"] @ t[pre + f"{blk}.{p}.lora_A.weight"])
    after = dequant_linear(mw.layers[1].wqkv)
    want = before["wqkv"].clone()
    want[:q] += delta("self_attn", "q_proj")
    want[q + kv:] += delta("self_attn", "v_proj")
    assert (after - want).abs().max() <= tol * want.abs().max()
    assert torch.equal(after[q:q + kv], before["wqkv"][q:q + kv]) or fmt == "fp8_block"   # k rows: no adapter
    gu = dequant_linear(mw.layers[1].w_gate_up)
    want = before["w_gate_up"].clone()
    want[I:] += delta("mlp", "up_proj")
    assert (gu - want).abs().max() <= tol * want.abs().max()
    wd = dequant_linear(mw.layers[1].w_down)
    assert (wd - (before["w_down"] + delta("mlp", "down_proj"))).abs().max() <= tol * wd.abs().max()
    assert torch.equal(dequant_linear(mw.layers[1].wo), before["wo"])
    assert torch.equal(dequant_linear(mw.layers[0].wqkv), untouched)


def test_adapter_files_and_refusals(tmp_path):
    from safetensors.torch import save_file

    cfg = tiny("llama", weight_format="bf16")
    t = _adapter_tensors(cfg, 2, [0], ["o_proj"])
    save_file(t, str(tmp_path / "adapter_model.safetensors"))
    (tmp_path / "adapter_config.json").write_text(json.dumps({"r": 2, "lora_alpha": 4, "target_modules": ["o_proj"]}))
    ad = load_lora(str(tmp_path))
    assert ad.r == 2 and ad.scale == 2.0 and list(ad.pairs) == [(0, "o_proj")]
    mw = random_weights(cfg, torch.device("cpu"), seed=2, std=0.05)
    assert merge_lora(mw, ad) == 1
    with pytest.raises(ValueError):
        adapter_from_tensors({"x.layers.0.mlp.up_proj.lora_A.weight": torch.zeros(2, 4)}, 2, 2)
    with pytest.raises(ValueError):
        adapter_from_tensors({"unrelated": torch.zeros(1)}, 2, 2)
    bad = _adapter_tensors(tiny("llama", weight_format="bf16", hidden=128), 2, [0], ["q_proj"])
    with pytest.raises(ValueError):
        merge_lora(mw, adapter_from_tensors(bad, 2, 2))
    q8 = random_weights(tiny("llama", weight_format="q8_0"), torch.device("cpu"), seed=2, std=0.05)
    with pytest.raises(ValueError):
        merge_lora(q8, ad)


@pytest.mark.parametrize("fmt", ["bf16", "fp8_block"])
def test_adapters_are_swapped_in_place_and_a_detach_is_exact(fmt):
    from loken_b200.models.lora import AdapterSet

    kw = dict(head_dim=128, n_q=4, n_kv=2, hidden=512, intermediate=1024) if fmt == "fp8_block" else {}
    cfg = tiny("llama", weight_format=fmt, **kw)
    mw = random_weights(cfg, torch.device("cpu"), seed=2, std=0.05)
    ref = random_weights(cfg, torch.device("cpu"), seed=2, std=0.05)          # the same model, merged the load-time way
    raw = lambda lin: lin.weight if lin.kind == "bf16" else lin.weight.data.view(torch.uint8)
    ptrs = [raw(getattr(l, n)).data_ptr() for l in mw.layers for n in ("wqkv", "wo", "w_gate_up", "w_down")]
    before = [raw(getattr(l, n)).clone() for l in mw.layers for n in ("wqkv", "wo", "w_gate_up", "w_down")]
    ads = {"a": adapter_from_tensors(_adapter_tensors(cfg, 4, [1], ["q_proj", "v_proj", "down_proj"]), 4, 8.0),
           "b": adapter_from_tensors(_adapter_tensors(cfg, 2, [0, 1], ["o_proj", "down_proj"]), 2, 2.0)}
    s = AdapterSet(mw)
    rep = s.apply({"a": 0.5}, loader=ads.__getitem__)
    assert rep["attached"] == ["a"] and rep["projections"] == 2
    merge_lora(ref, ads["a"], 0.5)
    for l, r in zip(mw.layers, ref.layers):
        for n in ("wqkv", "wo", "w_gate_up", "w_down"):
            assert torch.equal(raw(getattr(l, n)), raw(getattr(r, n))), n                 # the same bits as a merge at load
    # the set the model should end up with: a stays at another weight, b joins; both touch layer 1's down projection
    rep = s.apply({"a": 1.0, "b": 0.25}, loader=ads.__getitem__)
    assert rep == {"attached": ["b"], "detached": [], "kept": ["a"], "projections": 5}
    want = dequant_linear(AdapterSet._host_copy(random_weights(cfg, torch.device("cpu"), seed=2, std=0.05).layers[1].w_down))
    for name, w in (("a", 1.0), ("b", 0.25)):
        A, B = ads[name].pairs[(1, "down_proj")]
        want = want + w * ads[name].scale * (B @ A)
    got = dequant_linear(mw.layers[1].w_down)
    assert (got - want).abs().max() <= (2e-2 if fmt == "bf16" else 8e-2) * want.abs().max()
    # everything detached: the stored bytes are back, and no tensor was replaced on the way
    rep = s.apply({}, loader=ads.__getitem__)
    assert rep["detached"] == ["a", "b"] and rep["attached"] == []
    after = [raw(getattr(l, n)) for l in mw.layers for n in ("wqkv", "wo", "w_gate_up", "w_down")]
    assert all(torch.equal(x, y) for x, y in zip(before, after))
    assert ptrs == [t.data_ptr() for t in after]
    # a bad adapter changes nothing
    bad = adapter_from_tensors(_adapter_tensors(cfg, 4, [7], ["q_proj"]), 4, 8.0)
    with pytest.raises(ValueError):
        s.apply({"a": 1.0, "bad": 1.0}, loader={"a": ads["a"], "bad": bad}.__getitem__)
    assert all(torch.equal(x, raw(getattr(l, n))) for x, (l, n) in
               zip(before, [(l, n) for l in mw.layers for n in ("wqkv", "wo", "w_gate_up", "w_down")]))
