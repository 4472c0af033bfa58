"""Weight containers and random initialisation of a model (or of one tensor-parallel shard).

Formats a linear layer can be held in on the device:
  bf16       plain [N, K]
  fp8_block  e4m3 + one f32 scale per 128x128 block (block-fp8 safetensors)
  gguf       raw GGUF blocks (Q8_0 / Q4_K / Q6_K / MXFP4) run by the dequant-fused kernels

Tensor-parallel sharding follows the usual column / row split: qkv and gate_up are split along
their output rows (whole heads / whole intermediate columns per rank), o_proj and down along
their input columns; ranks with fewer kv heads than the degree replicate them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..ops import gemm
from .config import ModelConfig


@dataclass
class Linear:
    kind: str                       # bf16 | fp8_block | gguf
    weight: object                  # tensor, Fp8Weight or QuantWeight
    bias: Optional[torch.Tensor] = None   # f32
    n_out: int = 0
    n_in: int = 0

    @property
    def wants_fp8(self) -> bool:
        return self.kind == "fp8_block"


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    wqkv: Linear
    wo: Linear
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    sinks: Optional[torch.Tensor] = None
    w_gate_up: Optional[Linear] = None
    w_down: Optional[Linear] = None
    moe: Optional[object] = None
    window: int = 0


@dataclass
class ModelWeights:
    cfg: ModelConfig
    embed: torch.Tensor             # bf16 [vocab, hidden]
    out_norm: torch.Tensor
    lm_head: torch.Tensor           # bf16 [vocab_local, hidden]
    layers: List[LayerWeights] = field(default_factory=list)
    inv_freq: Optional[torch.Tensor] = None
    rope_mscale: float = 1.0
    tp_rank: int = 0
    tp_size: int = 1
    n_q_local: int = 0
    n_kv_local: int = 0
    vocab_local: int = 0
    vocab_start: int = 0
    layer_range: Optional[tuple] = None      # pipeline stage: the layers held here (others are None)


def make_linear(w: torch.Tensor, fmt: str, bias: Optional[torch.Tensor] = None) -> Linear:
    n_out, n_in = w.shape
    if fmt == "fp8_block":
        return Linear("fp8_block", gemm.quantize_weight_fp8(w), bias, n_out, n_in)
    if fmt == "bf16":
        return Linear("bf16", w.bfloat16().contiguous(), bias, n_out, n_in)
    from ..ops import quant

    # on the GPU the torch encoders write the device planes directly (seconds for billions of values);
    # on the host the C++ encoders of the file formats are used
    q = quant.quantize_weight_torch(w, fmt) if w.is_cuda else quant.quantize_weight(w, fmt)
    return Linear("gguf", q, bias, n_out, n_in)


def dequant_linear(lin: Linear) -> torch.Tensor:
    """fp32 [N, K] view of what the kernels multiply by (for references and tests)."""
    if lin.kind == "bf16":
        return lin.weight.float()
    if lin.kind == "fp8_block":
        return gemm.dequantize_weight_fp8(lin.weight)
    from ..ops import quant

    return quant.dequantize_weight(lin.weight)


def _randn(gen, shape, std, device):
    return torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std


def embed_lookup(w: "ModelWeights", ids: torch.Tensor) -> torch.Tensor:
    """Rows `ids` of the embedding table as fp32, whether the table is bf16 or held in a block format."""
    t = w.embed
    if isinstance(t, torch.Tensor):
        return t[ids.long().to(t.device)].float()
    return t.rows_float(ids)


def head_matrix(w: "ModelWeights") -> torch.Tensor:
    """The output head as fp32 [vocab_local, hidden] (oracles and exports; never the hot path)."""
    t = w.lm_head
    if isinstance(t, torch.Tensor):
        return t.float()
    from ..ops.quant import dequantize_weight

    return dequantize_weight(t)


def linear_format(cfg: ModelConfig, role: str) -> str:
    """Per-tensor storage format.  Q4_K_M mixes Q4_K with Q6_K for `ffn_down` / `attn_v`
    (reference: per-tensor `GgmlDType`, `gguf_file.rs:380-395`); gpt-oss keeps attention in bf16
    and only its experts in MXFP4."""
    f = cfg.weight_format
    if f in ("bf16", "fp8_block"):
        return f
    if f == "mxfp4":
        return "mxfp4" if role == "expert" else "bf16"
    if f == "q4_k_m":
        return "q6_k" if role in ("down", "v") else "q4_k"
    return f


def random_weights(cfg: ModelConfig, device, seed: int = 0, tp_rank: int = 0, tp_size: int = 1,
                   std: float = 0.02, ep_rank: int = 0, ep_size: int = 1, layer_range=None) -> ModelWeights:
    """Random N(0, std) weights of the architecture, quantised to the configured format, holding
    only this rank's tensor-parallel (and expert-parallel) shard.  Every rank draws the full
    tensors from the same seed, so shards of different degrees describe the same model."""
    assert cfg.n_q % tp_size == 0
    hd, H = cfg.head_dim, cfg.hidden
    nql = cfg.n_q // tp_size
    if cfg.n_kv >= tp_size:
        assert cfg.n_kv % tp_size == 0
        nkvl = cfg.n_kv // tp_size
        kv_heads = list(range(tp_rank * nkvl, (tp_rank + 1) * nkvl))
    else:
        nkvl = 1
        kv_heads = [tp_rank * cfg.n_kv // tp_size]
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    embed = _randn(gen, (cfg.vocab, H), std, device).bfloat16()
    if cfg.tie_embeddings:
        head_full = embed
    else:
        head_full = _randn(gen, (cfg.vocab, H), std, device).bfloat16()
    assert cfg.vocab % tp_size == 0 or tp_size == 1
    vl = cfg.vocab // tp_size
    lm_head = head_full[tp_rank * vl:(tp_rank + 1) * vl].contiguous() if tp_size > 1 else head_full
    if tp_size == 1 and cfg.weight_format in ("q8_0", "q4_k", "q4_k_m", "q6_k") and H % 256 == 0 \
            and str(device).startswith("cuda"):
        # as the files of these mixes store them: table and head one step above the matrices (Q6_K under a
        # 4-bit mix, Q8_0 under Q8_0), kept in that format on one rank
        from ..ops.quant import quantize_weight_torch

        tf = "q8_0" if cfg.weight_format == "q8_0" else "q6_k"
        embed = quantize_weight_torch(embed.float(), tf)
        lm_head = embed if cfg.tie_embeddings else quantize_weight_torch(head_full.float(), tf)
    inv, mscale = cfg.rope_tables()
    mw = ModelWeights(cfg, embed, torch.ones(H, device=device), lm_head, [],
                      torch.tensor(inv, dtype=torch.float32, device=device), mscale, tp_rank, tp_size, nql, nkvl, vl,
                      tp_rank * vl)
    qsl = slice(tp_rank * nql * hd, (tp_rank + 1) * nql * hd)
    for il in range(cfg.n_layers):
        wq = _randn(gen, (cfg.n_q * hd, H), std, device)[qsl]
        wk = _randn(gen, (cfg.n_kv * hd, H), std, device).view(cfg.n_kv, hd, H)[kv_heads].reshape(-1, H)
        wv = _randn(gen, (cfg.n_kv * hd, H), std, device).view(cfg.n_kv, hd, H)[kv_heads].reshape(-1, H)
        wqkv = torch.cat([wq, wk, wv], 0)
        bqkv = None
        if cfg.attn_bias:
            bq = _randn(gen, (cfg.n_q * hd,), std, device)[qsl]
            bk = _randn(gen, (cfg.n_kv, hd), std, device)[kv_heads].reshape(-1)
            bv = _randn(gen, (cfg.n_kv, hd), std, device)[kv_heads].reshape(-1)
            bqkv = torch.cat([bq, bk, bv]).contiguous()
        wo = _randn(gen, (H, cfg.n_q * hd), std, device)[:, qsl].contiguous()
        bo = None
        if cfg.attn_bias:
            bo = _randn(gen, (H,), std, device)
            if tp_rank != 0:
                bo = torch.zeros_like(bo)       # the bias joins the sum once
        lw = LayerWeights(
            attn_norm=torch.ones(H, device=device) + _randn(gen, (H,), 0.02, device),
            ffn_norm=torch.ones(H, device=device) + _randn(gen, (H,), 0.02, device),
            wqkv=make_linear(wqkv, linear_format(cfg, "qkv"), bqkv),
            wo=make_linear(wo, linear_format(cfg, "o"), bo),
            window=cfg.layer_window(il))
        del wq, wk, wv, wqkv, wo
        if cfg.qk_norm:
            wq_, wk_ = (cfg.n_q * hd, cfg.n_kv * hd) if cfg.qk_norm_wide else (hd, hd)
            lw.q_norm = torch.ones(wq_, device=device) + _randn(gen, (wq_,), 0.02, device)
            lw.k_norm = torch.ones(wk_, device=device) + _randn(gen, (wk_,), 0.02, device)
        if cfg.sinks:
            lw.sinks = _randn(gen, (cfg.n_q,), 1.0, device)[tp_rank * nql:(tp_rank + 1) * nql].contiguous()
        if cfg.is_moe:
            from .moe import random_moe

            lw.moe = random_moe(cfg, gen, device, std, ep_rank, ep_size, il=il)
        else:
            I = cfg.intermediate
            assert I % tp_size == 0
            il_ = I // tp_size
            isl = slice(tp_rank * il_, (tp_rank + 1) * il_)
            wg = _randn(gen, (I, H), std, device)[isl]
            wu = _randn(gen, (I, H), std, device)[isl]
            lw.w_gate_up = make_linear(torch.cat([wg, wu], 0), linear_format(cfg, "gate_up"))
            del wg, wu
            wd = _randn(gen, (H, I), std, device)[:, isl].contiguous()
            lw.w_down = make_linear(wd, linear_format(cfg, "down"))
            del wd
        # a pipeline stage keeps only its own layers; the others were drawn so every stage sees
        # the same random stream, and are dropped here
        keep = layer_range is None or layer_range[0] <= il < layer_range[1]
        mw.layers.append(lw if keep else None)
    mw.layer_range = layer_range
    return mw
