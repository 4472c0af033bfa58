"""Plain PyTorch fp32 restatement of the decoder: the oracle the CUDA path is tested against.

It multiplies by the dequantised weights the kernels hold (so weight quantisation is not an
error source) and keeps activations and KV in fp32 (so activation / KV quantisation and bf16
rounding ARE visible as the difference).  Covers dense and MoE layers, GQA, both RoPE
pairings, per-head q/k norm, sliding windows, attention sinks and the clamped gpt-oss SwiGLU
(the model math the reference pins down in `src/inference/model_facts.rs:152-311`,
`generic_transformer/moe_weights.rs:2378-2382`, `hetero.rs:4286-4296`).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..ops.attention import attention_ref
from .config import ModelConfig
from .weights import embed_lookup, head_matrix, ModelWeights, dequant_linear


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, inv_freq, pairing, rope_dim, mscale):
    ang = pos.float()[:, None] * inv_freq[None, :]
    cs, sn = (torch.cos(ang) * mscale)[:, None], (torch.sin(ang) * mscale)[:, None]
    out = x.clone()
    half = rope_dim // 2
    if pairing == 0:
        a, b = x[..., 0:rope_dim:2], x[..., 1:rope_dim:2]
        out[..., 0:rope_dim:2] = a * cs - b * sn
        out[..., 1:rope_dim:2] = a * sn + b * cs
    else:
        a, b = x[..., :half], x[..., half:rope_dim]
        out[..., :half] = a * cs - b * sn
        out[..., half:rope_dim] = b * cs + a * sn
    return out


def glu_ref(g, u, cfg: ModelConfig):
    if cfg.glu_mode == 0:
        return torch.nn.functional.silu(g) * u
    gg = g.clamp(max=cfg.glu_limit)
    uu = u.clamp(-cfg.glu_limit, cfg.glu_limit)
    return gg * torch.sigmoid(cfg.glu_alpha * gg) * (1 + uu)


def route_ref(logits: torch.Tensor, cfg: ModelConfig):
    """Router semantics: returns (expert ids [T, k], weights [T, k])."""
    k = cfg.top_k
    if cfg.router == "softmax_topk":
        top = torch.topk(logits, k, dim=-1)
        return top.indices, torch.softmax(top.values, dim=-1)
    if cfg.router == "softmax":
        p = torch.softmax(logits, dim=-1)
        top = torch.topk(p, k, dim=-1)
        w = top.values / top.values.sum(-1, keepdim=True) if cfg.renorm else top.values
        return top.indices, w
    if cfg.router == "sigmoid":
        p = torch.sigmoid(logits)
        top = torch.topk(p, k, dim=-1)
        w = top.values / top.values.sum(-1, keepdim=True).clamp_min(6.1035156e-5) if cfg.renorm else top.values
        return top.indices, w
    raise ValueError(cfg.router)


def moe_ref(x: torch.Tensor, moe, cfg: ModelConfig) -> torch.Tensor:
    from .moe import dequant_experts

    wr = moe.router_w.float()
    logits = x @ wr.t() + (moe.router_b.float() if moe.router_b is not None else 0)
    ids, wts = route_ref(logits, cfg)
    gu_w, dn_w = dequant_experts(moe)          # [E, 2I, H], [E, H, I] fp32 (all experts)
    out = torch.zeros_like(x)
    I = gu_w.shape[1] // 2
    for t in range(x.shape[0]):
        for j in range(cfg.top_k):
            e = int(ids[t, j])
            gu = gu_w[e] @ x[t]
            if moe.gate_up_b is not None:
                gu = gu + moe.gate_up_b[e].float()
            h = glu_ref(gu[:I], gu[I:], cfg)
            y = dn_w[e] @ h
            if moe.down_b is not None:
                y = y + moe.down_b[e].float()
            out[t] += wts[t, j] * y
    return out


@torch.no_grad()
def forward_ref(w: ModelWeights, tokens: Sequence[int], *, bf16_stream: bool = True, probe=None) -> torch.Tensor:
    """Full causal forward over `tokens`; returns fp32 logits [T, vocab] (single rank only).
    With `bf16_stream` the residual stream is rounded to bf16 where the kernels round it.
    `probe(layer, role, x)` is called with the input rows of every dense linear layer (roles qkv, o,
    gate_up, down): what a calibration pass records."""
    cfg = w.cfg
    assert w.tp_size == 1
    dev = w.embed.device
    T = len(tokens)
    tok = torch.tensor(list(tokens), device=dev, dtype=torch.long)
    pos = torch.arange(T, device=dev)
    rd = lambda t: t.bfloat16().float() if bf16_stream else t
    x = embed_lookup(w, tok) * cfg.embedding_scale
    hd, nq, nkv = cfg.head_dim, cfg.n_q, cfg.n_kv
    rope_dim = cfg.rope_dim or hd
    for il, lw in enumerate(w.layers):
        h = rd(_rms(x, lw.attn_norm, cfg.rms_eps))
        if probe is not None:
            probe(il, "qkv", h)
        qkv = h @ dequant_linear(lw.wqkv).t()
        if lw.wqkv.bias is not None:
            qkv = qkv + lw.wqkv.bias
        qkv = rd(qkv).view(T, nq + 2 * nkv, hd)
        q, k, v = qkv[:, :nq], qkv[:, nq:nq + nkv], qkv[:, nq + nkv:]
        if lw.q_norm is not None and cfg.qk_norm_wide:
            # over the token's whole projection (OLMoE), one weight per column
            q = _rms(q.reshape(T, nq * hd), lw.q_norm, cfg.rms_eps).view(T, nq, hd)
            k = _rms(k.reshape(T, nkv * hd), lw.k_norm, cfg.rms_eps).view(T, nkv, hd)
        elif lw.q_norm is not None:
            q = _rms(q, lw.q_norm, cfg.rms_eps)
            k = _rms(k, lw.k_norm, cfg.rms_eps)
        q = rd(_rope(q, pos, w.inv_freq, cfg.rope_pairing, rope_dim, w.rope_mscale))
        k = rd(_rope(k, pos, w.inv_freq, cfg.rope_pairing, rope_dim, w.rope_mscale))
        a = attention_ref(q, k, v, 0, scale=cfg.softmax_scale(), window=lw.window, sinks=lw.sinks)
        if probe is not None:
            probe(il, "o", rd(a))
        d = rd(a) @ dequant_linear(lw.wo).t()
        if lw.wo.bias is not None:
            d = d + lw.wo.bias
        x = rd(x + rd(d))
        h = rd(_rms(x, lw.ffn_norm, cfg.rms_eps))
        if probe is not None:
            probe(il, "gate_up", h)
        if cfg.is_moe:
            d = moe_ref(h, lw.moe, cfg)
        else:
            gu = rd(h @ dequant_linear(lw.w_gate_up).t())
            I = gu.shape[1] // 2
            act = rd(glu_ref(gu[:, :I], gu[:, I:], cfg))
            if probe is not None:
                probe(il, "down", act)
            d = act @ dequant_linear(lw.w_down).t()
        x = rd(x + rd(d))
    h = rd(_rms(x, w.out_norm, cfg.rms_eps))
    return (h @ head_matrix(w).t()) * cfg.logit_scale
