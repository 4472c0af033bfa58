"""Model files: GGUF -> `ModelWeights` (one tensor-parallel / expert-parallel shard per rank), and
the writer that turns a random-init model into a GGUF file with tokenizer metadata.

Loading keeps quantised tensors in their stored blocks: Q8_0 / Q4_K / Q6_K / MXFP4 payloads are
re-laid for the dequant-fused GEMM without a float round trip; F32 / F16 / BF16 tensors become
bf16 (or block-scaled fp8 when `requant="fp8_block"`).  q/k/v and gate/up are fused at load like
the reference does (`src/inference/generic_transformer/loader.rs:3745`); when the fused parts
are stored in different block formats (Q4_K_M keeps `attn_v` in Q6_K) the fused tensor is
expanded and kept in bf16.  Tensor names follow llama.cpp's GGUF convention
(`token_embd`, `blk.N.attn_q`, `ffn_gate_exps`, ...).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..formats import gguf as G
from ..ops import quant
from .config import ModelConfig
from .moe import MoeWeights
from .weights import LayerWeights, Linear, ModelWeights, linear_format, make_linear

QUANT_TYPES = {G.Q8_0: "q8_0", G.Q4_K: "q4_k", G.Q6_K: "q6_k", G.MXFP4: "mxfp4"}
KEEP_QUANT_TABLES = True    # embedding table and output head of a quantised file stay in their block format on one rank
FMT_TYPES = {v: k for k, v in QUANT_TYPES.items()}


class _Src:
    """One stored 2-D tensor [rows, K] with lazy access to raw blocks or floats."""

    def __init__(self, info: G.TensorInfo):
        self.info = info
        self.rows, self.K = int(np.prod(info.shape[:-1])), int(info.shape[-1])
        self.type = info.ggml_type

    @property
    def quantised(self) -> bool:
        return self.type in QUANT_TYPES

    def floats(self, row_sl: Optional[slice] = None, col_sl: Optional[slice] = None) -> np.ndarray:
        if self.quantised or self.type in (G.F16, G.BF16, G.F32):
            if row_sl is not None and self.quantised:
                raw, rows = self.raw_rows(row_sl)
                x = G.dequantize(raw, self.type, (rows, self.K))
            else:
                x = G.dequantize(self.info.data, self.type, (self.rows, self.K))
                if row_sl is not None:
                    x = x[row_sl]
            return x[:, col_sl] if col_sl is not None else x
        raise ValueError(f"{self.info.name}: unsupported tensor type {G.TYPE_NAMES.get(self.type, self.type)}")

    def raw_rows(self, row_sl: slice) -> Tuple[np.ndarray, int]:
        bv, bb = G.block_info(self.type)
        per_row = self.K // bv * bb
        a = self.info.data.reshape(self.rows, per_row)[row_sl]
        return np.ascontiguousarray(a).reshape(-1), a.shape[0]

    def raw_cols(self, col_sl: slice) -> Tuple[np.ndarray, int]:
        """Raw blocks of a K range; the range must fall on block boundaries."""
        bv, bb = G.block_info(self.type)
        lo, hi = col_sl.start or 0, col_sl.stop if col_sl.stop is not None else self.K
        if lo % bv or hi % bv:
            raise ValueError(f"{self.info.name}: column shard {lo}:{hi} splits a {bv}-value block")
        a = self.info.data.reshape(self.rows, self.K // bv, bb)[:, lo // bv:hi // bv]
        return np.ascontiguousarray(a).reshape(-1), hi - lo


def _linear_from(parts: List[Tuple[_Src, Optional[slice]]], device, requant: Optional[str], bias=None,
                 col_sl: Optional[slice] = None) -> Linear:
    """Stack row slices of stored tensors into one linear layer."""
    types = {s.type for s, _ in parts}
    K = parts[0][0].K if col_sl is None else (col_sl.stop - col_sl.start)
    if len(types) == 1 and parts[0][0].quantised and requant is None and K % 64 == 0:
        ty = parts[0][0].type
        raws, rows = [], 0
        for s, sl in parts:
            if col_sl is not None:
                assert sl is None
                r, _ = s.raw_cols(col_sl)
                n = s.rows
            else:
                r, n = s.raw_rows(sl if sl is not None else slice(None))
            raws.append(r)
            rows += n
        try:
            qw = quant.from_blocks(np.concatenate(raws), ty, rows, K, device)
            return Linear("gguf", qw, bias, rows, K)
        except (ValueError, AssertionError):
            pass        # shapes the fused kernel cannot take: fall through to floats
    w = np.concatenate([s.floats(sl, col_sl) for s, sl in parts], 0)
    t = torch.from_numpy(np.ascontiguousarray(w)).to(device)
    fmt = requant or "bf16"
    if fmt not in ("bf16", "fp8_block") and (K % 256 or t.shape[0] % 16):
        fmt = "bf16"
    if fmt == "fp8_block" and (K % 128 or t.shape[0] % 128):
        fmt = "bf16"
    return make_linear(t, fmt, bias)


def _scale_linear(lin: Linear, mul: float) -> Linear:
    """Folds a multiplier on the layer's output into its weights (Granite's residual multiplier)."""
    if mul == 1.0:
        return lin
    if lin.kind == "bf16":
        lin.weight = (lin.weight.float() * mul).bfloat16()
    elif lin.kind == "gguf":
        quant.scale_weight_(lin.weight, mul)
    else:
        raise NotImplementedError(f"a residual multiplier on {lin.kind} weights")
    if lin.bias is not None:
        lin.bias = lin.bias * mul
    return lin


def _vec(r: G.GGUFReader, name: str, device, sl: Optional[slice] = None) -> Optional[torch.Tensor]:
    if name not in r.tensors:
        return None
    x = r.tensors[name].to_float().reshape(-1)
    if sl is not None:
        x = x[sl]
    return torch.from_numpy(np.ascontiguousarray(x)).to(device=device, dtype=torch.float32)


def load_gguf(path: str, device, *, tp_rank: int = 0, tp_size: int = 1, ep_rank: int = 0, ep_size: int = 1,
              requant: Optional[str] = None, kv_format: Optional[str] = None, name: Optional[str] = None,
              layer_range: Optional[Tuple[int, int]] = None):
    """-> (ModelWeights, meta dict).  The caller builds the tokenizer from `meta`.  With `layer_range`
    only layers [lo, hi) are read (a pipeline segment); the others are None."""
    r = G.GGUFReader(path)
    meta = dict(r.meta)
    if "token_embd.weight" in r.tensors:
        meta["_vocab"] = r.tensors["token_embd.weight"].shape[0]
    cfg = ModelConfig.from_gguf_meta(meta, name or meta.get("general.name", "gguf"))
    if not cfg.vocab:
        cfg.vocab = int(meta["_vocab"])
    if kv_format:
        cfg.kv_format = kv_format
    T = lambda n: _Src(r.tensors[n])
    has = lambda n: n in r.tensors
    hd, H = cfg.head_dim, cfg.hidden
    assert cfg.n_q % tp_size == 0
    nql = cfg.n_q // tp_size
    if cfg.n_kv >= tp_size:
        assert cfg.n_kv % tp_size == 0
        nkvl = cfg.n_kv // tp_size
        kv_lo = tp_rank * nkvl
    else:
        nkvl = 1
        kv_lo = tp_rank * cfg.n_kv // tp_size
    q_sl = slice(tp_rank * nql * hd, (tp_rank + 1) * nql * hd)
    kv_sl = slice(kv_lo * hd, (kv_lo + nkvl) * hd)
    emb = T("token_embd.weight")

    def keep_planes(src: _Src) -> bool:
        """A table or head stays in its block format (decoded row by row in the gather, read by the GEMV up to
        eight token rows) on one rank, when nothing asks for another format and the kernels know the type."""
        return (KEEP_QUANT_TABLES and tp_size == 1 and requant is None and H % 256 == 0
                and src.type in (G.Q8_0, G.Q6_K, G.Q4_K) and str(device).startswith("cuda"))

    if keep_planes(emb):
        from ..ops.quant import from_blocks

        embed = from_blocks(emb.info.data, emb.type, emb.rows, emb.K, device)
    else:
        embed = torch.from_numpy(emb.floats()).to(device).bfloat16()
    if has("output.weight"):
        vl = cfg.vocab // tp_size if tp_size > 1 else cfg.vocab
        v_sl = slice(tp_rank * vl, (tp_rank + 1) * vl)
        osrc = T("output.weight")
        if keep_planes(osrc):
            from ..ops.quant import from_blocks

            lm_head = from_blocks(osrc.info.data, osrc.type, osrc.rows, osrc.K, device)
        else:
            lm_head = torch.from_numpy(osrc.floats(v_sl)).to(device).bfloat16()
    else:
        cfg.tie_embeddings = True
        vl = cfg.vocab // tp_size if tp_size > 1 else cfg.vocab
        lm_head = embed[tp_rank * vl:(tp_rank + 1) * vl].contiguous() if tp_size > 1 else embed
    cfg.attn_bias = cfg.attn_bias or has("blk.0.attn_q.bias")
    cfg.qk_norm = cfg.qk_norm or has("blk.0.attn_q_norm.weight")
    cfg.sinks = cfg.sinks or has("blk.0.attn_sinks.weight")
    cfg.expert_bias = cfg.expert_bias or has("blk.0.ffn_gate_exps.bias")
    first = r.tensors.get("blk.0.attn_q.weight")
    if first is not None:
        cfg.weight_format = requant or QUANT_TYPES.get(first.ggml_type, "bf16")
    inv, mscale = cfg.rope_tables()
    mw = ModelWeights(cfg, embed, _vec(r, "output_norm.weight", device), lm_head, [],
                      torch.tensor(inv, dtype=torch.float32, device=device), mscale, tp_rank, tp_size, nql, nkvl, vl,
                      tp_rank * vl if tp_size > 1 else 0)
    mw.layer_range = tuple(layer_range) if layer_range is not None else None
    # Granite: every block's output is multiplied before it joins the residual stream; folded into the weights
    res_mul = float(meta.get(f"{cfg.arch}.residual_scale", 1.0) or 1.0) if cfg.arch in ("granite", "granitemoe") else 1.0
    for il in range(cfg.n_layers):
        if layer_range is not None and not (layer_range[0] <= il < layer_range[1]):
            mw.layers.append(None)
            continue
        p = f"blk.{il}."
        if has(p + "attn_qkv.weight"):
            s = T(p + "attn_qkv.weight")
            nq, nk = cfg.n_q * hd, cfg.n_kv * hd
            parts = [(s, q_sl), (s, slice(nq + kv_sl.start, nq + kv_sl.stop)),
                     (s, slice(nq + nk + kv_sl.start, nq + nk + kv_sl.stop))]
        else:
            parts = [(T(p + "attn_q.weight"), q_sl), (T(p + "attn_k.weight"), kv_sl), (T(p + "attn_v.weight"), kv_sl)]
        bqkv = None
        if cfg.attn_bias:
            bq, bk, bv = (_vec(r, p + f"attn_{x}.bias", device) for x in "qkv")
            bqkv = torch.cat([bq[q_sl], bk[kv_sl], bv[kv_sl]]).contiguous()
        wqkv = _linear_from(parts, device, requant, bqkv)
        bo = _vec(r, p + "attn_output.bias", device)
        if bo is not None and tp_rank != 0:
            bo = torch.zeros_like(bo)
        wo = _scale_linear(_linear_from([(T(p + "attn_output.weight"), None)], device, requant, bo,
                                        col_sl=q_sl if tp_size > 1 else None), res_mul)
        ffn_norm = _vec(r, p + "ffn_norm.weight", device)
        if ffn_norm is None:
            ffn_norm = _vec(r, p + "post_attention_norm.weight", device)
        lw = LayerWeights(attn_norm=_vec(r, p + "attn_norm.weight", device), ffn_norm=ffn_norm, wqkv=wqkv, wo=wo,
                          window=cfg.layer_window(il))
        lw.q_norm = _vec(r, p + "attn_q_norm.weight", device)
        lw.k_norm = _vec(r, p + "attn_k_norm.weight", device)
        sk = _vec(r, p + "attn_sinks.weight", device)
        if sk is not None:
            lw.sinks = sk[tp_rank * nql:(tp_rank + 1) * nql].contiguous()
        if cfg.is_moe and has(p + "ffn_gate_exps.weight"):
            lw.moe = _load_moe(r, cfg, p, device, ep_rank, ep_size, requant, res_mul)
        else:
            I = cfg.intermediate
            il_ = I // tp_size
            i_sl = slice(tp_rank * il_, (tp_rank + 1) * il_)
            if has(p + "ffn_gate.weight"):
                gu_parts = [(T(p + "ffn_gate.weight"), i_sl), (T(p + "ffn_up.weight"), i_sl)]
            else:           # Phi-3: gate rows, then up rows, in one tensor
                up = T(p + "ffn_up.weight")
                gu_parts = [(up, i_sl), (up, slice(I + i_sl.start, I + i_sl.stop))]
            lw.w_gate_up = _linear_from(gu_parts, device, requant)
            lw.w_down = _scale_linear(_linear_from([(T(p + "ffn_down.weight"), None)], device, requant,
                                                   col_sl=i_sl if tp_size > 1 else None), res_mul)
        mw.layers.append(lw)
    r.close()
    return mw, meta


def _load_moe(r: G.GGUFReader, cfg: ModelConfig, p: str, device, ep_rank: int, ep_size: int,
              requant: Optional[str], out_mul: float = 1.0) -> MoeWeights:
    E, H, I = cfg.n_experts, cfg.hidden, cfg.expert_intermediate
    ecnt = E // ep_size
    elo = ep_rank * ecnt
    router_w = torch.from_numpy(r.tensors[p + "ffn_gate_inp.weight"].to_float().reshape(E, H)).to(device).bfloat16()
    router_b = _vec(r, p + "ffn_gate_inp.bias", device)
    g, u, d = (_Src(r.tensors[p + f"ffn_{x}_exps.weight"]) for x in ("gate", "up", "down"))
    # stacked [E, rows, K] tensors: expert e owns rows e*rows .. (e+1)*rows of the flattened matrix
    parts_gu: List[Tuple[_Src, slice]] = []
    for e in range(elo, elo + ecnt):
        parts_gu += [(g, slice(e * I, (e + 1) * I)), (u, slice(e * I, (e + 1) * I))]
    gu = _linear_from(parts_gu, device, requant)
    dn = _scale_linear(_linear_from([(d, slice(elo * H, (elo + ecnt) * H))], device, requant), out_mul)   # Granite's residual multiplier
    gub = dnb = None
    if (p + "ffn_gate_exps.bias") in r.tensors:
        bg = r.tensors[p + "ffn_gate_exps.bias"].to_float().reshape(E, I)[elo:elo + ecnt]
        bu = r.tensors[p + "ffn_up_exps.bias"].to_float().reshape(E, I)[elo:elo + ecnt]
        gub = torch.from_numpy(np.concatenate([bg, bu], 1)).to(device).contiguous()
        dnb = torch.from_numpy(r.tensors[p + "ffn_down_exps.bias"].to_float().reshape(E, H)[elo:elo + ecnt].copy()
                               ).to(device) * out_mul
    fmt = "bf16" if gu.kind == "bf16" else QUANT_TYPES.get(gu.weight.ggml_type, "gguf")
    return MoeWeights(router_w, router_b, gu.weight, dn.weight, gub, dnb, elo, ecnt, fmt)


# ------------------------------------------------------------------------------ writer
def export_random_gguf(path: str, cfg: ModelConfig, *, seed: int = 0, std: float = 0.02,
                       tokenizer_meta: Optional[Dict[str, object]] = None, threads: int = 8) -> None:
    """Writes a random-init model of `cfg`'s architecture in `cfg.weight_format` (per-tensor types
    as `linear_format` picks them), with the metadata `ModelConfig.from_gguf_meta` reads back.
    Used to produce benchmark and test model files where no checkpoint can be downloaded."""
    rng = np.random.default_rng(seed)
    w = G.GGUFWriter(path)
    a = cfg.arch
    w.add_meta("general.architecture", a)
    w.add_meta("general.name", cfg.name)
    for k, v in ((f"{a}.block_count", cfg.n_layers), (f"{a}.embedding_length", cfg.hidden),
                 (f"{a}.attention.head_count", cfg.n_q), (f"{a}.attention.head_count_kv", cfg.n_kv),
                 (f"{a}.attention.key_length", cfg.head_dim), (f"{a}.feed_forward_length", cfg.intermediate),
                 (f"{a}.context_length", cfg.context_length), (f"{a}.vocab_size", cfg.vocab)):
        w.add_meta(k, int(v))
    w.add_meta(f"{a}.rope.freq_base", float(cfg.rope_theta))
    w.add_meta(f"{a}.attention.layer_norm_rms_epsilon", float(cfg.rms_eps))
    if cfg.sliding_window:
        w.add_meta(f"{a}.attention.sliding_window", int(cfg.sliding_window))
    if cfg.is_moe:
        w.add_meta(f"{a}.expert_count", int(cfg.n_experts))
        w.add_meta(f"{a}.expert_used_count", int(cfg.top_k))
        w.add_meta(f"{a}.expert_feed_forward_length", int(cfg.expert_intermediate))
    sc = cfg.rope_scaling
    if sc is not None and sc.kind:
        w.add_meta(f"{a}.rope.scaling.type", sc.kind)
        w.add_meta(f"{a}.rope.scaling.factor", float(sc.factor))
        w.add_meta(f"{a}.rope.scaling.original_context_length", int(sc.original_context))
    for k, v in (tokenizer_meta or {}).items():
        w.add_meta(k, v)

    def ty(role: str, K: int) -> int:
        f = linear_format(cfg, role)
        t = FMT_TYPES.get(f, G.BF16 if f in ("bf16", "fp8_block") else G.F32)
        bv, _ = G.block_info(t) if t in QUANT_TYPES else (1, 0)
        return t if K % bv == 0 else G.BF16

    def mat(name: str, rows: int, K: int, role: str, scale: float = 1.0):
        x = (rng.standard_normal((rows, K), dtype=np.float32) * (std * scale))
        w.add_tensor(name, x, ty(role, K))

    def vec(name: str, n: int, centre: float = 1.0, spread: float = 0.02):
        w.add_tensor(name, (centre + rng.standard_normal(n, dtype=np.float32) * spread).astype(np.float32), G.F32)

    hd, H = cfg.head_dim, cfg.hidden
    mat("token_embd.weight", cfg.vocab, H, "embed")
    vec("output_norm.weight", H)
    if not cfg.tie_embeddings:
        mat("output.weight", cfg.vocab, H, "embed")
    for il in range(cfg.n_layers):
        p = f"blk.{il}."
        vec(p + "attn_norm.weight", H)
        mat(p + "attn_q.weight", cfg.n_q * hd, H, "qkv")
        mat(p + "attn_k.weight", cfg.n_kv * hd, H, "qkv")
        mat(p + "attn_v.weight", cfg.n_kv * hd, H, "v")
        mat(p + "attn_output.weight", H, cfg.n_q * hd, "o")
        if cfg.attn_bias:
            vec(p + "attn_q.bias", cfg.n_q * hd, 0.0, std)
            vec(p + "attn_k.bias", cfg.n_kv * hd, 0.0, std)
            vec(p + "attn_v.bias", cfg.n_kv * hd, 0.0, std)
            vec(p + "attn_output.bias", H, 0.0, std)
        if cfg.qk_norm:
            vec(p + "attn_q_norm.weight", cfg.n_q * hd if cfg.qk_norm_wide else hd)
            vec(p + "attn_k_norm.weight", cfg.n_kv * hd if cfg.qk_norm_wide else hd)
        if cfg.sinks:
            vec(p + "attn_sinks.weight", cfg.n_q, 0.0, 1.0)
        vec(p + "ffn_norm.weight", H)
        if cfg.is_moe:
            E, I = cfg.n_experts, cfg.expert_intermediate
            mat(p + "ffn_gate_inp.weight", E, H, "router", 4.0)
            for nm, rows, K in (("gate", E * I, H), ("up", E * I, H), ("down", E * H, I)):
                arr = rng.standard_normal((rows, K), dtype=np.float32) * std
                t = ty("expert", K)
                raw = G.quantize(arr, t, threads) if t != G.F32 else arr.reshape(-1)
                w.add_tensor(p + f"ffn_{nm}_exps.weight", _ShapeOnly((E, rows // E, K)), t, raw=raw)
            if cfg.expert_bias:
                vec(p + "ffn_gate_inp.bias", E, 0.0, std)
                for nm, n in (("gate", E * I), ("up", E * I), ("down", E * H)):
                    w.add_tensor(p + f"ffn_{nm}_exps.bias",
                                 (rng.standard_normal((E, n // E), dtype=np.float32) * std), G.F32)
        else:
            I = cfg.intermediate
            mat(p + "ffn_gate.weight", I, H, "gate_up")
            mat(p + "ffn_up.weight", I, H, "gate_up")
            mat(p + "ffn_down.weight", H, I, "down")
    w.close()


class _ShapeOnly:
    """Stands in for an array when only its shape is needed (the payload is given raw)."""

    def __init__(self, shape):
        self.shape = tuple(shape)


def peek_config(model: str) -> ModelConfig:
    """The shape of `model` (a Hugging Face checkpoint directory, a GGUF file or the name of a built-in
    shape) without reading a tensor: what has to be known before the weights load, e.g. to size the
    symmetric heap of a tensor-parallel group."""
    import json
    import os

    if os.path.isdir(model) and os.path.exists(os.path.join(model, "config.json")):
        from .loader_hf import config_from_hf

        with open(os.path.join(model, "config.json")) as f:
            return config_from_hf(json.load(f), os.path.basename(os.path.normpath(model)))
    if os.path.exists(model):
        from ..formats.gguf import GGUFReader

        meta = GGUFReader(model).meta
        return ModelConfig.from_gguf_meta(meta, meta.get("general.name", "gguf"))
    from .config import get_config

    return get_config(model)
