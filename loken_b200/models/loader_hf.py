"""Hugging Face safetensors checkpoints of Llama-family models, including block-fp8 ones.

Block-fp8 layout (`src/inference/generic_transformer/dense.rs:221`, `:314`;
`src/tensor/blockscaled/fp8.rs:1-9`): `<stem>.weight` in e4m3 with `<stem>.weight_scale_inv`, one
f32 per `quantization_config.weight_block_size` tile (128 x 128), partial edge tiles allowed.
Such tensors are kept as they are (the GEMM consumes e4m3 + block scales); row-parallel slices
must fall on tile boundaries.  q/k/v and gate/up are fused at load; bf16 / f16 / f32 tensors
become bf16 (or are re-encoded to block-fp8 with `requant="fp8_block"`).
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, Optional

import torch

from ..ops import gemm
from .config import ARCH_FACTS, ModelConfig, RopeScaling
from .weights import LayerWeights, Linear, ModelWeights, make_linear

HF_ARCH = {"LlamaForCausalLM": "llama", "MistralForCausalLM": "mistral", "Qwen2ForCausalLM": "qwen2",
           "Qwen3ForCausalLM": "qwen3", "GptOssForCausalLM": "gpt-oss", "MixtralForCausalLM": "mixtral",
           "Qwen3MoeForCausalLM": "qwen3moe", "Phi3ForCausalLM": "phi3", "GraniteForCausalLM": "granite",
           "OlmoeForCausalLM": "olmoe", "GraniteMoeForCausalLM": "granitemoe",
           # families that are one of the above in every respect the engine sees (checked against transformers):
           # GLM = fused gate / up, partial rotary, q / k / v biases; ERNIE 4.5 and Helium = Llama; Seed-OSS = Qwen2
           "GlmForCausalLM": "phi3", "Ernie4_5ForCausalLM": "llama", "HeliumForCausalLM": "llama",
           "SeedOssForCausalLM": "qwen2"}
# of which these rotate adjacent lanes (2i, 2i+1) instead of the half-split pairs the library layout usually means
HF_ADJACENT_ROPE = {"GlmForCausalLM", "Ernie4_5ForCausalLM", "HeliumForCausalLM"}
# mixture families that store one tensor per expert and matrix: (router, expert stem, gate, up, down)
HF_EXPERT_NAMES = {
    "mixtral": ("block_sparse_moe.gate", "block_sparse_moe.experts.{e}.", "w1", "w3", "w2"),
    "qwen3moe": ("mlp.gate", "mlp.experts.{e}.", "gate_proj", "up_proj", "down_proj"),
    "olmoe": ("mlp.gate", "mlp.experts.{e}.", "gate_proj", "up_proj", "down_proj"),
}


def config_from_hf(cfg: dict, name: str = "hf") -> ModelConfig:
    arch = HF_ARCH.get((cfg.get("architectures") or ["LlamaForCausalLM"])[0], "llama")
    facts = ARCH_FACTS.get(arch, {})
    n_q = int(cfg["num_attention_heads"])
    hidden = int(cfg["hidden_size"])
    sc = RopeScaling()
    # `rope_scaling` in older files, `rope_parameters` (which also carries the base) in newer ones
    rs = cfg.get("rope_scaling") or cfg.get("rope_parameters") or {}
    theta = cfg.get("rope_theta") or rs.get("rope_theta")
    kind = rs.get("rope_type", rs.get("type"))
    if kind in ("linear", "yarn"):
        sc = RopeScaling(kind=kind, factor=float(rs.get("factor", 1.0)),
                         original_context=int(rs.get("original_max_position_embeddings", 8192)),
                         beta_fast=float(rs.get("beta_fast") or 32.0), beta_slow=float(rs.get("beta_slow") or 1.0),
                         attn_factor=rs.get("attention_factor"), truncate=bool(rs.get("truncate", True)))
        if kind == "yarn" and sc.attn_factor is None and sc.factor > 1:
            import math

            sc.attn_factor = 0.1 * math.log(sc.factor) + 1.0        # what these files mean when they say nothing
    elif kind == "llama3":
        sc = RopeScaling(kind="llama3", factor=float(rs.get("factor", 8.0)),
                         original_context=int(rs.get("original_max_position_embeddings", 8192)),
                         low_freq_factor=float(rs.get("low_freq_factor", 1.0)),
                         high_freq_factor=float(rs.get("high_freq_factor", 4.0)))
    qc = cfg.get("quantization_config") or {}
    fmt = "fp8_block" if qc.get("quant_method") == "fp8" and qc.get("weight_block_size") else "bf16"
    if arch == "gpt-oss":
        # mixture of experts with MXFP4 expert matrices (`*_blocks` / `*_scales`), attention sinks, a sliding
        # window on alternate layers, YaRN, biases everywhere, the clamped SwiGLU
        if kind == "yarn":
            sc = RopeScaling(kind="yarn", factor=float(rs.get("factor", 32.0)),
                             original_context=int(rs.get("original_max_position_embeddings", 4096)),
                             beta_fast=float(rs.get("beta_fast", 32.0)), beta_slow=float(rs.get("beta_slow", 1.0)),
                             attn_factor=rs.get("attention_factor"), truncate=bool(rs.get("truncate", True)))
        out = ModelConfig(name=name, arch=arch, n_layers=int(cfg["num_hidden_layers"]), hidden=hidden, n_q=n_q,
                          n_kv=int(cfg.get("num_key_value_heads", n_q)), head_dim=int(cfg.get("head_dim") or hidden // n_q),
                          intermediate=int(cfg["intermediate_size"]), vocab=int(cfg["vocab_size"]),
                          rope_theta=float(theta or 150000.0), rope_pairing=1, rope_scaling=sc,
                          rms_eps=float(cfg.get("rms_norm_eps", 1e-5)), attn_bias=True,
                          context_length=int(cfg.get("max_position_embeddings", 131072)),
                          tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
                          sliding_window=int(cfg.get("sliding_window") or 128), swa_period=facts.get("swa_period", 2),
                          sinks=True, n_experts=int(cfg.get("num_local_experts") or cfg.get("num_experts")),
                          top_k=int(cfg.get("num_experts_per_tok") or cfg.get("experts_per_token") or 4),
                          expert_intermediate=int(cfg["intermediate_size"]), router=facts.get("router", "softmax_topk"),
                          expert_bias=True, glu_mode=1, glu_alpha=facts.get("glu_alpha", 1.702),
                          glu_limit=float(cfg.get("swiglu_limit", facts.get("glu_limit", 7.0))),
                          weight_format="mxfp4" if qc.get("quant_method") == "mxfp4" else "bf16")
        kinds = cfg.get("layer_types")
        if isinstance(kinds, list) and len(kinds) == out.n_layers:
            out.swa_layers = [k == "sliding_attention" for k in kinds]
        return out
    extra = {}
    if kind in ("longrope", "su"):
        # Phi-3 long-context files: one divisor per rotary pair, the long list once the context exceeds the
        # length the model was trained at (chosen for the configured context, not per sequence), and a
        # magnitude factor on cos / sin
        import math

        orig = int(cfg.get("original_max_position_embeddings") or rs.get("original_max_position_embeddings") or 4096)
        ctx = int(cfg.get("max_position_embeddings", orig))
        extra["rope_freq_factors"] = [float(x) for x in (rs["long_factor"] if ctx > orig else rs["short_factor"])]
        f = rs.get("attention_factor")
        if f is None:
            f = math.sqrt(1.0 + math.log(ctx / orig) / math.log(orig)) if ctx > orig else 1.0
        sc = RopeScaling(kind="none", attn_factor=float(f))
    if arch in ("granite", "granitemoe"):
        # four multipliers: on the embeddings, on the attention scores (instead of 1 / sqrt(head_dim)), on every
        # block's output before it joins the residual stream (folded into the o and down projections at load),
        # and a divisor of the logits
        extra.update(embedding_scale=float(cfg.get("embedding_multiplier", 1.0)),
                     attn_scale=float(cfg["attention_multiplier"]) if cfg.get("attention_multiplier") else None,
                     logit_scale=1.0 / float(cfg.get("logits_scaling", 1.0) or 1.0))
    if cfg.get("partial_rotary_factor") not in (None, 1.0):
        extra["rope_dim"] = int(float(cfg["partial_rotary_factor"]) * int(cfg.get("head_dim") or hidden // n_q))
    moe = extra
    if arch == "granitemoe":
        # the k best router logits are chosen first and the softmax runs over those alone
        moe = dict(extra, n_experts=int(cfg["num_local_experts"]), top_k=int(cfg.get("num_experts_per_tok", 2)),
                   expert_intermediate=int(cfg["intermediate_size"]), router="softmax_topk", renorm=True)
    if arch in HF_EXPERT_NAMES:
        # softmax over all experts, the best k kept (and, unless the file says otherwise, renormalised)
        n_exp = int(cfg.get("num_local_experts") or cfg.get("num_experts"))
        moe = dict(extra, n_experts=n_exp, top_k=int(cfg.get("num_experts_per_tok", 2)),
                   expert_intermediate=int(cfg.get("moe_intermediate_size") or cfg["intermediate_size"]),
                   router=facts.get("router", "softmax"),
                   renorm=bool(cfg.get("norm_topk_prob", arch == "qwen3moe")) if arch in ("qwen3moe", "olmoe")
                   else facts.get("renorm", True), qk_norm_wide=facts.get("qk_norm_wide", False))
        if any(int(x) for x in (cfg.get("mlp_only_layers") or [])) or int(cfg.get("decoder_sparse_step", 1) or 1) != 1:
            raise ValueError("checkpoints that mix dense and mixture layers are not read")
    # HF checkpoints store q/k in the half-split (NeoX) layout whatever the family
    return ModelConfig(name=name, arch=arch, n_layers=int(cfg["num_hidden_layers"]), hidden=hidden, n_q=n_q, **moe,
                       sliding_window=int(cfg.get("sliding_window") or 0) if arch in ("mistral", "mixtral") else 0,
                       n_kv=int(cfg.get("num_key_value_heads", n_q)),
                       head_dim=int(cfg.get("head_dim") or hidden // n_q),
                       intermediate=int(cfg["intermediate_size"]), vocab=int(cfg["vocab_size"]),
                       rope_theta=float(theta or 10000.0), rope_pairing=1, rope_scaling=sc,
                       rms_eps=float(cfg.get("rms_norm_eps", 1e-5)), qk_norm=facts.get("qk_norm", False),
                       attn_bias=bool(cfg.get("attention_bias", facts.get("attn_bias", False))),
                       context_length=int(cfg.get("max_position_embeddings", 8192)),
                       tie_embeddings=bool(cfg.get("tie_word_embeddings", False)), weight_format=fmt)


class _Shards:
    """The tensors of a checkpoint directory by name: safetensors shards, or (older repositories)
    `pytorch_model*.bin` files read without unpickling code (`formats/pth.py`)."""

    def __init__(self, directory: str):
        from safetensors import safe_open

        self.files = sorted(glob.glob(os.path.join(directory, "*.safetensors")))
        if self.files:
            self.handles = [safe_open(f, framework="pt", device="cpu") for f in self.files]
        else:
            from ..formats.pth import PthReader

            self.files = sorted(glob.glob(os.path.join(directory, "pytorch_model*.bin")))
            if not self.files:
                raise FileNotFoundError(f"no .safetensors or pytorch_model*.bin files in {directory}")
            self.handles = [PthReader(f) for f in self.files]
        self.where: Dict[str, int] = {}
        for i, h in enumerate(self.handles):
            for k in h.keys():
                self.where[k] = i

    def has(self, name: str) -> bool:
        return name in self.where

    def get(self, name: str) -> torch.Tensor:
        return self.handles[self.where[name]].get_tensor(name)


def config_from_native_params(p: dict) -> dict:
    """A vendor's own release (`params.json` beside `consolidated*.safetensors`) as the configuration dict the
    library layout carries: the text model is the llama family's (reference: `src/inference/load/awq_loader.rs:246-321`).
    A `yarn` block becomes the rope block (`beta` / `alpha` are the fast / slow betas)."""
    for k in ("dim", "n_layers", "n_heads", "hidden_dim", "vocab_size"):
        if k not in p:
            raise ValueError(f"params.json: missing {k}")
    hf = {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "hidden_size": int(p["dim"]),
          "num_hidden_layers": int(p["n_layers"]), "num_attention_heads": int(p["n_heads"]),
          "num_key_value_heads": int(p.get("n_kv_heads") or p["n_heads"]), "intermediate_size": int(p["hidden_dim"]),
          "vocab_size": int(p["vocab_size"]), "rope_theta": float(p.get("rope_theta", 10000.0)),
          "rms_norm_eps": float(p.get("norm_eps", 1e-5)), "tie_word_embeddings": bool(p.get("tied_embeddings", False)),
          "max_position_embeddings": int(p.get("max_seq_len") or p.get("max_position_embeddings") or 32768)}
    if p.get("head_dim"):
        hf["head_dim"] = int(p["head_dim"])
    if p.get("sliding_window"):
        hf["sliding_window"] = int(p["sliding_window"])
    y = p.get("yarn")
    if isinstance(y, dict):
        hf["rope_parameters"] = {"rope_type": "yarn", "rope_theta": hf["rope_theta"], "factor": float(y.get("factor", 1.0)),
                                 "original_max_position_embeddings": int(y.get("original_max_position_embeddings", 8192)),
                                 "beta_fast": float(y.get("beta", 32.0)), "beta_slow": float(y.get("alpha", 1.0)), "mscale": 1.0,
                                 "mscale_all_dim": 0.0 if y.get("apply_scale") else 1.0}
    return hf


_NATIVE_NAMES = (("model.embed_tokens.", "tok_embeddings."), ("model.norm.", "norm."), ("lm_head.", "output."),
                 (".self_attn.q_proj.", ".attention.wq."), (".self_attn.k_proj.", ".attention.wk."),
                 (".self_attn.v_proj.", ".attention.wv."), (".self_attn.o_proj.", ".attention.wo."),
                 (".mlp.gate_proj.", ".feed_forward.w1."), (".mlp.up_proj.", ".feed_forward.w3."),
                 (".mlp.down_proj.", ".feed_forward.w2."), (".input_layernorm.", ".attention_norm."),
                 (".post_attention_layernorm.", ".ffn_norm."), ("model.layers.", "layers."))


class _NativeShards(_Shards):
    """`consolidated*.safetensors` under the names the rest of the loader asks for."""

    def __init__(self, directory: str):
        from safetensors import safe_open

        self.files = sorted(glob.glob(os.path.join(directory, "consolidated*.safetensors")))
        if not self.files:
            raise FileNotFoundError(f"params.json without consolidated*.safetensors in {directory}")
        self.handles = [safe_open(f, framework="pt", device="cpu") for f in self.files]
        self.where = {}
        for i, h in enumerate(self.handles):
            for k in h.keys():
                self.where[k] = i

    @staticmethod
    def _native(name: str) -> str:
        for lib, nat in _NATIVE_NAMES:
            name = name.replace(lib, nat)
        return name

    def has(self, name: str) -> bool:
        return self._native(name) in self.where

    def get(self, name: str) -> torch.Tensor:
        n = self._native(name)
        return self.handles[self.where[n]].get_tensor(n)


def _fp8_linear(sh: _Shards, stems, rows, device, col: Optional[slice] = None, bias=None) -> Optional[Linear]:
    """Stacks row slices of block-fp8 tensors; None when a slice does not fall on tile boundaries."""
    datas, scales = [], []
    for stem, sl in zip(stems, rows):
        w = sh.get(stem + ".weight")
        s = sh.get(stem + ".weight_scale_inv").float()
        lo, hi = (sl.start or 0, sl.stop if sl.stop is not None else w.shape[0]) if sl is not None else (0, w.shape[0])
        if lo % 128 or (hi % 128 and hi != w.shape[0]):
            return None
        w, s = w[lo:hi], s[lo // 128:(hi + 127) // 128]
        if col is not None:
            if col.start % 128 or (col.stop % 128 and col.stop != w.shape[1]):
                return None
            w, s = w[:, col], s[:, col.start // 128:(col.stop + 127) // 128]
        if w.shape[0] % 128 and len(stems) > 1:
            return None            # a partial edge tile in the middle of a fused tensor
        datas.append(w)
        scales.append(s)
    data = torch.cat(datas, 0).contiguous().to(device)
    scale = torch.cat(scales, 0).contiguous().to(device)
    return Linear("fp8_block", gemm.Fp8Weight(data, scale), bias, data.shape[0], data.shape[1])


AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)     # nibble i of a packed int32 holds output column 8 j + AWQ_ORDER[i]


def awq_unpack(t: torch.Tensor) -> torch.Tensor:
    """int32 [rows, n / 8] -> int32 [rows, n]: eight 4-bit values per word in AWQ's column order."""
    rows, packed = t.shape
    out = torch.empty(rows, packed * 8, dtype=torch.int32)
    t = t.to(torch.int32)
    for i, col in enumerate(AWQ_ORDER):
        out[:, col::8] = (t >> (4 * i)) & 0xF
    return out


def awq_planes(sh: "_Shards", stems, rows, device, bias=None) -> Optional[Linear]:
    """AWQ tensors with groups of 128 kept as 4-bit planes (`ops/quant.py: from_awq`): up to eight token rows run
    as the dp4a GEMV on the stored codes, more are decoded once per call for the bf16 GEMM.  None when a tensor is
    not AWQ or its groups are not 128 wide."""
    from ..ops import quant as Q

    qs, zs, ss = [], [], []
    for stem, sl in zip(stems, rows):
        if not sh.has(stem + ".qweight"):
            return None
        q = awq_unpack(sh.get(stem + ".qweight").cpu())               # [in, out]
        z = awq_unpack(sh.get(stem + ".qzeros").cpu())                # [in / g, out]
        s = sh.get(stem + ".scales").cpu()                            # [in / g, out]
        if q.shape[0] // z.shape[0] != 128 or q.shape[0] % 128:
            return None
        q, z, s = q.t(), z.t(), s.t()                                 # rows = output features
        if sl is not None:
            q, z, s = q[sl], z[sl], s[sl]
        qs.append(q)
        zs.append(z)
        ss.append(s)
    w = Q.from_awq(torch.cat(qs, 0).contiguous(), torch.cat(zs, 0).contiguous(), torch.cat(ss, 0).contiguous(), device)
    return Linear("gguf", w, bias, w.rows, w.K)


def awq_dequant(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """AutoAWQ "gemm" tensors -> float weight [out, in]: qweight int32 [in, out / 8], qzeros int32
    [in / g, out / 8], scales f16 [in / g, out]; w = (q - zero) * scale with 4-bit q and zero."""
    unpack = awq_unpack
    q = unpack(qweight.cpu())
    z = unpack(qzeros.cpu())
    n_in, n_out = q.shape
    g = n_in // z.shape[0]
    w = (q - z.repeat_interleave(g, 0)).float() * scales.cpu().float().repeat_interleave(g, 0)
    return w.t().contiguous()


def _float_rows(sh: _Shards, stem: str, sl, col=None) -> torch.Tensor:
    if not sh.has(stem + ".weight") and sh.has(stem + ".qweight"):
        # AWQ int4 expanded to floats: the path of tensor-parallel shards, of another target format and of
        # group sizes other than 128 (otherwise `awq_planes` keeps the 4-bit codes)
        w = awq_dequant(sh.get(stem + ".qweight"), sh.get(stem + ".qzeros"), sh.get(stem + ".scales"))
        if sl is not None:
            w = w[sl]
        return w[:, col] if col is not None else w
    w = sh.get(stem + ".weight")
    if w.dtype == torch.float8_e4m3fn:
        s = sh.get(stem + ".weight_scale_inv").float()
        w = w.float() * s.repeat_interleave(128, 0)[:w.shape[0]].repeat_interleave(128, 1)[:, :w.shape[1]]
    w = w.float()
    if sl is not None:
        w = w[sl]
    return w[:, col] if col is not None else w


def _oss_experts(sh: _Shards, stem: str, what: str, cfg: ModelConfig, elo: int, ecnt: int, device, requant):
    """One stacked expert matrix of a gpt-oss checkpoint -> (weight, bias) in this library's layout.

    `what` = "gate_up" ([E, 2I, H]: rows alternate gate_0, up_0, gate_1, ...; here every expert's gate rows
    come first, then its up rows) or "down" ([E, H, I]).  MXFP4 files hold `<name>_blocks` uint8
    [E, rows, K / 32, 16] (two values per byte, the even one in the low nibble: this library's own nibble
    plane) and `<name>_scales` uint8 [E, rows, K / 32] (E8M0); bf16 files hold `<name>` as [E, K, rows]."""
    from ..ops import quant as Q

    name = stem + ("gate_up_proj" if what == "gate_up" else "down_proj")
    E, H, I = cfg.n_experts, cfg.hidden, cfg.expert_intermediate
    rows, K = (2 * I, H) if what == "gate_up" else (H, I)
    bias = sh.get(name + "_bias")[elo:elo + ecnt].float() if sh.has(name + "_bias") else None
    if what == "gate_up" and bias is not None:
        bias = torch.cat([bias[:, 0::2], bias[:, 1::2]], 1)
    if sh.has(name + "_blocks"):
        blocks = sh.get(name + "_blocks")[elo:elo + ecnt]                 # [e, rows, K/32, 16]
        scales = sh.get(name + "_scales")[elo:elo + ecnt]                 # [e, rows, K/32]
        if tuple(blocks.shape[1:]) != (rows, K // 32, 16):
            raise ValueError(f"{name}_blocks has shape {tuple(blocks.shape)}, expected [E, {rows}, {K // 32}, 16]")
        codes = blocks.reshape(ecnt, rows, K // 2)
        if what == "gate_up":
            codes = torch.cat([codes[:, 0::2], codes[:, 1::2]], 1)
            scales = torch.cat([scales[:, 0::2], scales[:, 1::2]], 1)
        if requant in (None, "mxfp4") and K % 32 == 0:
            ex = torch.zeros(ecnt * rows, Q.mx_sf_pitch(K), dtype=torch.uint8)
            ex[:, :K // 32] = scales.reshape(ecnt * rows, K // 32)
            from ..formats import gguf as G

            w = Q.QuantWeight(Q.AQ_MX4, G.MXFP4, ecnt * rows, K, codes.reshape(ecnt * rows, K // 2).contiguous().to(device),
                              ex.to(device))
            return w, (bias.to(device).contiguous() if bias is not None else None), "mxfp4"
        # another target format: decode the nibbles (E2M1 values times 2^(e - 127)) and re-encode
        lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6])
        c = codes.reshape(ecnt * rows, K // 2)
        vals = torch.stack([lut[(c & 0xF).long()], lut[(c >> 4).long()]], -1).reshape(ecnt * rows, K)
        dense = vals * torch.exp2(scales.reshape(ecnt * rows, K // 32).float() - 127.0).repeat_interleave(32, 1)
    else:
        dense = sh.get(name)[elo:elo + ecnt].float().transpose(1, 2)     # [e, rows, K]
        if what == "gate_up":
            dense = torch.cat([dense[:, 0::2], dense[:, 1::2]], 1)
        dense = dense.reshape(ecnt * rows, K)
    fmt = requant or "bf16"
    w = dense.to(device).bfloat16() if fmt == "bf16" else Q.quantize_weight(dense.to(device), fmt)
    return w, (bias.to(device).contiguous() if bias is not None else None), fmt


def _stacked_experts(sh: _Shards, layer_stem: str, cfg: ModelConfig, elo: int, ecnt: int, device, requant):
    """Experts stored one tensor per expert and matrix (Mixtral: w1 / w3 / w2; Qwen3-MoE: gate_proj / up_proj /
    down_proj) -> this library's stacked layout: [E_local * 2I, H] with every expert's gate rows first, then
    its up rows, and [E_local * H, I]."""
    from ..ops import quant as Q
    from .moe import MoeWeights

    router, stem, gname, uname, dname = HF_EXPERT_NAMES[cfg.arch]
    gu, dn = [], []
    for e in range(elo, elo + ecnt):
        es = layer_stem + stem.format(e=e)
        gu += [sh.get(es + gname + ".weight").float(), sh.get(es + uname + ".weight").float()]
        dn.append(sh.get(es + dname + ".weight").float())
    gu, dn = torch.cat(gu, 0), torch.cat(dn, 0)
    fmt = requant if requant in ("mxfp4", "q8_0", "q4_k", "q6_k") else "bf16"
    conv = (lambda w: w.to(device).bfloat16()) if fmt == "bf16" else (lambda w: Q.quantize_weight(w.to(device), fmt))
    return MoeWeights(sh.get(layer_stem + router + ".weight").to(device).bfloat16(), None, conv(gu), conv(dn), None, None,
                      elo, ecnt, fmt)


def load_hf(directory: str, device, *, tp_rank: int = 0, tp_size: int = 1, requant: Optional[str] = None,
            kv_format: Optional[str] = None):
    """-> (ModelWeights, hf config dict).  Under tensor parallelism a mixture model's experts are split
    over the same ranks (expert-parallel degree = tensor-parallel degree)."""
    native = not os.path.exists(os.path.join(directory, "config.json")) and os.path.exists(os.path.join(directory, "params.json"))
    if native:
        with open(os.path.join(directory, "params.json")) as f:
            hf = config_from_native_params(json.load(f))
    else:
        with open(os.path.join(directory, "config.json")) as f:
            hf = json.load(f)
    cfg = config_from_hf(hf, os.path.basename(os.path.normpath(directory)))
    if native or (hf.get("architectures") or [""])[0] in HF_ADJACENT_ROPE:
        cfg.rope_pairing = 0        # the vendor's own files, and these families, keep q / k rows in adjacent-pair order
    if kv_format:
        cfg.kv_format = kv_format
    if requant and not cfg.is_moe:
        cfg.weight_format = requant
    sh = _NativeShards(directory) if native else _Shards(directory)
    hd, H = cfg.head_dim, cfg.hidden
    nql = cfg.n_q // tp_size
    nkvl = max(1, cfg.n_kv // tp_size)
    kv_lo = (tp_rank * cfg.n_kv // tp_size) if cfg.n_kv < tp_size else tp_rank * nkvl
    q_sl = slice(tp_rank * nql * hd, (tp_rank + 1) * nql * hd)
    kv_sl = slice(kv_lo * hd, (kv_lo + nkvl) * hd)
    il_ = cfg.intermediate // tp_size
    i_sl = slice(tp_rank * il_, (tp_rank + 1) * il_)
    vec = lambda n: sh.get(n).float().to(device)
    embed = sh.get("model.embed_tokens.weight").to(device).bfloat16()
    vl = cfg.vocab // tp_size if tp_size > 1 else cfg.vocab
    head = sh.get("lm_head.weight") if sh.has("lm_head.weight") else sh.get("model.embed_tokens.weight")
    lm_head = head[tp_rank * vl:(tp_rank + 1) * vl].to(device).bfloat16().contiguous() if tp_size > 1 \
        else head.to(device).bfloat16()
    inv, mscale = cfg.rope_tables()
    mw = ModelWeights(cfg, embed, vec("model.norm.weight"), lm_head, [],
                      torch.tensor(inv, dtype=torch.float32, device=device), mscale, tp_rank, tp_size, nql, nkvl, vl,
                      tp_rank * vl if tp_size > 1 else 0)

    # Granite: every block's output is multiplied before it joins the residual stream; folded into the weights
    res_mul = float(hf.get("residual_multiplier", 1.0) or 1.0) if cfg.arch in ("granite", "granitemoe") else 1.0

    def linear(stems, rows, col=None, bias=None, mul: float = 1.0):
        if requant is None and tp_size == 1 and col is None and mul == 1.0 and sh.has(stems[0] + ".qweight"):
            lin = awq_planes(sh, stems, rows, device, bias)
            if lin is not None:
                return lin
        fp8 = all(sh.has(s + ".weight") and sh.get(s + ".weight").dtype == torch.float8_e4m3fn for s in stems)
        if fp8 and requant in (None, "fp8_block") and mul == 1.0:
            lin = _fp8_linear(sh, stems, rows, device, col, bias)
            if lin is not None:
                return lin
        w = torch.cat([_float_rows(sh, s, r, col) for s, r in zip(stems, rows)], 0).to(device)
        if mul != 1.0:
            w = w * mul
            bias = bias * mul if bias is not None else None
        fmt = requant or ("fp8_block" if fp8 else "bf16")
        if fmt == "fp8_block" and (w.shape[0] % 128 or w.shape[1] % 128):
            fmt = "bf16"
        return make_linear(w, fmt, bias)

    for il in range(cfg.n_layers):
        p = f"model.layers.{il}."
        a = p + "self_attn."
        bqkv = bo = None
        if sh.has(a + "q_proj.bias"):               # Qwen2 files carry q/k/v biases without saying so in the config
            bqkv = torch.cat([vec(a + "q_proj.bias")[q_sl], vec(a + "k_proj.bias")[kv_sl],
                              vec(a + "v_proj.bias")[kv_sl]]).contiguous()
            if sh.has(a + "o_proj.bias"):
                bo = vec(a + "o_proj.bias") if tp_rank == 0 else torch.zeros(H, device=device)
        if sh.has(a + "qkv_proj.weight"):
            # Phi-3: one tensor holds the q rows, then the k rows, then the v rows
            k0, v0 = cfg.n_q * hd, (cfg.n_q + cfg.n_kv) * hd
            shift = lambda sl, off: slice(sl.start + off, sl.stop + off)
            wqkv = linear([a + "qkv_proj"] * 3, [q_sl, shift(kv_sl, k0), shift(kv_sl, v0)], bias=bqkv)
        else:
            wqkv = linear([a + "q_proj", a + "k_proj", a + "v_proj"], [q_sl, kv_sl, kv_sl], bias=bqkv)
        lw = LayerWeights(attn_norm=vec(p + "input_layernorm.weight"),
                          ffn_norm=vec(p + "post_attention_layernorm.weight"), wqkv=wqkv,
                          wo=linear([a + "o_proj"], [None], col=q_sl if tp_size > 1 else None, bias=bo, mul=res_mul),
                          window=cfg.layer_window(il))
        if sh.has(a + "q_norm.weight"):
            lw.q_norm, lw.k_norm = vec(a + "q_norm.weight"), vec(a + "k_norm.weight")
        m = p + "mlp."
        if sh.has(a + "sinks"):
            lw.sinks = vec(a + "sinks")[tp_rank * nql:(tp_rank + 1) * nql].contiguous()
        if cfg.is_moe and sh.has(m + "router.weight"):
            from .moe import MoeWeights

            ecnt = cfg.n_experts // tp_size
            elo = tp_rank * ecnt
            mreq = requant if requant in ("mxfp4", "bf16", "q8_0") else None
            gu, gub, fmt = _oss_experts(sh, m + "experts.", "gate_up", cfg, elo, ecnt, device, mreq)
            dn, dnb, _ = _oss_experts(sh, m + "experts.", "down", cfg, elo, ecnt, device, mreq)
            lw.moe = MoeWeights(sh.get(m + "router.weight").to(device).bfloat16(),
                                vec(m + "router.bias") if sh.has(m + "router.bias") else None,
                                gu, dn, gub, dnb, elo, ecnt, fmt)
        elif cfg.is_moe and sh.has(p + "block_sparse_moe.input_linear.weight"):
            # Granite's mixture: experts stacked in two tensors, [E, 2I, H] (gate rows, then up rows) and [E, H, I];
            # the residual multiplier is folded into the down projections like into the dense ones
            from ..ops import quant as Q
            from .moe import MoeWeights

            ecnt = cfg.n_experts // tp_size
            elo = tp_rank * ecnt
            b = p + "block_sparse_moe."
            gu = sh.get(b + "input_linear.weight")[elo:elo + ecnt].float()
            dn = sh.get(b + "output_linear.weight")[elo:elo + ecnt].float() * res_mul
            gu, dn = gu.reshape(-1, gu.shape[-1]), dn.reshape(-1, dn.shape[-1])
            fmt = requant if requant in ("mxfp4", "q8_0", "q4_k", "q6_k") else "bf16"
            conv = (lambda w: w.to(device).bfloat16()) if fmt == "bf16" else (lambda w: Q.quantize_weight(w.to(device), fmt))
            lw.moe = MoeWeights(sh.get(b + "router.layer.weight").to(device).bfloat16(), None, conv(gu), conv(dn), None, None,
                                elo, ecnt, fmt)
        elif cfg.is_moe and cfg.arch in HF_EXPERT_NAMES:
            ecnt = cfg.n_experts // tp_size
            lw.moe = _stacked_experts(sh, p, cfg, tp_rank * ecnt, ecnt, device, requant)
        else:
            if sh.has(m + "gate_up_proj.weight"):          # Phi-3: gate rows, then up rows, in one tensor
                I = cfg.intermediate
                lw.w_gate_up = linear([m + "gate_up_proj"] * 2, [i_sl, slice(i_sl.start + I, i_sl.stop + I)])
            else:
                lw.w_gate_up = linear([m + "gate_proj", m + "up_proj"], [i_sl, i_sl])
            lw.w_down = linear([m + "down_proj"], [None], col=i_sl if tp_size > 1 else None, mul=res_mul)
        mw.layers.append(lw)
    return mw, hf


def save_hf_gpt_oss(directory: str, cfg: ModelConfig, mw: ModelWeights) -> None:
    """Writes a one-rank gpt-oss-shaped model in the checkpoint layout `load_hf` reads: MXFP4 experts as
    `*_blocks` / `*_scales` with interleaved gate / up rows, bf16 attention, sinks, biases (test files)."""
    from safetensors.torch import save_file

    from ..ops import quant as Q

    os.makedirs(directory, exist_ok=True)
    hd, H, I, E = cfg.head_dim, cfg.hidden, cfg.expert_intermediate, cfg.n_experts
    t: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": mw.embed.cpu(), "model.norm.weight": mw.out_norm.cpu(),
                                  "lm_head.weight": mw.lm_head.cpu()}
    nq, nk = cfg.n_q * hd, cfg.n_kv * hd

    def inter(x):            # [E, 2I, ...] gate rows then up rows -> rows alternating gate_i, up_i
        g, u = x[:, :I], x[:, I:]
        return torch.stack([g, u], 2).reshape(x.shape)

    for il, lw in enumerate(mw.layers):
        p = f"model.layers.{il}."
        t[p + "input_layernorm.weight"] = lw.attn_norm.cpu()
        t[p + "post_attention_layernorm.weight"] = lw.ffn_norm.cpu()
        w = lw.wqkv.weight.cpu()
        b = lw.wqkv.bias.cpu()
        for nm, r0, r1 in (("q_proj", 0, nq), ("k_proj", nq, nq + nk), ("v_proj", nq + nk, nq + 2 * nk)):
            t[p + f"self_attn.{nm}.weight"] = w[r0:r1].contiguous()
            t[p + f"self_attn.{nm}.bias"] = b[r0:r1].contiguous()
        t[p + "self_attn.o_proj.weight"] = lw.wo.weight.cpu().contiguous()
        t[p + "self_attn.o_proj.bias"] = lw.wo.bias.cpu()
        t[p + "self_attn.sinks"] = lw.sinks.cpu()
        moe = lw.moe
        t[p + "mlp.router.weight"] = moe.router_w.cpu()
        t[p + "mlp.router.bias"] = moe.router_b.cpu()
        for nm, qw, bias, rows, K in (("gate_up_proj", moe.gate_up, moe.gate_up_b, 2 * I, H),
                                      ("down_proj", moe.down, moe.down_b, H, I)):
            assert isinstance(qw, Q.QuantWeight) and qw.aq_fmt == Q.AQ_MX4
            codes = qw.codes.cpu().reshape(E, rows, K // 32, 16)
            sc = qw.scales.cpu()[:, :K // 32].reshape(E, rows, K // 32)
            bias = bias.cpu()
            if nm == "gate_up_proj":
                codes, sc, bias = inter(codes), inter(sc), inter(bias)
            t[p + f"mlp.experts.{nm}_blocks"] = codes.contiguous()
            t[p + f"mlp.experts.{nm}_scales"] = sc.contiguous()
            t[p + f"mlp.experts.{nm}_bias"] = bias.contiguous()
    save_file(t, os.path.join(directory, "model.safetensors"))
    hf = {"architectures": ["GptOssForCausalLM"], "num_hidden_layers": cfg.n_layers, "hidden_size": H,
          "num_attention_heads": cfg.n_q, "num_key_value_heads": cfg.n_kv, "head_dim": hd, "intermediate_size": I,
          "vocab_size": cfg.vocab, "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_eps,
          "max_position_embeddings": cfg.context_length, "sliding_window": cfg.sliding_window,
          "layer_types": ["sliding_attention" if cfg.layer_window(i) else "full_attention" for i in range(cfg.n_layers)],
          "num_local_experts": E, "num_experts_per_tok": cfg.top_k, "swiglu_limit": cfg.glu_limit,
          "quantization_config": {"quant_method": "mxfp4"},
          "rope_scaling": {"rope_type": "yarn", "factor": cfg.rope_scaling.factor,
                           "original_max_position_embeddings": cfg.rope_scaling.original_context,
                           "beta_fast": getattr(cfg.rope_scaling, "beta_fast", 32.0),
                           "beta_slow": getattr(cfg.rope_scaling, "beta_slow", 1.0)}}
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(hf, f)


def save_hf_fp8(directory: str, cfg: ModelConfig, mw: ModelWeights) -> None:
    """Writes an unsharded model in the block-fp8 safetensors layout (test and benchmark files)."""
    from safetensors.torch import save_file

    os.makedirs(directory, exist_ok=True)
    hd = cfg.head_dim
    t: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": mw.embed.cpu(), "model.norm.weight": mw.out_norm.cpu()}
    if not cfg.tie_embeddings:
        t["lm_head.weight"] = mw.lm_head.cpu()

    def put(stem: str, lin: Linear, r0: int, r1: int):
        if lin.kind == "fp8_block":
            t[stem + ".weight"] = lin.weight.data[r0:r1].contiguous().cpu()
            t[stem + ".weight_scale_inv"] = lin.weight.scale[r0 // 128:(r1 + 127) // 128].contiguous().cpu()
        else:
            t[stem + ".weight"] = lin.weight[r0:r1].contiguous().cpu()

    for il, lw in enumerate(mw.layers):
        p = f"model.layers.{il}."
        t[p + "input_layernorm.weight"] = lw.attn_norm.cpu()
        t[p + "post_attention_layernorm.weight"] = lw.ffn_norm.cpu()
        nq, nk = cfg.n_q * hd, cfg.n_kv * hd
        put(p + "self_attn.q_proj", lw.wqkv, 0, nq)
        put(p + "self_attn.k_proj", lw.wqkv, nq, nq + nk)
        put(p + "self_attn.v_proj", lw.wqkv, nq + nk, nq + 2 * nk)
        put(p + "self_attn.o_proj", lw.wo, 0, cfg.hidden)
        I = cfg.intermediate
        put(p + "mlp.gate_proj", lw.w_gate_up, 0, I)
        put(p + "mlp.up_proj", lw.w_gate_up, I, 2 * I)
        put(p + "mlp.down_proj", lw.w_down, 0, cfg.hidden)
    save_file(t, os.path.join(directory, "model.safetensors"))
    hf = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": cfg.n_layers, "hidden_size": cfg.hidden,
          "num_attention_heads": cfg.n_q, "num_key_value_heads": cfg.n_kv, "head_dim": hd,
          "intermediate_size": cfg.intermediate, "vocab_size": cfg.vocab, "rope_theta": cfg.rope_theta,
          "rms_norm_eps": cfg.rms_eps, "max_position_embeddings": cfg.context_length,
          "tie_word_embeddings": cfg.tie_embeddings}
    if cfg.weight_format == "fp8_block":
        hf["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128]}
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(hf, f)
