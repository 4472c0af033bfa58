"""Model configuration: one description for every text decoder the engine runs.

The reference reads these from GGUF metadata (`src/inference/generic_transformer/config.rs:613-837`)
plus a per-architecture facts table (`src/inference/model_facts.rs:152-311`): RoPE pairing,
sliding-window period, YaRN defaults, the clamped SwiGLU of gpt-oss.  `ModelConfig.from_gguf_meta`
does the same; the presets below are the benchmark shapes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional

# RoPE pairing per architecture: 0 = adjacent lane pairs, 1 = half-split (NeoX)
ARCH_FACTS: Dict[str, dict] = {
    "llama": dict(rope_pairing=0),
    "mistral": dict(rope_pairing=0),
    "qwen2": dict(rope_pairing=1, attn_bias=True),
    "qwen3": dict(rope_pairing=1, qk_norm=True),
    "qwen3moe": dict(rope_pairing=1, qk_norm=True, router="softmax", renorm=True),
    "gpt-oss": dict(rope_pairing=1, swa_period=2, yarn_by_default=True, glu_mode=1, glu_alpha=1.702, glu_limit=7.0,
                    attn_bias=True, sinks=True, router="softmax_topk", expert_bias=True),
    "gptoss": dict(rope_pairing=1, swa_period=2, yarn_by_default=True, glu_mode=1, glu_alpha=1.702, glu_limit=7.0,
                   attn_bias=True, sinks=True, router="softmax_topk", expert_bias=True),
    "gemma3": dict(rope_pairing=1, swa_period=6),
    "mixtral": dict(rope_pairing=0, router="softmax", renorm=True),
    "olmoe": dict(rope_pairing=1, router="softmax", renorm=False, qk_norm=True, qk_norm_wide=True),
    "phi3": dict(rope_pairing=1),
    "granite": dict(rope_pairing=0),
    "granitemoe": dict(rope_pairing=0, router="softmax_topk", renorm=True),
}


@dataclass
class RopeScaling:
    kind: str = "none"             # none | linear | llama3 | yarn
    factor: float = 1.0
    original_context: int = 8192
    low_freq_factor: float = 1.0   # llama3
    high_freq_factor: float = 4.0  # llama3
    beta_fast: float = 32.0        # yarn
    beta_slow: float = 1.0         # yarn
    attn_factor: Optional[float] = None
    truncate: bool = True          # yarn: the correction range is rounded outwards to whole dimensions (GGUF
                                   # runtimes do; gpt-oss checkpoints say "truncate": false)


@dataclass
class ModelConfig:
    name: str = "model"
    arch: str = "llama"
    n_layers: int = 2
    hidden: int = 256
    n_q: int = 4
    n_kv: int = 2
    head_dim: int = 64
    intermediate: int = 512
    vocab: int = 1024
    rope_theta: float = 10000.0
    rope_pairing: int = 0
    rope_dim: Optional[int] = None
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    rope_freq_factors: Optional[List[float]] = None   # `rope_freqs.weight` of Llama-3.1 GGUFs
    qk_norm_wide: bool = False     # the q / k norm runs over all heads of a token at once (OLMoE), not per head
    rms_eps: float = 1e-5
    qk_norm: bool = False
    tie_embeddings: bool = False
    attn_bias: bool = False
    context_length: int = 8192
    # sliding window / sinks
    sliding_window: int = 0
    swa_period: int = 0            # layer il is windowed iff il % period < period - 1
    swa_layers: Optional[List[bool]] = None
    sinks: bool = False
    # MoE
    n_experts: int = 0
    top_k: int = 0
    expert_intermediate: int = 0
    router: str = "softmax_topk"   # softmax_topk: softmax over the chosen logits | softmax: full softmax | sigmoid
    renorm: bool = True
    expert_bias: bool = False
    glu_mode: int = 0              # 0 silu(g)*u, 1 clamped gpt-oss form
    glu_alpha: float = 1.702
    glu_limit: float = 7.0
    # storage
    weight_format: str = "bf16"    # bf16 | fp8_block | q8_0 | q4_k_m | mxfp4 (experts; attention bf16)
    kv_format: str = "q8"          # q8 | bf16
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    attn_scale: Optional[float] = None

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    @property
    def group(self) -> int:
        return self.n_q // self.n_kv

    def layer_window(self, il: int) -> int:
        if self.sliding_window <= 0:
            return 0
        if self.swa_layers is not None:
            return self.sliding_window if self.swa_layers[il] else 0
        if self.swa_period > 0:
            return self.sliding_window if (il % self.swa_period) < self.swa_period - 1 else 0
        return self.sliding_window

    def softmax_scale(self) -> float:
        return self.attn_scale if self.attn_scale is not None else 1.0 / math.sqrt(self.head_dim)

    def rope_tables(self):
        """Inverse frequencies [rope_dim/2] and the cos/sin magnitude factor.
        Linear scaling, Llama-3 frequency factors and YaRN all fold into this table
        (reference: `generic_transformer/mod.rs:544-548`, `config.rs:687-712`)."""
        rd = self.rope_dim or self.head_dim
        half = rd // 2
        inv = [self.rope_theta ** (-(2.0 * i) / rd) for i in range(half)]
        sc = self.rope_scaling
        mscale = 1.0
        if self.rope_freq_factors is not None:
            inv = [f / d for f, d in zip(inv, self.rope_freq_factors)]
            if sc.attn_factor is not None:
                mscale = sc.attn_factor
        elif sc.kind == "linear":
            inv = [f / sc.factor for f in inv]
        elif sc.kind == "llama3":
            out = []
            low_wl = sc.original_context / sc.low_freq_factor
            high_wl = sc.original_context / sc.high_freq_factor
            for f in inv:
                wl = 2 * math.pi / f
                if wl < high_wl:
                    out.append(f)
                elif wl > low_wl:
                    out.append(f / sc.factor)
                else:
                    smooth = (sc.original_context / wl - sc.low_freq_factor) / (sc.high_freq_factor - sc.low_freq_factor)
                    out.append((1 - smooth) * f / sc.factor + smooth * f)
            inv = out
        elif sc.kind == "yarn":
            def corr_dim(n_rot):
                return (rd * math.log(sc.original_context / (n_rot * 2 * math.pi))) / (2 * math.log(self.rope_theta))
            lo, hi = corr_dim(sc.beta_fast), corr_dim(sc.beta_slow)
            if sc.truncate:
                lo, hi = math.floor(lo), math.ceil(hi)
            lo, hi = max(lo, 0), min(hi, rd - 1)
            out = []
            for i, f in enumerate(inv):
                ramp = min(max((i - lo) / max(hi - lo, 1e-3), 0.0), 1.0)
                extrap = 1.0 - ramp      # 1 = keep the original frequency
                out.append(f / sc.factor * (1 - extrap) + f * extrap)
            inv = out
            if sc.attn_factor is not None:
                mscale = sc.attn_factor
            elif self.arch in ("gpt-oss", "gptoss"):
                mscale = 1.0 + 0.1 * math.log(sc.factor) if sc.factor > 1 else 1.0
            else:
                mscale = 1.0
        return inv, mscale

    def param_count(self) -> int:
        h, L = self.hidden, self.n_layers
        attn = h * (self.n_q + 2 * self.n_kv) * self.head_dim + self.n_q * self.head_dim * h
        if self.is_moe:
            ffn = self.n_experts * 3 * h * self.expert_intermediate + h * self.n_experts
        else:
            ffn = 3 * h * self.intermediate
        emb = self.vocab * h * (1 if self.tie_embeddings else 2)
        return L * (attn + ffn) + emb

    @classmethod
    def from_gguf_meta(cls, meta: dict, name: str = "gguf") -> "ModelConfig":
        arch = meta.get("general.architecture", "llama")
        g = lambda k, d=None: meta.get(f"{arch}.{k}", d)
        facts = ARCH_FACTS.get(arch, {})
        n_q = int(g("attention.head_count", 1))
        hidden = int(g("embedding_length", 0))
        hd = int(g("attention.key_length", hidden // max(n_q, 1)))
        sc = RopeScaling()
        kind = g("rope.scaling.type")
        if kind in ("linear", "yarn") or (kind is None and facts.get("yarn_by_default") and g("rope.scaling.factor")):
            sc = RopeScaling(kind=kind or "yarn", factor=float(g("rope.scaling.factor", 1.0)),
                             original_context=int(g("rope.scaling.original_context_length", 8192)),
                             beta_fast=float(g("rope.scaling.beta_fast", 32.0)),
                             beta_slow=float(g("rope.scaling.beta_slow", 1.0)),
                             attn_factor=g("rope.scaling.attn_factor"))
        cfg = cls(name=name, arch=arch, n_layers=int(g("block_count", 0)), hidden=hidden, n_q=n_q,
                  n_kv=int(g("attention.head_count_kv", n_q)), head_dim=hd,
                  intermediate=int(g("feed_forward_length", 0)), vocab=int(g("vocab_size", meta.get("_vocab", 0))),
                  rope_theta=float(g("rope.freq_base", 10000.0)), rope_pairing=facts.get("rope_pairing", 0),
                  rope_dim=g("rope.dimension_count"), rope_scaling=sc,
                  rms_eps=float(g("attention.layer_norm_rms_epsilon", 1e-5)), qk_norm=facts.get("qk_norm", False),
                  attn_bias=facts.get("attn_bias", False), context_length=int(g("context_length", 8192)),
                  sliding_window=int(g("attention.sliding_window", 0) or 0), swa_period=facts.get("swa_period", 0),
                  sinks=facts.get("sinks", False), n_experts=int(g("expert_count", 0) or 0),
                  top_k=int(g("expert_used_count", 0) or 0),
                  expert_intermediate=int(g("expert_feed_forward_length", 0) or 0),
                  router=facts.get("router", "softmax_topk"), renorm=facts.get("renorm", True),
                  expert_bias=facts.get("expert_bias", False), glu_mode=facts.get("glu_mode", 0),
                  glu_alpha=facts.get("glu_alpha", 1.702), glu_limit=facts.get("glu_limit", 7.0),
                  embedding_scale=float(g("embedding_scale", 1.0) or 1.0),
                  logit_scale=float(g("logit_scale", 1.0) or 1.0), attn_scale=g("attention.scale"),
                  qk_norm_wide=facts.get("qk_norm_wide", False))
        if arch in ("granite", "granitemoe") and cfg.logit_scale not in (0.0, 1.0):
            cfg.logit_scale = 1.0 / cfg.logit_scale           # these files store the divisor of the logits
        pat = g("attention.sliding_window_pattern")
        if isinstance(pat, list):
            cfg.swa_layers = [bool(x) for x in pat]
        return cfg


_LLAMA3_SCALING = RopeScaling(kind="llama3", factor=8.0, original_context=8192, low_freq_factor=1.0,
                              high_freq_factor=4.0)

PRESETS: Dict[str, ModelConfig] = {
    # BASELINE config 1 (CPU) and the first GPU slice
    "qwen3-1.7b": ModelConfig(name="qwen3-1.7b", arch="qwen3", n_layers=28, hidden=2048, n_q=16, n_kv=8, head_dim=128,
                              intermediate=6144, vocab=151936, rope_theta=1e6, rope_pairing=1, qk_norm=True,
                              tie_embeddings=True, rms_eps=1e-6, weight_format="q8_0", context_length=40960),
    # BASELINE config 2 / 5 (target)
    "llama-3.1-8b": ModelConfig(name="llama-3.1-8b", arch="llama", n_layers=32, hidden=4096, n_q=32, n_kv=8,
                                head_dim=128, intermediate=14336, vocab=128256, rope_theta=5e5, rope_pairing=0,
                                rope_scaling=_LLAMA3_SCALING, weight_format="q4_k_m", context_length=131072),
    # shapes of models the reference publishes numbers for (deepseek-r1:32b is a Qwen2.5-32B; qwen3:8b)
    "qwen2.5-32b": ModelConfig(name="qwen2.5-32b", arch="qwen2", n_layers=64, hidden=5120, n_q=40, n_kv=8, head_dim=128,
                               intermediate=27648, vocab=152064, rope_theta=1e6, rope_pairing=1, attn_bias=True,
                               rms_eps=1e-5, weight_format="q4_k_m", context_length=131072),
    "qwen3-8b": ModelConfig(name="qwen3-8b", arch="qwen3", n_layers=36, hidden=4096, n_q=32, n_kv=8, head_dim=128,
                            intermediate=12288, vocab=151936, rope_theta=1e6, rope_pairing=1, qk_norm=True,
                            rms_eps=1e-6, weight_format="q4_k_m", context_length=40960),
    "qwen3-30b-a3b": ModelConfig(name="qwen3-30b-a3b", arch="qwen3moe", n_layers=48, hidden=2048, n_q=32, n_kv=4,
                                 head_dim=128, intermediate=6144, vocab=151936, rope_theta=1e6, rope_pairing=1, qk_norm=True,
                                 rms_eps=1e-6, n_experts=128, top_k=8, expert_intermediate=768, router="softmax",
                                 renorm=True, weight_format="q4_k_m", context_length=40960),
    "olmoe-1b-7b": ModelConfig(name="olmoe-1b-7b", arch="olmoe", n_layers=16, hidden=2048, n_q=16, n_kv=16, head_dim=128,
                               intermediate=1024, vocab=50304, rope_theta=10000.0, rope_pairing=1, qk_norm=True,
                               qk_norm_wide=True, rms_eps=1e-5, n_experts=64, top_k=8, expert_intermediate=1024,
                               router="softmax", renorm=False, weight_format="q4_k_m", context_length=4096),
    # BASELINE config 5 (draft)
    "llama-3.2-1b": ModelConfig(name="llama-3.2-1b", arch="llama", n_layers=16, hidden=2048, n_q=32, n_kv=8,
                                head_dim=64, intermediate=8192, vocab=128256, rope_theta=5e5, rope_pairing=0,
                                rope_scaling=replace(_LLAMA3_SCALING, factor=32.0), tie_embeddings=True,
                                weight_format="bf16", context_length=131072),
    # BASELINE config 3 (headline)
    "llama-3.3-70b": ModelConfig(name="llama-3.3-70b", arch="llama", n_layers=80, hidden=8192, n_q=64, n_kv=8,
                                 head_dim=128, intermediate=28672, vocab=128256, rope_theta=5e5, rope_pairing=0,
                                 rope_scaling=_LLAMA3_SCALING, weight_format="fp8_block", context_length=131072),
    # BASELINE config 4
    "gpt-oss-120b": ModelConfig(name="gpt-oss-120b", arch="gpt-oss", n_layers=36, hidden=2880, n_q=64, n_kv=8,
                                head_dim=64, intermediate=2880, vocab=201088, rope_theta=150000.0, rope_pairing=1,
                                rope_scaling=RopeScaling(kind="yarn", factor=32.0, original_context=4096),
                                attn_bias=True, sliding_window=128, swa_period=2, sinks=True, n_experts=128, top_k=4,
                                expert_intermediate=2880, router="softmax_topk", expert_bias=True, glu_mode=1,
                                weight_format="mxfp4", kv_format="q8", context_length=131072),
}


def tiny(arch: str = "llama", **kw) -> ModelConfig:
    """Small shapes for tests; dimensions keep every kernel constraint (hidden % 128 == 0)."""
    base = dict(name=f"tiny-{arch}", arch=arch, n_layers=2, hidden=256, n_q=4, n_kv=2, head_dim=64,
                intermediate=512, vocab=512, rope_theta=10000.0, context_length=4096)
    base.update(ARCH_FACTS.get(arch, {}))
    allowed = set(ModelConfig.__dataclass_fields__)
    base = {k: v for k, v in base.items() if k in allowed}
    if arch in ("gpt-oss", "gptoss"):
        base.update(n_experts=8, top_k=2, expert_intermediate=256, sliding_window=32, hidden=256, head_dim=64)
    base.update(kw)
    return ModelConfig(**base)


def get_config(name: str, **overrides) -> ModelConfig:
    if name in PRESETS:
        return replace(PRESETS[name], **overrides)
    if name.startswith("tiny-"):
        return tiny(name[5:], **overrides)
    raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}")
