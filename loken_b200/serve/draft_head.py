"""Draft heads: a small network on top of the target's own hidden states proposes the next tokens.

Two published forms share one structure here:

  EAGLE-1   h = fc([embed(t_{p+1}) ; f_p]) -> one decoder layer -> f'_{p+1} -> the target's norm + head
  MTP       h = proj([RMSNorm_e(embed(t_{p+1})) ; RMSNorm_h(f_p)]) -> one decoder layer -> shared norm + head

where f_p is the target's final hidden state (before its output norm) at position p and t_{p+1} the
token sampled there.  The head keeps its own one-layer paged cache over "pair positions" p.  A cycle:

  1. the target's verify pass has just produced f for the rows it accepted; `observe()` stores them as
     pending real pairs (t_{p+1}, f_p);
  2. `propose()` feeds the pending pairs in one multi-row forward (their K/V replace what the last
     cycle's guesses wrote), takes the logits of the last one as the first draft token, and continues
     k - 1 steps on its own predicted features.

Verification (`speculative.Speculator`) is what keeps the output exact; the head only decides how
many tokens a cycle commits.  A sequence met for the first time starts with an empty head cache (the
prompt's features are not replayed into it): the first cycles draft from little context and improve
as pairs accumulate.  The reference's heads are `src/inference/generic_transformer/draft_head.rs` and
`src/inference/serve/eagle.rs`; its block-draft variant is not built.
"""
from __future__ import annotations

import dataclasses
import time
from typing import Dict, List, Optional, Sequence as Seq

import torch

from ..models.weights import embed_lookup
from .kv_manager import PagedKvAllocator
from .scheduler import Sequence
from .speculative import DRAFT_MAX, _RowView, _greedy_twin


@dataclasses.dataclass
class DraftHeadWeights:
    kind: str                                  # "eagle" | "mtp"
    fc: torch.Tensor                           # bf16 [H, 2H]: the [embedding ; feature] projection
    fc_bias: Optional[torch.Tensor]            # f32 [H]
    layer: object                              # models.weights.LayerWeights of the one decoder layer
    enorm: Optional[torch.Tensor] = None       # f32 [H] (mtp): norm weight on the embedding
    hnorm: Optional[torch.Tensor] = None       # f32 [H] (mtp): norm weight on the feature


def random_draft_head(cfg, device, kind: str = "eagle", seed: int = 0, std: float = 0.02) -> DraftHeadWeights:
    """A random-init head of the target's width (tests, benchmarks)."""
    from ..models.weights import random_weights

    one = dataclasses.replace(cfg, n_layers=1, weight_format="bf16", n_experts=0, top_k=0, sliding_window=0,
                              swa_layers=None, sinks=False)
    w = random_weights(one, device, seed=seed + 17, std=std)
    g = torch.Generator(device="cpu").manual_seed(seed + 23)
    H = cfg.hidden
    fc = (torch.randn(H, 2 * H, generator=g) * std).to(device).bfloat16()
    ones = torch.ones(H, device=device)
    return DraftHeadWeights(kind, fc, None, w.layers[0], ones.clone() if kind == "mtp" else None,
                            ones.clone() if kind == "mtp" else None)


def load_draft_head(directory: str, cfg, device) -> DraftHeadWeights:
    """Reads a head in the published safetensors layouts: EAGLE (`fc.weight` [H, 2H], optional `fc.bias`,
    `layers.0.*` with the usual projection names) or MTP (`enorm.weight`, `hnorm.weight`, `eh_proj.weight`,
    `layers.0.*` / `mtp_block.*`)."""
    import glob
    import os

    from safetensors import safe_open

    from ..models.weights import LayerWeights, make_linear

    t: Dict[str, torch.Tensor] = {}
    if os.path.isfile(directory) and directory.endswith(".gguf"):
        # the companion `loken draft-head` writes: the checkpoint's mtp.* tensors under their own names
        from ..formats import gguf as G

        r = G.GGUFReader(directory)
        try:
            for k, ti in r.tensors.items():
                t[k.removeprefix("mtp.")] = torch.from_numpy(ti.to_float().copy())
        finally:
            r.close()
    for f in sorted(glob.glob(os.path.join(directory, "*.safetensors"))):
        with safe_open(f, framework="pt", device="cpu") as h:
            for k in h.keys():
                t[k.removeprefix("model.").removeprefix("mtp.")] = h.get_tensor(k)
    if not t:
        raise FileNotFoundError(f"no .safetensors files (and no .gguf companion) at {directory}")
    kind = "mtp" if "eh_proj.weight" in t else "eagle"
    fc = t["eh_proj.weight" if kind == "mtp" else "fc.weight"]
    H = cfg.hidden
    if tuple(fc.shape) != (H, 2 * H):
        raise ValueError(f"the head projects {tuple(fc.shape)}, the target needs [{H}, {2 * H}]")
    pre = next((p for p in ("layers.0.", "mtp_block.", "block.") if p + "self_attn.q_proj.weight" in t), None)
    if pre is None:
        raise ValueError("no decoder layer (layers.0.self_attn.q_proj.weight) in the head's files")
    get = lambda n: t[pre + n].to(device)
    vec = lambda n, d=None: t[pre + n].float().to(device) if pre + n in t else d
    wq = torch.cat([get("self_attn.q_proj.weight"), get("self_attn.k_proj.weight"), get("self_attn.v_proj.weight")], 0)
    ones = torch.ones(H, device=device)
    lw = LayerWeights(attn_norm=vec("input_layernorm.weight", ones.clone()),
                      ffn_norm=vec("post_attention_layernorm.weight", ones.clone()),
                      wqkv=make_linear(wq.bfloat16(), "bf16", None),
                      wo=make_linear(get("self_attn.o_proj.weight").bfloat16(), "bf16", None), window=0)
    lw.w_gate_up = make_linear(torch.cat([get("mlp.gate_proj.weight"), get("mlp.up_proj.weight")], 0).bfloat16(), "bf16", None)
    lw.w_down = make_linear(get("mlp.down_proj.weight").bfloat16(), "bf16", None)
    return DraftHeadWeights(kind, fc.to(device).bfloat16(), t["fc.bias"].float().to(device) if "fc.bias" in t else None, lw,
                            t["enorm.weight"].float().to(device) if "enorm.weight" in t else None,
                            t["hnorm.weight"].float().to(device) if "hnorm.weight" in t else None)


def head_input(hw: DraftHeadWeights, emb: torch.Tensor, feat: torch.Tensor, eps: float) -> torch.Tensor:
    """[n, H] embeddings and [n, H] features -> the head layer's input rows (bf16).  Plain torch: the
    rows of a cycle are few (sequences x a handful) and the two matrices are small next to the target."""
    e, f = emb.float(), feat.float()
    if hw.enorm is not None:
        e = e * torch.rsqrt(e.pow(2).mean(-1, keepdim=True) + eps) * hw.enorm
    if hw.hnorm is not None:
        f = f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps) * hw.hnorm
    x = torch.cat([e, f], -1).bfloat16() @ hw.fc.t()
    if hw.fc_bias is not None:
        x = x.float() + hw.fc_bias
    return x.bfloat16()


class HeadDrafter:
    """The drafter interface of `speculative.py` over a draft head."""
    name = "head"

    def __init__(self, target_weights, head: DraftHeadWeights, *, max_seqs: int, max_ctx: int, block_size: int = 16,
                 model_id: str = "draft-head"):
        from ..models.weights import ModelWeights
        from .runner import ModelRunner

        tw = target_weights
        cfg = dataclasses.replace(tw.cfg, n_layers=1, weight_format="bf16", n_experts=0, top_k=0, sliding_window=0,
                                  swa_layers=None, sinks=False, kv_format="bf16")
        self.cfg, self.tw, self.head = cfg, tw, head
        self.model_id = f"{model_id} ({head.kind})"
        # the one-layer model shares the target's embedding table, output norm and head
        w = ModelWeights(cfg, tw.embed, tw.out_norm, tw.lm_head, [head.layer], tw.inv_freq, tw.rope_mscale, 0, 1,
                         cfg.n_q, cfg.n_kv, tw.vocab_local, 0)
        blocks = max_seqs * ((max_ctx + DRAFT_MAX + block_size - 1) // block_size + 1) + 8
        self.alloc = PagedKvAllocator(blocks, block_size, enable_prefix_cache=False)
        self.runner = ModelRunner(cfg, w, num_blocks=blocks, block_size=block_size, max_seqs=max_seqs,
                                  max_tokens=max(max_seqs * (DRAFT_MAX + 2), 512), max_ctx=max_ctx + DRAFT_MAX,
                                  use_graphs=False)
        # per sequence: pairs the target has confirmed but the head has not read yet, and where they start
        self.pending: Dict[int, List[tuple]] = {}
        self.known: Dict[int, int] = {}        # head positions whose K/V come from real pairs
        self.seconds_per_token = 0.0

    # ---- what the verify pass tells the head ----
    def observe(self, seq: Sequence, base_pos: int, feats: torch.Tensor, tokens: Seq[int]):
        """After a verify pass: `feats[i]` is the target's final hidden state at position base_pos + i (rows
        the target accepted) and `tokens[i]` the token at position base_pos + i + 1 (sampled there)."""
        sid = seq.seq_id
        have = self.known.get(sid)
        if have is None:
            if not self.alloc.allocate(sid, DRAFT_MAX + len(tokens)):
                return
            self.known[sid] = 0                  # the head's position 0 is the first pair it is shown
            self.pending[sid] = []
        pend = self.pending[sid]
        for i, tok in enumerate(tokens):
            pend.append((int(tok), feats[i].detach().clone()))

    def propose(self, seqs: Seq[Sequence], k: int) -> List[List[int]]:
        t0 = time.perf_counter()
        live = [s for s in seqs if self.pending.get(s.seq_id)]
        drafts: Dict[int, List[int]] = {s.seq_id: [] for s in seqs}
        if not live or k <= 0:
            return [drafts[s.seq_id] for s in seqs]
        eps = self.cfg.rms_eps
        items, embs, lens = [], [], []
        for s in live:
            sid = s.seq_id
            pend = self.pending[sid]
            start = self.known[sid]
            want = start + len(pend) + DRAFT_MAX
            cur = self.alloc.length(sid)
            if want > cur and not self.alloc.append(sid, want - cur):
                continue
            toks = [t for t, _ in pend]
            f = torch.stack([x for _, x in pend])
            e = embed_lookup(self.tw, torch.tensor(toks, device=f.device)) * self.cfg.embedding_scale
            embs.append(head_input(self.head, e, f, eps))
            items.append((s, toks, start))
            lens.append(len(pend))
        if not items:
            return [drafts[s.seq_id] for s in seqs]
        live = [it[0] for it in items]
        logits = self.runner.forward_rows(items, self.alloc, last_only=True, embeds=torch.cat(embs))
        feats = self._last_rows(lens)
        views = [_RowView(_greedy_twin(s), []) for s in live]
        tok = self.runner.sample_rows(logits, views, [0.0] * len(live))
        pos = []
        for s, n, t in zip(live, lens, tok):
            self.known[s.seq_id] += n
            self.pending[s.seq_id] = []
            drafts[s.seq_id].append(int(t))
            pos.append(self.known[s.seq_id])
        for step in range(1, k):
            # the head's own prediction stands in for the feature it has not seen
            e = embed_lookup(self.tw, torch.tensor([drafts[s.seq_id][-1] for s in live], device=feats.device)) \
                * self.cfg.embedding_scale
            x = head_input(self.head, e, feats, eps)
            items = [(s, [drafts[s.seq_id][-1]], p + step - 1) for s, p in zip(live, pos)]
            logits = self.runner.forward_rows(items, self.alloc, last_only=True, embeds=x)
            feats = self._last_rows([1] * len(live))
            tok = self.runner.sample_rows(logits, views, [0.0] * len(live))
            for s, t in zip(live, tok):
                drafts[s.seq_id].append(int(t))
        dt = time.perf_counter() - t0
        self.seconds_per_token += (dt / max(k, 1) - self.seconds_per_token) * 0.2
        return [drafts[s.seq_id] for s in seqs]

    def _last_rows(self, lens: Seq[int]) -> torch.Tensor:
        """The head layer's output (its residual stream) at the last row of every item of the forward just run."""
        x = self.runner.model.buf.x
        idx, r = [], 0
        for n in lens:
            r += n
            idx.append(r - 1)
        return x[torch.tensor(idx, device=x.device)].clone()

    def commit(self, seq: Sequence, new_len: int):
        pass

    def release(self, seq_id: int):
        if seq_id in self.known:
            self.alloc.free(seq_id)
            self.known.pop(seq_id, None)
            self.pending.pop(seq_id, None)

    def status(self) -> dict:
        return {"method": self.name, "model": self.model_id, "sequences": len(self.known),
                "seconds_per_token": round(self.seconds_per_token, 6)}
