"""The generic decoder: one forward for every text architecture, configured by ModelConfig
(the reference's "one route", `src/inference/generic_transformer/hetero.rs`: batched paged decode
`:1408`, mixed paged prefill `:2320`, lm head `:2082`).

Every op below is one launch of a kernel of this library on the current CUDA stream; the
Python code only orders them and owns the static activation buffers, so a decode step can be
captured in a CUDA graph as is.  Per layer (dense, block-fp8):

  add+RMSNorm(+e4m3 quantise) -> qkv GEMM -> q/k norm + RoPE + paged KV write -> attention
  (-> e4m3) -> o_proj GEMM [-> sum over tensor-parallel ranks] -> add+RMSNorm(+quantise)
  -> gate_up GEMM -> SwiGLU(+quantise) -> down GEMM [-> sum over ranks]

Under tensor parallelism with symmetric memory and a decode-size step, the sum over ranks, the
residual add, the norm and the quantise of each boundary are ONE kernel (`SymmComm.sum_norm`,
csrc/cuda/tp_fused.cu) and the residual stream is sharded by rows between the row-parallel
layers: a rank only ever updates and normalises the rows it owns, and the all-gather carries the
next GEMM's e4m3 input.  The reference keeps the stream replicated and runs all-reduce, add and
norm as separate launches over every row on every card
(`src/inference/generic_transformer/tp_forward.rs:70-128`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..utils import nvtx
from ..ops import attention, gemm, rows
from ..ops.gemm import Fp8Act
from ..ops.rows import KVCacheLayer
from .config import ModelConfig
from .weights import Linear, ModelWeights

# Decode-size steps of a dense GGUF model run each layer as four GEMVs with the norms, the gated unit and
# the residual adds inside them (`DecoderModel._layer_fused`); False keeps the separate kernels.
# 1 (norms and residual adds inside the GEMVs, the gated unit a kernel of its own) measured fastest: 2.73 ms per
# single-stream step of an 8B Q4_K_M model against 2.87 (0) and 2.81 (2: every CTA of the down projection
# then evaluates the whole gated unit).
FUSE_GEMV_FRONT = 1      # 2: norms, gated unit and residual adds; 1: without the gated unit; 0: off


@dataclass
class StepInputs:
    """Device-side inputs of one forward.  All tensors are static buffers sized for the
    model's `max_tokens`; `T` rows of them are live."""
    T: int
    tokens: torch.Tensor          # int32 [cap]
    positions: torch.Tensor       # int32 [cap]
    slots: torch.Tensor           # int32 [cap]  KV slot of each row (-1: do not store)
    mode: str                     # "decode" | "prefill"
    block_table: torch.Tensor     # int32 [n_seqs, max_blocks]
    seq_lens: Optional[torch.Tensor] = None      # decode: int32 [cap] keys visible to each row
    row_seq: Optional[torch.Tensor] = None       # decode: block-table row per query row
    nsplit: int = 1
    plan: Optional[attention.PrefillPlan] = None
    logit_rows: Optional[torch.Tensor] = None    # int64 rows that need logits (None: all T)
    n_logit_rows: int = 0
    embed_overrides: Optional[list] = None       # [(first row, bf16 [n, H])]: rows given as embeddings (prompt_embeds)


class Buffers:
    def __init__(self, cfg: ModelConfig, w: ModelWeights, cap: int, device):
        H, hd = cfg.hidden, cfg.head_dim
        nq, nkv = w.n_q_local, w.n_kv_local
        bf = dict(dtype=torch.bfloat16, device=device)
        self.cap = cap
        self.x = torch.zeros(cap, H, **bf)
        self.h = torch.zeros(cap, H, **bf)
        self.delta = torch.zeros(cap, H, **bf)
        self.delta2 = torch.zeros(min(cap, 8), H, **bf)      # second update buffer of the fused decode layers
        self.qk_rinv = torch.zeros(cap, 2, dtype=torch.float32, device=device) if cfg.qk_norm_wide else None
        self.qkv = torch.zeros(cap, (nq + 2 * nkv) * hd, **bf)
        self.q = torch.zeros(cap, nq, hd, **bf)
        self.attn = torch.zeros(cap, nq * hd, **bf)
        fp8_ok = H % 128 == 0
        self.h8 = rows.alloc_fp8_act(cap, H, device) if fp8_ok else None
        self.attn8 = rows.alloc_fp8_act(cap, nq * hd, device) if (nq * hd) % 128 == 0 else None
        if not cfg.is_moe:
            il = next(l for l in w.layers if l is not None).w_gate_up.n_out // 2
            self.gu = torch.zeros(cap, 2 * il, **bf)
            self.act = torch.zeros(cap, il, **bf)
            self.act8 = rows.alloc_fp8_act(cap, il, device) if il % 128 == 0 else None
        self.logits = torch.zeros(cap, w.vocab_local, dtype=torch.float32, device=device)
        self.hsel = torch.zeros(cap, H, **bf)


class DecoderModel:
    def __init__(self, weights: ModelWeights, kv: List[KVCacheLayer], block_size: int, max_tokens: int,
                 comm=None, moe_runner=None):
        self.w = weights
        self.cfg = weights.cfg
        self.kv = kv
        self.block_size = block_size
        self.comm = comm
        self.device = weights.embed.device
        if self.cfg.qk_norm_wide and weights.tp_size > 1:
            raise NotImplementedError("a q / k norm over all heads of a token needs every head on one rank")
        self.buf = Buffers(self.cfg, weights, max_tokens, self.device)
        self.moe_runner = moe_runner
        self._kg = None    # gathered K / V^T scratch for prefill, grown on demand
        self._delta_local = False   # the pending update is complete for the owned rows (after a sharded mixture layer)
        self.sharded_steps = 0   # forwards issued with the row-sharded residual stream (eager or captured)

    # ---- one linear layer in whatever format its weights are held ----
    def _linear(self, lin: Linear, x_bf16, x_fp8: Optional[Fp8Act], out, T: int, reduce: bool = False):
        """`reduce`: the layer is row-parallel, its output is summed over the tensor-parallel ranks.
        With symmetric memory the sum happens inside the GEMM's epilogue (tiles are pushed to the
        peers as they finish); otherwise, or when the grid is too large to be resident at once, the
        GEMM is followed by the communicator's all-reduce."""
        tp = reduce and self.comm is not None and self.comm.size > 1
        symm = getattr(self.comm, "heap", None) if (tp and getattr(self.comm, "fused_gemm", False)) else None
        if lin.kind == "fp8_block":
            gemm.linear_fp8(x_fp8, lin.weight, bias=lin.bias, out=out[:T], rows=T, symm=symm)
        elif lin.kind == "bf16":
            gemm.linear_bf16(x_bf16[:T], lin.weight, bias=lin.bias, out=out[:T], symm=symm)
        else:
            from ..ops import quant

            quant.linear_gguf(x_bf16[:T], lin.weight, bias=lin.bias, out=out[:T])
            symm = None
        if tp and not (symm is not None and gemm.gemm_raw.last_fused):
            self.comm.all_reduce(out, T)
        return out

    def _reduce(self, t: torch.Tensor, T: int):
        if self.comm is not None and self.comm.size > 1:
            self.comm.all_reduce(t, T)

    def _gather_scratch(self, plan: attention.PrefillPlan):
        need = plan.total_kv_pad
        nkv, hd = self.w.n_kv_local, self.cfg.head_dim
        if self._kg is None or self._kg[0].shape[0] < need:
            cap = max(need, 4096)
            self._kg = (torch.zeros(cap, nkv, hd, dtype=torch.bfloat16, device=self.device),
                        torch.zeros(nkv, hd, cap, dtype=torch.bfloat16, device=self.device))
        return self._kg

    # ---- attention of one layer over rows [0, T) ----
    def _attention(self, il: int, inp: StepInputs, T: int, want_fp8: bool):
        cfg, w, b = self.cfg, self.w, self.buf
        lw = w.layers[il]
        cache = self.kv[il]
        rows.rope_kv(b.qkv, inp.positions, inp.slots, cache, w.n_q_local, w.inv_freq,
                     rope_dim=cfg.rope_dim or cfg.head_dim, pairing=cfg.rope_pairing, mscale=w.rope_mscale,
                     q_norm_w=lw.q_norm, k_norm_w=lw.k_norm, eps=cfg.rms_eps, q_out=b.q, rows=T,
                     wide_rinv=b.qk_rinv if (cfg.qk_norm_wide and lw.q_norm is not None) else None)
        scale = cfg.softmax_scale()
        if inp.mode == "decode":
            use8 = want_fp8 and cfg.head_dim == 128 and b.attn8 is not None
            attention.decode(b.q, cache, inp.block_table, inp.seq_lens, block_size=self.block_size, scale=scale,
                             window=lw.window, sinks=lw.sinks, row_seq=inp.row_seq,
                             out=None if use8 else b.attn, out_fp8=b.attn8 if use8 else None, nsplit=inp.nsplit,
                             rows=T)
            return use8
        plan = inp.plan
        kbuf, vtbuf = self._gather_scratch(plan)
        attention.kv_gather(cache, inp.block_table, plan, self.block_size, kbuf, vtbuf)
        attention.prefill(b.q[:T], kbuf, vtbuf, plan, scale=scale, window=lw.window, sinks=lw.sinks, out=b.attn[:T])
        return False

    def forward(self, inp: StepInputs) -> torch.Tensor:
        """Runs the decoder over inp.T rows; returns fp32 logits [n_logit_rows, vocab_local]."""
        self.embed_rows(inp)
        delta = self.run_layers(inp, 0, len(self.w.layers))
        return self.head(inp, delta)

    def profile_layers(self, inp: StepInputs):
        """One forward over `inp` with CUDA events around the embedding, every layer and the head;
        returns [{"stage", "ms"}] (`/api/layer_perf`, the reference's `layer_perf.rs`)."""
        ev = lambda: torch.cuda.Event(enable_timing=True)
        marks = [("embed", ev())]
        marks[0][1].record()
        self.embed_rows(inp)
        delta = None
        lo, hi = (self.w.layer_range if getattr(self.w, "layer_range", None) else (0, len(self.w.layers)))
        for il in range(lo, hi):
            e = ev()
            e.record()
            marks.append((f"layer {il}", e))
            delta = self.run_layers(inp, il, il + 1, delta)
        e = ev()
        e.record()
        marks.append(("head", e))
        self.head(inp, delta)
        end = ev()
        end.record()
        end.synchronize()
        out = []
        for (name, a), (_, b) in zip(marks, marks[1:] + [("end", end)]):
            out.append({"stage": name, "ms": round(a.elapsed_time(b), 4)})
        return out

    def embed_rows(self, inp: StepInputs):
        T = inp.T
        assert T <= self.buf.cap
        if isinstance(self.w.embed, torch.Tensor):
            rows.embed(inp.tokens[:T], self.w.embed, out=self.buf.x[:T], scale=self.cfg.embedding_scale)
        else:       # a table kept in its block format: rows are decoded as they are gathered
            from ..ops import quant

            quant.embed_gguf(inp.tokens[:T], self.w.embed, out=self.buf.x[:T], scale=self.cfg.embedding_scale)
        for r0, t in (inp.embed_overrides or ()):
            self.buf.x[r0:r0 + t.shape[0]].copy_(t)       # a prompt given as embedding rows takes the table's place
        self._delta_local = False

    def sharded(self, T: int) -> bool:
        """True when this step keeps the residual stream sharded by rows over the tensor-parallel
        ranks: `delta` then holds this rank's PARTIAL sums and every norm is `comm.sum_norm`."""
        c = self.comm
        if not (c is not None and c.size > 1 and getattr(c, "fused_norm", False)
                and getattr(self.w, "layer_range", None) is None and c.can_sum_norm(T, self.cfg.hidden)):
            return False
        # a mixture model also needs the expert-parallel dispatch to fit this step
        return not self.cfg.is_moe or self.moe_runner.can_dispatch(T)

    def _norm(self, x, w, delta, T: int, f8: bool, shard: bool, out=None, gather: bool = True,
              local: bool = False):
        """x += delta; RMSNorm(x) * w -> b.h8 (e4m3) or `out` / b.h (bf16).  Sharded: `delta` is this
        rank's partial of a row-parallel layer (or, `local`, the finished update of the rows it owns)
        and the sum over ranks happens here; without `gather` the normalised rows stay on their owner."""
        b = self.buf
        out = b.h if out is None else out
        if shard and delta is not None:
            self.comm.sum_norm(delta, x, w, self.cfg.rms_eps, T, out=None if f8 else out,
                               out_fp8=b.h8 if f8 else None, gather=gather, local=local)
        else:
            rows.add_rmsnorm(x, w, self.cfg.rms_eps, delta=delta, out=None if f8 else out,
                             out_fp8=b.h8 if f8 else None, rows=T)

    def _fused_front_ok(self, lw, T: int, shard: bool) -> bool:
        """A dense layer whose four matrices run as quantised GEMVs at this many rows: norms, the gated unit
        and the residual adds then ride inside those GEMVs (ops/quant.py: GemvFront)."""
        if not FUSE_GEMV_FRONT or shard or self.cfg.is_moe or lw.w_gate_up is None:
            return False
        if self.comm is not None and self.comm.size > 1:
            return False                # row-parallel layers are summed over the ranks between the GEMVs
        from ..ops import quant

        b = self.buf
        return (quant.gemv_takes(T, lw.wqkv.weight, b.x.stride(0)) and quant.gemv_takes(T, lw.wo.weight, b.attn.stride(0))
                and quant.gemv_takes(T, lw.w_gate_up.weight, b.x.stride(0))
                and quant.gemv_takes(T, lw.w_down.weight, b.gu.stride(0))
                and all(l.kind == "gguf" for l in (lw.wqkv, lw.wo, lw.w_gate_up, lw.w_down)))

    def _fused_attn_ok(self, lw, T: int, shard: bool) -> bool:
        """A mixture layer on one rank whose attention matrices run as quantised GEMVs at this many rows."""
        if not FUSE_GEMV_FRONT or shard or not self.cfg.is_moe or lw.moe is None or (self.comm is not None and self.comm.size > 1):
            return False
        from ..ops import quant

        b = self.buf
        return (lw.wqkv.kind == "gguf" and lw.wo.kind == "gguf" and quant.gemv_takes(T, lw.wqkv.weight, b.x.stride(0))
                and quant.gemv_takes(T, lw.wo.weight, b.attn.stride(0)))

    def _layer_fused_attn_moe(self, il: int, inp: StepInputs, T: int, pend: Optional[torch.Tensor]) -> torch.Tensor:
        """The attention half as in `_layer_fused` (norm in front of the q/k/v GEMV, the pending update folded in by
        the o-projection GEMV); the feed-forward norm stays a kernel, since the router and the experts both read
        its rows.  The mixture's output is the update pending on x."""
        from ..ops import quant

        cfg, b = self.cfg, self.buf
        lw = self.w.layers[il]
        F = quant.GemvFront
        quant.linear_gguf(b.x[:T], lw.wqkv.weight, bias=lw.wqkv.bias, out=b.qkv[:T],
                          front=F(norm=lw.attn_norm, eps=cfg.rms_eps, delta=pend))
        self._attention(il, inp, T, False)
        d1 = b.delta2 if pend is not b.delta2 else b.delta
        quant.linear_gguf(b.attn[:T], lw.wo.weight, bias=lw.wo.bias, out=d1[:T],
                          front=F(update=(b.x, pend)) if pend is not None else None)
        rows.add_rmsnorm(b.x, lw.ffn_norm, cfg.rms_eps, delta=d1, out=b.h, rows=T)
        out = b.delta if d1 is not b.delta else b.delta2
        self.moe_runner.forward(il, lw.moe, b.h, out, T)
        return out

    def _layer_fused(self, il: int, inp: StepInputs, T: int, pend: Optional[torch.Tensor]) -> torch.Tensor:
        """One dense layer as four GEMVs, rope + cache write and attention: five kernels fewer than the
        separate form.  Each norm runs in front of its GEMV on (x + the update still pending); the GEMV
        after it folds that update into x on the side (all readers of the old rows are done by then), so
        the two updates of a layer alternate between two buffers.  Returns the update pending on x."""
        from ..ops import quant

        cfg, b = self.cfg, self.buf
        lw = self.w.layers[il]
        F = quant.GemvFront
        quant.linear_gguf(b.x[:T], lw.wqkv.weight, bias=lw.wqkv.bias, out=b.qkv[:T],
                          front=F(norm=lw.attn_norm, eps=cfg.rms_eps, delta=pend))
        self._attention(il, inp, T, False)
        d1 = b.delta if pend is not b.delta else b.delta2
        quant.linear_gguf(b.attn[:T], lw.wo.weight, bias=lw.wo.bias, out=d1[:T],
                          front=F(update=(b.x, pend)) if pend is not None else None)
        quant.linear_gguf(b.x[:T], lw.w_gate_up.weight, bias=lw.w_gate_up.bias, out=b.gu[:T],
                          front=F(norm=lw.ffn_norm, eps=cfg.rms_eps, delta=d1))
        d2 = b.delta2 if d1 is b.delta else b.delta
        if FUSE_GEMV_FRONT >= 2:
            quant.linear_gguf(b.gu[:T], lw.w_down.weight, bias=lw.w_down.bias, out=d2[:T],
                              front=F(glu=(cfg.glu_mode, cfg.glu_alpha, cfg.glu_limit), update=(b.x, d1)))
        else:
            rows.glu(b.gu, mode=cfg.glu_mode, alpha=cfg.glu_alpha, limit=cfg.glu_limit, out=b.act, rows=T)
            quant.linear_gguf(b.act[:T], lw.w_down.weight, bias=lw.w_down.bias, out=d2[:T], front=F(update=(b.x, d1)))
        return d2

    def run_layers(self, inp: StepInputs, lo: int, hi: int, delta: Optional[torch.Tensor] = None):
        """Layers [lo, hi) over the residual stream in `buf.x`; returns the pending residual update
        (the next norm, or `fold_residual`, adds it).  In a sharded step (see `sharded`) the update
        is this rank's partial sum and `buf.x` is current only in the rows this rank owns."""
        cfg, w, b = self.cfg, self.w, self.buf
        T = inp.T
        shard = self.sharded(T)
        self.sharded_steps += int(shard)
        for il in range(lo, hi):
            lw = w.layers[il]
            nvtx.mark(f"layer {il}", level=2)
            if T <= b.delta2.shape[0] and not self._delta_local and self._fused_front_ok(lw, T, shard):
                delta = self._layer_fused(il, inp, T, delta)
                continue
            if T <= b.delta2.shape[0] and not self._delta_local and self._fused_attn_ok(lw, T, shard):
                delta = self._layer_fused_attn_moe(il, inp, T, delta)
                continue
            # attention block
            self._norm(b.x, lw.attn_norm, delta, T, lw.wqkv.wants_fp8, shard, local=self._delta_local)
            self._delta_local = False
            self._linear(lw.wqkv, b.h, b.h8, b.qkv, T)
            got8 = self._attention(il, inp, T, lw.wo.wants_fp8)
            if lw.wo.wants_fp8 and not got8:
                rows.quant_fp8(b.attn, out=b.attn8, rows=T)
            self._linear(lw.wo, b.attn, b.attn8, b.delta, T, reduce=not shard)
            # feed-forward block
            if cfg.is_moe and shard:
                # token-sharded mixture layer: the owner of a row normalises it, routes it and sends its
                # pairs to the experts' ranks; the combined output is the finished update of its own rows
                self._norm(b.x, lw.ffn_norm, b.delta, T, False, True, gather=False)
                self.moe_runner.forward_ep(il, lw.moe, b.h, b.delta, T)
                self._delta_local = True
            elif cfg.is_moe:
                rows.add_rmsnorm(b.x, lw.ffn_norm, cfg.rms_eps, delta=b.delta, out=b.h, rows=T)
                self.moe_runner.forward(il, lw.moe, b.h, b.delta, T)
            else:
                self._norm(b.x, lw.ffn_norm, b.delta, T, lw.w_gate_up.wants_fp8, shard)
                self._linear(lw.w_gate_up, b.h, b.h8, b.gu, T)
                d8 = lw.w_down.wants_fp8
                rows.glu(b.gu, mode=cfg.glu_mode, alpha=cfg.glu_alpha, limit=cfg.glu_limit,
                         out=None if d8 else b.act, out_fp8=b.act8 if d8 else None, rows=T)
                self._linear(lw.w_down, b.act, b.act8, b.delta, T, reduce=not shard)
            delta = b.delta
        return delta

    def fold_residual(self, inp: StepInputs, delta: Optional[torch.Tensor]) -> torch.Tensor:
        """Adds the pending update into the residual stream and returns it (what a pipeline stage
        hands to the next one)."""
        T = inp.T
        if delta is not None:
            self.buf.x[:T].add_(delta[:T])
        return self.buf.x[:T]

    def head(self, inp: StepInputs, delta: Optional[torch.Tensor]) -> torch.Tensor:
        cfg, w, b = self.cfg, self.w, self.buf
        T = inp.T
        self._norm(b.x, w.out_norm, delta, T, False, self.sharded(T), local=self._delta_local)
        self._delta_local = False
        if inp.logit_rows is not None:
            n = inp.n_logit_rows
            torch.index_select(b.h, 0, inp.logit_rows[:n], out=b.hsel[:n])
            hsrc = b.hsel
        else:
            n = T
            hsrc = b.h
        if isinstance(w.lm_head, torch.Tensor):
            gemm.linear_bf16(hsrc[:n], w.lm_head, out=b.logits[:n], out_fp32=True)
        else:       # a head kept in its block format (GEMV on int8 activations up to eight rows)
            from ..ops import quant

            quant.linear_gguf(hsrc[:n], w.lm_head, out=b.logits[:n], out_fp32=True)
        logits = b.logits[:n]
        if cfg.logit_scale != 1.0:
            logits.mul_(cfg.logit_scale)
        if self.comm is not None and self.comm.size > 1:
            logits = self.comm.all_gather_cols(logits)
        return logits


def make_kv_cache(cfg: ModelConfig, n_kv_local: int, num_blocks: int, block_size: int, device,
                  layer_range=None) -> List[Optional[KVCacheLayer]]:
    q8 = cfg.kv_format == "q8"
    lo, hi = layer_range if layer_range is not None else (0, cfg.n_layers)
    return [KVCacheLayer(num_blocks * block_size, n_kv_local, cfg.head_dim, device, q8=q8) if lo <= il < hi else None
            for il in range(cfg.n_layers)]
