"""Mixture-of-experts feed-forward: weights, the single-GPU runner and the expert-parallel runner.

Per layer (gpt-oss semantics, `src/inference/generic_transformer/moe_weights.rs:2378-2382`,
`:2946-2975`): router logits = W_r x + b_r; top-k; weights = softmax over the chosen logits;
per chosen expert g, u = W_gu x + b_gu; h = clamped SwiGLU(g, u); y += w * (W_d h + b_d).
Other routers (full softmax with renormalisation, sigmoid scores) are selected by the config.

Kernel sequence: router GEMM -> lk_moe_route -> lk_moe_plan -> lk_moe_permute -> grouped GEMM
(gate_up, all experts in one launch, MXFP4 / GGUF weights expanded in-kernel or bf16 by TMA) ->
GLU -> grouped GEMM (down) -> lk_moe_combine.  Unlike the reference's expert parallelism, which
replicates every row to every shard and zero-weights foreign pairs (`moe_weights.rs:1845-1893`),
a rank only ever computes pairs routed to experts it owns.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import gemm, quant, rows
from ..ops._lib import GemmArgs, Workspace, check, cuda_lib, ptr, stream
from .config import ModelConfig

ROUTER_MODE = {"softmax_topk": 0, "softmax": 1, "sigmoid": 2}


@dataclass
class MoeWeights:
    router_w: torch.Tensor                 # bf16 [E, H]
    router_b: Optional[torch.Tensor]       # f32 [E]
    gate_up: object                        # stacked [E_local * 2I, H]: bf16 tensor or QuantWeight
    down: object                           # stacked [E_local * H, I]
    gate_up_b: Optional[torch.Tensor]      # f32 [E_local, 2I]
    down_b: Optional[torch.Tensor]         # f32 [E_local, H]
    e_lo: int = 0                          # first expert held by this rank
    e_cnt: int = 0                         # experts held by this rank
    fmt: str = "bf16"


def random_moe(cfg: ModelConfig, gen, device, std: float, ep_rank: int = 0, ep_size: int = 1, il: int = 0
               ) -> MoeWeights:
    """Random experts of one layer, holding only this rank's share.  Every expert has its own seed
    (derived from the model seed, the layer and the expert id), so a rank draws and quantises only the
    experts it holds, one at a time (a 120b-shaped layer is 3.2 G values), and the model is the same at
    every expert-parallel degree."""
    from .weights import linear_format

    E, H, I = cfg.n_experts, cfg.hidden, cfg.expert_intermediate
    assert E % ep_size == 0
    ecnt = E // ep_size
    elo = ep_rank * ecnt
    rn = lambda *s: torch.randn(*s, generator=gen, device=device, dtype=torch.float32) * std
    router_w = (rn(E, H) * 4).bfloat16()          # spread the logits so routing is not a coin toss
    router_b = rn(E) if cfg.expert_bias else None
    fmt = linear_format(cfg, "expert")
    base = int(gen.initial_seed())
    gu_parts, dn_parts, gub, dnb = [], [], [], []
    for e in range(elo, elo + ecnt):
        ge = torch.Generator(device=device)
        ge.manual_seed((base * 1000003 + il * 4099 + e) & 0x7FFFFFFFFFFFFFFF)
        re_ = lambda *s: torch.randn(*s, generator=ge, device=device, dtype=torch.float32) * std
        gu = torch.cat([re_(I, H), re_(I, H)], 0)
        dn = re_(H, I)
        if cfg.expert_bias:
            gub.append(re_(2 * I))
            dnb.append(re_(H))
        if fmt == "bf16":
            gu_parts.append(gu.bfloat16())
            dn_parts.append(dn.bfloat16())
        else:
            qz = quant.quantize_weight_torch if gu.is_cuda else quant.quantize_weight
            gu_parts.append(qz(gu, fmt))
            dn_parts.append(qz(dn, fmt))
        del gu, dn
    if fmt == "bf16":
        gu_w, dn_w = torch.cat(gu_parts, 0).contiguous(), torch.cat(dn_parts, 0).contiguous()
    else:
        def stack(parts):
            p0 = parts[0]
            return quant.QuantWeight(p0.aq_fmt, p0.ggml_type, sum(p.rows for p in parts), p0.K,
                                     torch.cat([p.codes for p in parts], 0).contiguous(),
                                     torch.cat([p.scales for p in parts], 0).contiguous())
        gu_w, dn_w = stack(gu_parts), stack(dn_parts)
    return MoeWeights(router_w, router_b, gu_w, dn_w,
                      torch.stack(gub).contiguous() if gub else None,
                      torch.stack(dnb).contiguous() if dnb else None, elo, ecnt, fmt)


def dequant_experts(moe: MoeWeights):
    """fp32 (gate_up [E_local, 2I, H], down [E_local, H, I]) of the experts this rank holds."""
    def dq(w):
        return w.float() if isinstance(w, torch.Tensor) else quant.dequantize_weight(w)
    gu, dn = dq(moe.gate_up), dq(moe.down)
    E = moe.e_cnt
    return gu.view(E, -1, gu.shape[1]), dn.view(E, -1, dn.shape[1])


def grouped_linear(xs: torch.Tensor, w, rows_per_expert: int, plan: "MoePlan", bias: Optional[torch.Tensor],
                   out: torch.Tensor):
    """out[r, :] = W[expert(r)] xs[r, :] (+ bias[expert(r)]) for every sorted token row r, all
    experts in one launch of the tcgen05 GEMM walking the plan's tile list."""
    K = xs.shape[1]
    wsp = Workspace.get(xs.device)
    a = GemmArgs()
    a.kind = gemm.KIND_BF16
    a.B = ptr(xs)
    a.Rb, a.K, a.ldb = xs.shape[0], K, xs.stride(0)
    a.out, a.out_sa, a.out_sb = ptr(out), 1, out.stride(0)
    a.bias, a.bias_on_a = ptr(bias), 1
    a.bn, a.splits = plan.bn, 1
    a.status = ptr(wsp.status)
    if isinstance(w, torch.Tensor):
        a.A, a.lda, a.Ra = ptr(w), w.stride(0), w.shape[0]
    else:
        a.A, a.lda, a.Ra = None, K, w.rows
        a.aq_fmt, a.aq, a.aq_scale = w.aq_fmt, ptr(w.codes), ptr(w.scales)
        a.aq_ld, a.aq_sld = w.codes.stride(0), w.scales.stride(0)
    a.g_rows_per_expert, a.g_max_tiles = rows_per_expert, plan.max_tiles
    a.g_tile_expert, a.g_tile_row0, a.g_tile_rows = ptr(plan.tile_expert), ptr(plan.tile_row0), ptr(plan.tile_rows)
    a.g_ntiles = ptr(plan.ntiles)
    check(cuda_lib().lk_gemm_tc(C.byref(a), stream()), "lk_gemm_tc (grouped)")
    return out


class MoePlan:
    """Static device buffers of one routing plan (sized for `cap` tokens)."""

    def __init__(self, cap: int, k: int, e_cnt: int, device):
        P = cap * k
        i32 = dict(dtype=torch.int32, device=device)
        self.ids = torch.zeros(cap, k, **i32)
        self.wts = torch.zeros(cap, k, dtype=torch.float32, device=device)
        self.offsets = torch.zeros(e_cnt + 1, **i32)
        self.pair_row = torch.zeros(P, **i32)
        self.max_tiles = e_cnt + (P + 15) // 16
        self.tile_expert = torch.zeros(self.max_tiles, **i32)
        self.tile_row0 = torch.zeros(self.max_tiles, **i32)
        self.tile_rows = torch.zeros(self.max_tiles, **i32)
        self.ntiles = torch.zeros(1, **i32)
        self.bn = 16
        # expert-parallel receive side: expert id (-1 = empty) and (source rank, token, choice) of every slot
        self.slot_expert = torch.full((P,), -1, **i32)
        self.slot_src = torch.zeros(P, **i32)


def pick_group_bn(pairs: int, e_cnt: int, quantised: bool) -> int:
    avg = pairs / max(e_cnt, 1)
    if avg <= 16:
        return 16
    if avg <= 32 and quantised:
        return 32 if avg > 16 else 16
    if avg <= 64 or quantised and avg <= 96:
        return 64
    return 128 if quantised else 256


class MoeRunner:
    def __init__(self, cfg: ModelConfig, weights, cap: int, comm=None):
        self.cfg = cfg
        self.comm = comm
        dev = weights.embed.device
        self.device = dev
        m0 = next(l for l in weights.layers if l is not None).moe
        k, H, I = cfg.top_k, cfg.hidden, cfg.expert_intermediate
        world = comm.size if comm is not None else 1
        cap = cap + (world if world > 1 else 0)     # receive slots are rounded up to whole rows per rank
        self.cap = cap
        self.plan = MoePlan(cap, k, m0.e_cnt, dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        P = cap * k
        self.logits = torch.zeros(cap, cfg.n_experts, dtype=torch.float32, device=dev)
        self.xs = torch.zeros(P + 256, H, **bf)          # slack rows: a tile may read past the last pair
        self.gu = torch.zeros(P + 256, 2 * I, **bf)
        self.act = torch.zeros(P + 256, I, **bf)
        self.y = torch.zeros(P + 256, H, **bf)
        self.xr = torch.zeros(P, H, **bf) if world > 1 else None     # rows received from other ranks, one per slot
        self.wsp = Workspace.get(dev)
        # MXFP4 experts run as stored on the block-scaled tensor-core path (ops/mx.py): activations are
        # quantised to e4m3 + E8M0 exponents by the gather and by the GLU, nothing is dequantised
        self.use_mx = (m0.fmt == "mxfp4" and H % 32 == 0 and I % 32 == 0)
        if self.use_mx:
            from ..ops import mx

            self.xs8 = mx.alloc_mx_act(P + 256, H, dev)
            self.act8 = mx.alloc_mx_act(P + 256, I, dev)

    ROUTER_FUSED_MAX_T = 512     # above it the router runs as a tensor-core GEMM + the routing kernel

    def route(self, moe: MoeWeights, h: torch.Tensor, T: int):
        """Router logits and top-k of rows h[:T] -> plan.ids / plan.wts [T, k]."""
        cfg, pl = self.cfg, self.plan
        lib = cuda_lib()
        if T <= self.ROUTER_FUSED_MAX_T and cfg.hidden * 2 + 1024 <= 48 * 1024 and moe.router_w.is_contiguous():
            check(lib.lk_moe_router(ptr(h), C.c_longlong(h.stride(0)), ptr(moe.router_w), ptr(moe.router_b), T,
                                    cfg.hidden, cfg.n_experts, cfg.top_k, ROUTER_MODE[cfg.router], int(cfg.renorm),
                                    ptr(pl.ids), ptr(pl.wts), None, C.c_longlong(0), stream()), "lk_moe_router")
            return
        gemm.linear_bf16(h[:T], moe.router_w, bias=moe.router_b, out=self.logits[:T], out_fp32=True)
        check(lib.lk_moe_route(ptr(self.logits), C.c_longlong(self.logits.stride(0)), T, cfg.n_experts,
                               cfg.top_k, ROUTER_MODE[cfg.router], int(cfg.renorm), ptr(pl.ids), ptr(pl.wts),
                               stream()), "lk_moe_route")

    def make_plan(self, moe: MoeWeights, T: int):
        cfg, pl = self.cfg, self.plan
        P = T * cfg.top_k
        pl.bn = pick_group_bn(P * moe.e_cnt // cfg.n_experts, moe.e_cnt, not isinstance(moe.gate_up, torch.Tensor))
        check(cuda_lib().lk_moe_plan(ptr(pl.ids), P, cfg.n_experts, moe.e_lo, moe.e_cnt, pl.bn, pl.max_tiles,
                                     ptr(pl.offsets), ptr(pl.pair_row), ptr(pl.tile_expert), ptr(pl.tile_row0),
                                     ptr(pl.tile_rows), ptr(pl.ntiles), ptr(self.wsp.status), stream()),
              "lk_moe_plan")

    def expert_gemms(self, moe: MoeWeights, h: torch.Tensor, P: int, k: int):
        """gate_up -> GLU -> down over the planned pairs: pair p reads row p // k of `h`, its output lands
        in row plan.pair_row[p] of `self.y`."""
        cfg, pl = self.cfg, self.plan
        H, I = cfg.hidden, cfg.expert_intermediate
        lib = cuda_lib()
        if self.use_mx:
            from ..ops import mx

            if getattr(moe, "gate_up_mx", None) is None:
                moe.gate_up_mx, moe.down_mx = mx.mx_weight(moe.gate_up), mx.mx_weight(moe.down)
            mx.quant_mx8(h, out=self.xs8, rows=P, K=H, pair_row=pl.pair_row, kdiv=k)
            mx.grouped_linear_mx(self.xs8, moe.gate_up_mx, 2 * I, pl, moe.gate_up_b, self.gu)
            mx.quant_mx8(self.gu, out=self.act8, rows=P, K=I, glu_mode=cfg.glu_mode, alpha=cfg.glu_alpha,
                         limit=cfg.glu_limit)
            mx.grouped_linear_mx(self.act8, moe.down_mx, H, pl, moe.down_b, self.y)
        else:
            check(lib.lk_moe_permute(ptr(h), C.c_longlong(h.stride(0)), ptr(pl.pair_row), P, k, H, ptr(self.xs),
                                     C.c_longlong(self.xs.stride(0)), stream()), "lk_moe_permute")
            grouped_linear(self.xs, moe.gate_up, 2 * I, pl, moe.gate_up_b, self.gu)
            rows.glu(self.gu, mode=cfg.glu_mode, alpha=cfg.glu_alpha, limit=cfg.glu_limit, out=self.act, rows=P)
            grouped_linear(self.act, moe.down, H, pl, moe.down_b, self.y)

    def experts(self, moe: MoeWeights, h: torch.Tensor, T: int, out: torch.Tensor, accumulate: bool = False):
        """Runs this rank's experts over the planned pairs of h[:T] and writes (or adds) the
        weighted sum of their outputs to out[:T]."""
        cfg, pl = self.cfg, self.plan
        k, H = cfg.top_k, cfg.hidden
        self.expert_gemms(moe, h, T * k, k)
        check(cuda_lib().lk_moe_combine(ptr(self.y), C.c_longlong(self.y.stride(0)), ptr(pl.pair_row), ptr(pl.wts),
                                        T, k, H, ptr(out), C.c_longlong(out.stride(0)), int(accumulate), stream()),
              "lk_moe_combine")

    # ---- expert parallelism with a token-sharded residual stream (csrc/cuda/ep_moe.cu) ----
    def can_dispatch(self, T: int) -> bool:
        c = self.comm
        if c is None or c.size <= 1 or not hasattr(c, "heap") or self.cfg.n_experts % c.size:
            return False
        H, k = self.cfg.hidden, self.cfg.top_k
        rpr = (T + c.size - 1) // c.size
        need = 256 + c.size * rpr * k * (16 + 4 * H)
        return (T + c.size) * k <= self.plan.pair_row.numel() and need <= c.heap.ll_half_bytes

    def forward_ep(self, il: int, moe: MoeWeights, h: torch.Tensor, out: torch.Tensor, T: int):
        """Rows [lo, hi) of `h` are this rank's normalised hidden rows (the residual stream is sharded by
        rows); rows [lo, hi) of `out` receive their mixture output.  Every (token, choice) pair travels to
        the rank that holds its expert and its result travels back: dispatch -> grouped expert GEMMs ->
        combine in choice order with the router weights, all over peer memory, no host round trip."""
        cfg, pl, comm = self.cfg, self.plan, self.comm
        lib = cuda_lib()
        view = C.byref(comm.heap.view)
        k, H, E = cfg.top_k, cfg.hidden, cfg.n_experts
        lo, hi = comm.owned_rows(T)
        n = hi - lo
        st = ptr(self.wsp.status)
        if n > 0:
            self.route(moe, h[lo:hi], n)
        check(lib.lk_ep_dispatch(view, ptr(h), C.c_longlong(h.stride(0)), ptr(pl.ids), T, H, k, E, st, stream()),
              "lk_ep_dispatch")
        check(lib.lk_ep_meta(view, T, H, k, E, ptr(pl.slot_expert), ptr(pl.slot_src), st, stream()), "lk_ep_meta")
        S = int(lib.lk_ep_slots(view, T, k))
        pl.bn = pick_group_bn(T * k * moe.e_cnt // E, moe.e_cnt, not isinstance(moe.gate_up, torch.Tensor))
        check(lib.lk_moe_plan(ptr(pl.slot_expert), S, E, moe.e_lo, moe.e_cnt, pl.bn, pl.max_tiles, ptr(pl.offsets),
                              ptr(pl.pair_row), ptr(pl.tile_expert), ptr(pl.tile_row0), ptr(pl.tile_rows),
                              ptr(pl.ntiles), st, stream()), "lk_moe_plan")
        check(lib.lk_ep_gather(view, T, H, k, E, ptr(pl.slot_expert), ptr(self.xr), C.c_longlong(self.xr.stride(0)),
                               st, stream()), "lk_ep_gather")
        self.expert_gemms(moe, self.xr, S, 1)
        check(lib.lk_ep_return(view, T, H, k, E, ptr(pl.slot_src), ptr(pl.pair_row), ptr(self.y),
                               C.c_longlong(self.y.stride(0)), stream()), "lk_ep_return")
        check(lib.lk_ep_combine(view, T, H, k, E, ptr(pl.wts), ptr(out), C.c_longlong(out.stride(0)), st, stream()),
              "lk_ep_combine")
        comm.collectives += 2

    SLOT_MAX_PAIRS = 64      # up to this many (token, expert) pairs a decode step runs its experts as GEMV slots; 0: off

    def _slots_ok(self, moe: MoeWeights, T: int) -> bool:
        """Decode-size steps of GGUF experts held whole on this rank: the experts run as GEMV slots."""
        if not (0 < T * self.cfg.top_k <= self.SLOT_MAX_PAIRS) or self.use_mx or (self.comm is not None and self.comm.size > 1):
            return False
        ok = getattr(moe, "_slots_ok", None)
        if ok is None:
            from ..ops import quant

            ok = moe._slots_ok = bool(moe.e_cnt == self.cfg.n_experts and moe.e_lo == 0
                                      and quant.gemv_slots_takes(moe.gate_up, moe.e_cnt)
                                      and quant.gemv_slots_takes(moe.down, moe.e_cnt))
        return ok

    def forward_slots(self, moe: MoeWeights, h: torch.Tensor, out: torch.Tensor, T: int):
        """Router, then two launches of the streaming GEMV over (token, expert) slots (the expert of a slot is read
        on the device; the gated unit runs in front of the down projection), then the weighted sum: four kernels
        where the planned form takes seven, and no expert's weights are decoded to bf16."""
        from ..ops import quant

        cfg, pl = self.cfg, self.plan
        k, P = cfg.top_k, T * cfg.top_k
        self.route(moe, h, T)
        ids = pl.ids.view(-1)
        quant.gemv_slots(h, moe.gate_up, ids, P, k, moe.e_cnt, bias=moe.gate_up_b, out=self.gu[:P])
        quant.gemv_slots(self.gu[:P], moe.down, ids, P, 1, moe.e_cnt, bias=moe.down_b, out=self.y[:P],
                         glu=(cfg.glu_mode, cfg.glu_alpha, cfg.glu_limit))
        if getattr(self, "_ident", None) is None:
            self._ident = torch.arange(self.y.shape[0], dtype=torch.int32, device=self.device)
        check(cuda_lib().lk_moe_combine(ptr(self.y), C.c_longlong(self.y.stride(0)), ptr(self._ident), ptr(pl.wts),
                                        T, k, cfg.hidden, ptr(out), C.c_longlong(out.stride(0)), 0, stream()),
              "lk_moe_combine")

    def forward(self, il: int, moe: MoeWeights, h: torch.Tensor, out: torch.Tensor, T: int):
        """h [T, H] bf16 (normalised hidden states, replicated on every rank) -> out [T, H]."""
        if self._slots_ok(moe, T):
            return self.forward_slots(moe, h, out, T)
        self.route(moe, h, T)
        self.make_plan(moe, T)
        self.experts(moe, h, T, out)
        if self.comm is not None and self.comm.size > 1:
            # every rank summed only its own experts' pairs: the ranks' partial rows add up
            self.comm.all_reduce(out, T)
