"""Numerics of every CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _status():
    from loken_b200.ops._lib import Workspace

    w = Workspace.get(torch.device(DEV))
    s = w.read_status()
    w.clear_status()
    return s


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-9)).item()


# ------------------------------------------------------------------ GEMM (bf16)
@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (5, 384, 320), (16, 1024, 512), (64, 2048, 1024),
                                   (200, 640, 768), (300, 512, 256), (1000, 1280, 2048),
                                   (64, 19200, 512), (520, 9600, 256)])
def test_linear_bf16(M, N, K):
    from loken_b200.ops.gemm import linear_bf16

    torch.manual_seed(M * 7 + N)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().t()
    out = linear_bf16(x, w)
    torch.cuda.synchronize()
    assert _status() == 0
    assert out.shape == (M, N)
    assert rel_err(out, ref) < 1e-2


def test_linear_bf16_bias_residual_fp32_splitk():
    from loken_b200.ops.gemm import linear_bf16

    torch.manual_seed(3)
    M, N, K = 24, 512, 4096
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV)
    res = torch.randn(M, N, device=DEV).bfloat16()
    ref = x.float() @ w.float().t() + bias + res.float()
    for splits in (1, 2, 5, 8):
        out = linear_bf16(x, w, bias=bias, residual=res, splits=splits)
        torch.cuda.synchronize()
        assert _status() == 0
        assert rel_err(out, ref) < 1e-2, splits
    out32 = linear_bf16(x, w, out_fp32=True, splits=4)
    assert rel_err(out32, x.float() @ w.float().t()) < 2e-3
    # split-K is summed in split order: two runs agree bit for bit
    a = linear_bf16(x, w, splits=8).clone()
    b = linear_bf16(x, w, splits=8)
    assert torch.equal(a, b)


# ------------------------------------------------------------------ GEMM (block-scaled fp8)
@pytest.mark.parametrize("M,N,K", [(1, 256, 256), (7, 384, 512), (64, 1024, 1024), (128, 512, 2048),
                                   (256, 256, 384), (400, 768, 1024), (64, 19328, 512), (7, 19200, 384)])
@pytest.mark.parametrize("ue8m0", [True, False])
def test_linear_fp8_block(M, N, K, ue8m0):
    """Power-of-two (E8M0) block scales run on the block-scaled MMA for decode-size batches
    (gemm_mx.cu); arbitrary f32 scales, and larger batches, on the per-K-block fold of gemm_tc.cuh."""
    from loken_b200.ops import gemm

    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV) * torch.rand(M, 1, device=DEV) * 2
    w = torch.randn(N, K, device=DEV) * 0.05
    wq = gemm.quantize_weight_fp8(w, ue8m0=ue8m0)
    assert wq.pow2 == ue8m0
    xq = gemm.quantize_act_fp8_ref(x.bfloat16())
    ref = gemm.dequantize_act_fp8(xq, M) @ gemm.dequantize_weight_fp8(wq).t()
    out = gemm.linear_fp8(xq, wq)
    torch.cuda.synchronize()
    assert _status() == 0
    assert rel_err(out, ref) < 1e-2
    out2 = gemm.linear_fp8(xq, wq, splits=2)
    assert rel_err(out2, ref) < 1e-2


@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("M", [5, 64, 128])
@pytest.mark.parametrize("N,K,plan", [
    (1024, 1024, (2, 0, 0)), (1152, 2048, (3, 0, 0)),              # tile groups; 9 tiles: a group of 3 ends on the edge
    (1000, 2048, (3, 2, 3)), (640, 4096, (2, 1, 4)),                 # ragged last tile; remainder units of 2 / 1 tiles, K split
    (148 * 3 * 128 + 128 * 5, 1024, (3, 2, 2)),                      # whole rounds of 3-tile units, then 5 tiles as 2 + 2 + 1
    (148 * 2 * 128 + 128, 1536, (2, 2, 0)), (1536, 8192, (0, 0, 0)), # the cost model's own choice
])
def test_linear_fp8_block_tile_groups(M, N, K, plan, tiled):
    """The block-scaled path with several weight tiles per token tile and stage, whole and K-split units:
    every plan gives the fp32 result of the same quantised operands."""
    from loken_b200.ops import gemm

    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV) * torch.rand(M, 1, device=DEV) * 2
    w = torch.randn(N, K, device=DEV) * 0.05
    wq = gemm.quantize_weight_fp8(w, ue8m0=True)
    xq = gemm.quantize_act_fp8_ref(x.bfloat16())
    ref = gemm.dequantize_act_fp8(xq, M) @ gemm.dequantize_weight_fp8(wq).t()
    if tiled:
        wq.tile_major()                     # 16 KB per 128 x 128 tile in one piece
    bias = torch.randn(N, device=DEV)
    old = gemm.FP8_MX_MAX_M, gemm.FP8_MX_PLAN
    try:
        gemm.FP8_MX_MAX_M, gemm.FP8_MX_PLAN = 128, plan
        out = gemm.linear_fp8(xq, wq, bias=bias)
        again = gemm.linear_fp8(xq, wq, bias=bias)
    finally:
        gemm.FP8_MX_MAX_M, gemm.FP8_MX_PLAN = old
    torch.cuda.synchronize()
    assert _status() == 0
    assert rel_err(out, ref + bias) < 1e-2
    assert torch.equal(out, again)          # split partials are summed in split order


# ------------------------------------------------------------------ row kernels
def test_embed_add_rmsnorm_glu_quant():
    from loken_b200.ops import gemm, rows

    torch.manual_seed(0)
    T, H, V = 37, 1024, 5000
    table = torch.randn(V, H, device=DEV).bfloat16()
    tok = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    e = rows.embed(tok, table)
    assert torch.equal(e, table[tok.long()])

    x = torch.randn(T, H, device=DEV).bfloat16()
    d = torch.randn(T, H, device=DEV).bfloat16()
    w = torch.rand(H, device=DEV) + 0.5
    x0 = x.clone()
    out = torch.empty_like(x)
    q = rows.alloc_fp8_act(T, H, DEV)
    rows.add_rmsnorm(x, w, 1e-5, delta=d, out=out, out_fp8=q)
    xs = (x0.float() + d.float()).bfloat16()
    assert torch.equal(x, xs)
    ref = xs.float() * torch.rsqrt(xs.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w
    assert rel_err(out, ref) < 1e-2
    deq = gemm.dequantize_act_fp8(q, T)
    assert rel_err(deq, ref) < 0.07  # e4m3: 3 mantissa bits
    qr = gemm.quantize_act_fp8_ref(out)
    assert rel_err(q.scale_t[:, :T], qr.scale_t[:, :T]) < 1e-2

    I = 768
    gu = torch.randn(T, 2 * I, device=DEV).bfloat16() * 3
    o = torch.empty(T, I, device=DEV, dtype=torch.bfloat16)
    rows.glu(gu, out=o)
    g, u = gu[:, :I].float(), gu[:, I:].float()
    assert rel_err(o, torch.nn.functional.silu(g) * u) < 1e-2
    rows.glu(gu, mode=1, out=o)
    gg, uu = g.clamp(max=7.0), u.clamp(-7.0, 7.0)
    assert rel_err(o, gg * torch.sigmoid(1.702 * gg) * (1 + uu)) < 1e-2
    q2 = rows.alloc_fp8_act(T, I, DEV)
    rows.glu(gu, out_fp8=q2)
    assert rel_err(gemm.dequantize_act_fp8(q2, T), torch.nn.functional.silu(g) * u) < 0.07

    xq = rows.quant_fp8(gu)
    assert rel_err(gemm.dequantize_act_fp8(xq, T), gu) < 0.07


def _rope_ref(x, pos, inv_freq, pairing, rope_dim, mscale=1.0):
    # x [T, h, hd] float
    T, h, hd = x.shape
    ang = pos.float()[:, None] * inv_freq[None, :]
    cs, sn = torch.cos(ang) * mscale, torch.sin(ang) * mscale
    out = x.clone()
    half = rope_dim // 2
    if pairing == 0:
        a, b = x[..., 0:rope_dim:2], x[..., 1:rope_dim:2]
        out[..., 0:rope_dim:2] = a * cs[:, None] - b * sn[:, None]
        out[..., 1:rope_dim:2] = a * sn[:, None] + b * cs[:, None]
    else:
        a, b = x[..., :half], x[..., half:rope_dim]
        out[..., :half] = a * cs[:, None] - b * sn[:, None]
        out[..., half:rope_dim] = b * cs[:, None] + a * sn[:, None]
    return out


@pytest.mark.parametrize("hd,pairing,q8,qknorm", [(128, 1, True, True), (128, 0, False, False), (64, 1, True, False)])
def test_rope_kv(hd, pairing, q8, qknorm):
    from loken_b200.ops import rows

    torch.manual_seed(1)
    T, n_q, n_kv, slots = 19, 8, 2, 64
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, device=DEV).bfloat16()
    pos = torch.randint(0, 5000, (T,), device=DEV, dtype=torch.int32)
    slot = torch.randperm(slots, device=DEV)[:T].int()
    slot[3] = -1
    inv = (10000.0 ** (-torch.arange(0, hd, 2, device=DEV).float() / hd))
    cache = rows.KVCacheLayer(slots, n_kv, hd, DEV, q8=q8)
    qw = (torch.rand(hd, device=DEV) + 0.5) if qknorm else None
    kw = (torch.rand(hd, device=DEV) + 0.5) if qknorm else None
    q = rows.rope_kv(qkv, pos, slot, cache, n_q, inv, pairing=pairing, q_norm_w=qw, k_norm_w=kw, eps=1e-6)
    torch.cuda.synchronize()
    assert _status() == 0
    x = qkv.float().view(T, n_q + 2 * n_kv, hd)
    qf, kf, vf = x[:, :n_q], x[:, n_q:n_q + n_kv], x[:, n_q + n_kv:]
    if qknorm:
        qf = qf * torch.rsqrt(qf.pow(2).mean(-1, keepdim=True) + 1e-6) * qw
        kf = kf * torch.rsqrt(kf.pow(2).mean(-1, keepdim=True) + 1e-6) * kw
    qr = _rope_ref(qf, pos, inv, pairing, hd)
    kr = _rope_ref(kf, pos, inv, pairing, hd)
    assert rel_err(q, qr) < 1.5e-2
    kc, vc = cache.dequant()
    ok = slot >= 0
    tol = 2e-2 if q8 else 1.5e-2
    assert rel_err(kc[slot[ok].long()], kr[ok]) < tol
    assert rel_err(vc[slot[ok].long()], vf[ok]) < tol


# ------------------------------------------------------------------ attention
def _fill_cache(cache, k, v, slots):
    """k, v [T, n_kv, hd] float -> written at slots with the cache's own quantiser (reference)."""
    if cache.q8:
        for src, codes, sc in ((k, cache.k, cache.k_scale), (v, cache.v, cache.v_scale)):
            b = src.bfloat16().float().view(src.shape[0], src.shape[1], -1, 32)
            d = (b.abs().amax(-1) / 127.0).half()
            df = d.float()
            qv = torch.where(df[..., None] > 0, torch.round(b / df[..., None].clamp_min(1e-30)), torch.zeros_like(b))
            codes[slots] = qv.clamp(-127, 127).to(torch.int8).view(src.shape)
            sc[slots] = d
    else:
        cache.k[slots] = k.bfloat16()
        cache.v[slots] = v.bfloat16()


@pytest.mark.parametrize("hd,n_q,n_kv,q8,window,sinks,nsplit", [
    (128, 8, 1, True, 0, False, 1), (128, 8, 2, True, 0, False, 4), (128, 4, 4, False, 0, False, 2),
    (64, 8, 1, True, 128, True, 3), (64, 16, 2, True, 0, True, 1), (128, 16, 4, True, 100, False, 2),
    # groups of 3, 5, 6 and 7 heads (the paged q8 cache with 16-token blocks included: those take this kernel)
    (128, 6, 2, True, 0, False, 2), (128, 10, 2, True, 0, True, 3), (64, 12, 2, False, 50, False, 1),
    (128, 14, 2, True, 0, False, 1)])
def test_attn_decode(hd, n_q, n_kv, q8, window, sinks, nsplit):
    from loken_b200.ops import attention, rows

    torch.manual_seed(hd + n_q + nsplit)
    bs = 16
    lens = [1, 17, 300, 777, 64]
    B = len(lens)
    max_blocks = (max(lens) + bs - 1) // bs
    nblocks = B * max_blocks + 3
    cache = rows.KVCacheLayer(nblocks * bs, n_kv, hd, DEV, q8=q8)
    perm = torch.randperm(nblocks, device=DEV)[:B * max_blocks].view(B, max_blocks).int()
    ks, vs = [], []
    for s, L in enumerate(lens):
        k = torch.randn(L, n_kv, hd, device=DEV)
        v = torch.randn(L, n_kv, hd, device=DEV)
        t = torch.arange(L, device=DEV)
        slots = perm[s, (t // bs).long()].long() * bs + t % bs
        _fill_cache(cache, k, v, slots)
        ks.append(k)
        vs.append(v)
    kd, vd = cache.dequant()
    q = torch.randn(B, n_q, hd, device=DEV).bfloat16()
    sk = torch.randn(n_q, device=DEV) if sinks else None
    seq_lens = torch.tensor(lens, device=DEV, dtype=torch.int32)
    out = attention.decode(q, cache, perm, seq_lens, block_size=bs, window=window, sinks=sk, nsplit=nsplit)
    torch.cuda.synchronize()
    assert _status() == 0
    for s, L in enumerate(lens):
        t = torch.arange(L, device=DEV)
        slots = perm[s, (t // bs).long()].long() * bs + t % bs
        ref = attention.attention_ref(q[s:s + 1].float(), kd[slots], vd[slots], L - 1, window=window, sinks=sk)
        assert rel_err(out[s:s + 1], ref) < 2e-2, (s, L)


def test_attn_decode_fp8_out():
    from loken_b200.ops import attention, gemm, rows

    torch.manual_seed(5)
    hd, n_q, n_kv, bs, L, B = 128, 8, 2, 16, 200, 3
    max_blocks = (L + bs - 1) // bs
    cache = rows.KVCacheLayer(B * max_blocks * bs, n_kv, hd, DEV, q8=True)
    bt = torch.arange(B * max_blocks, device=DEV, dtype=torch.int32).view(B, max_blocks)
    k = torch.randn(B * max_blocks * bs, n_kv, hd, device=DEV)
    v = torch.randn_like(k)
    _fill_cache(cache, k, v, torch.arange(k.shape[0], device=DEV))
    q = torch.randn(B, n_q, hd, device=DEV).bfloat16()
    lens = torch.full((B,), L, device=DEV, dtype=torch.int32)
    ref = attention.decode(q, cache, bt, lens, block_size=bs, nsplit=2)
    f8 = rows.alloc_fp8_act(B, n_q * hd, DEV)
    attention.decode(q, cache, bt, lens, block_size=bs, nsplit=2, out_fp8=f8)
    assert rel_err(gemm.dequantize_act_fp8(f8, B), ref) < 0.07


@pytest.mark.parametrize("hd,n_q,n_kv,window,sinks", [(128, 8, 1, 0, False), (128, 8, 2, 0, False),
                                                       (128, 4, 4, 0, False), (64, 8, 1, 128, True),
                                                       (64, 16, 4, 0, True), (128, 16, 2, 200, False),
                                                       # groups of 3, 5 and 6 heads run in the next larger tile shape
                                                       (128, 6, 2, 0, False), (128, 10, 2, 100, True), (64, 12, 2, 0, False)])
def test_attn_prefill(hd, n_q, n_kv, window, sinks):
    from loken_b200.ops import attention, rows

    torch.manual_seed(hd + n_q + window)
    bs = 16
    q_lens = [5, 130, 300, 33]
    kv_lens = [5, 130, 450, 161]   # the last two continue a cached prefix
    B = len(q_lens)
    max_blocks = (max(kv_lens) + bs - 1) // bs
    nblocks = B * max_blocks + 2
    cache = rows.KVCacheLayer(nblocks * bs, n_kv, hd, DEV, q8=True)
    perm = torch.randperm(nblocks, device=DEV)[:B * max_blocks].view(B, max_blocks).int()
    for s, L in enumerate(kv_lens):
        k = torch.randn(L, n_kv, hd, device=DEV)
        v = torch.randn(L, n_kv, hd, device=DEV)
        t = torch.arange(L, device=DEV)
        _fill_cache(cache, k, v, perm[s, (t // bs).long()].long() * bs + t % bs)
    kd, vd = cache.dequant()
    G = n_q // n_kv
    plan = attention.plan_prefill(q_lens, kv_lens, G, DEV)
    kk, vt = attention.kv_gather(cache, perm, plan, bs)
    q = torch.randn(sum(q_lens), n_q, hd, device=DEV).bfloat16()
    sk = torch.randn(n_q, device=DEV) if sinks else None
    out = attention.prefill(q, kk, vt, plan, window=window, sinks=sk)
    torch.cuda.synchronize()
    assert _status() == 0
    qs = 0
    for s, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        t = torch.arange(kl, device=DEV)
        slots = perm[s, (t // bs).long()].long() * bs + t % bs
        # the gather itself
        off = int(plan.kv_off[s])
        assert rel_err(kk[off:off + kl], kd[slots]) < 1e-2
        assert rel_err(vt[:, :, off:off + kl].permute(2, 0, 1), vd[slots]) < 1e-2
        ref = attention.attention_ref(q[qs:qs + ql].float(), kd[slots], vd[slots], kl - ql, window=window, sinks=sk)
        assert rel_err(out[qs:qs + ql], ref) < 2e-2, (s, ql, kl)
        qs += ql


# ------------------------------------------------------------------ sampler
def test_argmax_and_penalty():
    from loken_b200.ops import sampling

    torch.manual_seed(2)
    B, V = 9, 50257
    x = torch.randn(B, V, device=DEV)
    x[0, 100] = x[0, 7] = 50.0   # tie: lowest index wins
    out = sampling.argmax(x)
    assert out[0].item() == 7
    assert torch.equal(out[1:].long(), x[1:].argmax(-1))
    recent = torch.full((B, 8), -1, device=DEV, dtype=torch.int32)
    recent[1, :3] = torch.tensor([5, 5, 9])
    pen = torch.full((B,), 1.0, device=DEV)
    pen[1] = 2.0
    x0 = x.clone()
    sampling.repeat_penalty_(x, recent, pen)
    for t in (5, 9):
        v = x0[1, t]
        assert torch.allclose(x[1, t], v / 2 if v > 0 else v * 2)
    x0[1, 5], x0[1, 9] = x[1, 5], x[1, 9]
    assert torch.equal(x, x0)


@pytest.mark.parametrize("T,k,p,mp", [(0.0, 0, 1.0, 0.0), (0.7, 0, 0.9, 0.0), (1.0, 40, 1.0, 0.0),
                                      (0.8, 40, 0.9, 0.0), (1.3, 0, 1.0, 0.05), (1.0, 5, 0.5, 0.0)])
def test_sample_matches_reference(T, k, p, mp):
    from loken_b200.ops import sampling

    torch.manual_seed(11)
    B, V = 16, 32000
    x = (torch.randn(B, V, device=DEV) * 2).bfloat16().float()   # bf16-rounded: ties at the cuts
    u = torch.rand(B, device=DEV)
    out = sampling.sample(x, torch.full((B,), T, device=DEV), u,
                          top_k=torch.full((B,), k, device=DEV, dtype=torch.int32),
                          top_p=torch.full((B,), p, device=DEV), min_p=torch.full((B,), mp, device=DEV))
    torch.cuda.synchronize()
    hits = 0
    for b in range(B):
        want = sampling.sample_ref(x[b], T, float(u[b]), k, p, mp)
        hits += int(out[b].item() == want)
    # fp32 exp on the device vs float64 on the host may move a draw that lands within rounding
    # of a boundary: allow one row of sixteen
    assert hits >= B - 1


@pytest.mark.parametrize("V", [1000, 32000, 128256, 151936])
def test_cluster_sampler_equals_the_one_cta_sampler(V):
    """Up to 37 rows a cluster of eight CTAs shares each row (logits in registers, histograms merged through
    distributed shared memory).  Masses are fixed-point integers, so every cut and draw equals the one-CTA
    kernel's exactly, whatever the mix of rules per row."""
    from loken_b200.ops import sampling
    from loken_b200.ops._lib import cuda_lib

    torch.manual_seed(V)
    B = 24
    x = (torch.randn(B, V, device=DEV) * 3).bfloat16().float()        # bf16-rounded: ties at the cuts
    x[3, 100:] = float("-inf")                                        # a nearly empty row
    x[4] = 0.25                                                       # one value everywhere: all ties
    x[5, ::2] = float("-inf")
    T = torch.tensor([0.0, 0.7, 1.0, 0.8, 1.3, 1.0] * 4, device=DEV)
    k = torch.tensor([0, 0, 40, 40, 0, 5] * 4, device=DEV, dtype=torch.int32)
    p = torch.tensor([1.0, 0.9, 1.0, 0.9, 1.0, 0.5] * 4, device=DEV)
    mp = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.05, 0.0] * 4, device=DEV)
    for seed in range(3):
        u = torch.rand(B, device=DEV, generator=torch.Generator(device=DEV).manual_seed(seed))
        got = sampling.sample(x, T, u, top_k=k, top_p=p, min_p=mp)
        try:
            cuda_lib().lk_sample_cluster(0)
            want = sampling.sample(x, T, u, top_k=k, top_p=p, min_p=mp)
        finally:
            cuda_lib().lk_sample_cluster(1)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (got.tolist(), want.tolist())
        assert ((got >= 0) & (got < V)).all()


def test_sample_distribution():
    from loken_b200.ops import sampling

    torch.manual_seed(4)
    V, N = 1000, 20000
    logits = torch.randn(V, device=DEV) * 2
    x = logits[None].expand(N, V).contiguous()
    u = torch.rand(N, device=DEV)
    out = sampling.sample(x, torch.full((N,), 1.0, device=DEV), u,
                          top_k=torch.full((N,), 10, device=DEV, dtype=torch.int32))
    top = torch.topk(logits, 10)
    probs = torch.softmax(top.values, 0)
    counts = torch.stack([(out == i).sum() for i in top.indices]).float() / N
    assert (out[:, None] == top.indices[None]).any(1).all()
    assert (counts - probs).abs().max() < 0.02


@pytest.mark.parametrize("n_q,n_kv,lens,window,sinks,nsplit,rows_per_seq", [
    (8, 1, [1, 17, 300, 777, 64], 0, False, 1, 1),
    (64, 8, [1056, 130, 2049], 0, False, 2, 1),
    (8, 2, [500, 33], 0, True, 3, 1),
    (16, 4, [400, 129, 128, 127], 100, False, 2, 1),
    (4, 4, [260], 0, False, 1, 1),
    (8, 1, [200, 90], 0, False, 2, 3),          # several query rows per sequence (verify rows)
])
def test_attn_decode_tensor_core_kernel(n_q, n_kv, lens, window, sinks, nsplit, rows_per_seq):
    """The tcgen05 decode kernel against the fp32 reference, and against the SIMT kernel."""
    from loken_b200.ops import attention, rows

    torch.manual_seed(n_q * 31 + len(lens))
    hd, bs = 128, 16
    B = len(lens)
    max_blocks = (max(lens) + bs - 1) // bs
    nblocks = B * max_blocks + 5
    cache = rows.KVCacheLayer(nblocks * bs, n_kv, hd, DEV, q8=True)
    perm = torch.randperm(nblocks, device=DEV)[:B * max_blocks].view(B, max_blocks).int()
    for s, L in enumerate(lens):
        k = torch.randn(L, n_kv, hd, device=DEV)
        v = torch.randn(L, n_kv, hd, device=DEV)
        t = torch.arange(L, device=DEV)
        _fill_cache(cache, k, v, perm[s, (t // bs).long()].long() * bs + t % bs)
    kd, vd = cache.dequant()
    R = B * rows_per_seq
    q = torch.randn(R, n_q, hd, device=DEV).bfloat16()
    sk = torch.randn(n_q, device=DEV) if sinks else None
    row_seq = torch.arange(B, device=DEV, dtype=torch.int32).repeat_interleave(rows_per_seq)
    # row j of a sequence sees all but the last (rows_per_seq - 1 - j) keys
    vis = torch.tensor([L - (rows_per_seq - 1 - j) for L in lens for j in range(rows_per_seq)], device=DEV,
                       dtype=torch.int32)
    outs = {}
    for kern in ("tc", "simt"):
        attention.DECODE_KERNEL = kern
        try:
            outs[kern] = attention.decode(q, cache, perm, vis, block_size=bs, window=window, sinks=sk, nsplit=nsplit,
                                          row_seq=row_seq if rows_per_seq > 1 else None).clone()
        finally:
            attention.DECODE_KERNEL = "tc"
        torch.cuda.synchronize()
        assert _status() == 0, kern
    for r in range(R):
        s = r // rows_per_seq
        L = int(vis[r])
        t = torch.arange(lens[s], device=DEV)
        slots = perm[s, (t // bs).long()].long() * bs + t % bs
        ref = attention.attention_ref(q[r:r + 1].float(), kd[slots][:L], vd[slots][:L], L - 1, window=window, sinks=sk)
        assert rel_err(outs["tc"][r:r + 1], ref) < 2e-2, (r, L)
    assert rel_err(outs["tc"], outs["simt"].float()) < 2e-2
