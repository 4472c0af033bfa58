"""The block-scaled (MX) path: activation quantiser and the `kind::mxf8f6f4.block_scale` GEMM with
MXFP4 weights as stored, each against a plain PyTorch fp32 reference of the same op."""
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


@pytest.mark.parametrize("R,K", [(1, 32), (5, 320), (64, 2880), (130, 4096)])
def test_quant_mx8_matches_reference(R, K):
    from loken_b200.ops import mx

    torch.manual_seed(R + K)
    x = (torch.randn(R, K, device=DEV) * torch.logspace(-3, 2, R, device=DEV)[:, None]).bfloat16()
    x[0, :32] = 0                               # an all-zero group
    got = mx.quant_mx8(x)
    ref = mx.quant_mx8_ref(x)
    torch.cuda.synchronize()
    assert torch.equal(got.sf, ref.sf)
    assert torch.equal(got.data.view(torch.uint8), ref.data.view(torch.uint8))
    # and it is a faithful quantisation: e4m3 has 3 mantissa bits
    back = mx.dequant_mx_act(got)
    err = (back - x.float()).abs().view(R, K // 32, 32)
    amax = x.float().abs().view(R, K // 32, 32).amax(2, keepdim=True)
    assert (err <= amax * 0.0625 + 1e-30).all()


def test_quant_mx8_gather_and_glu():
    from loken_b200.ops import mx

    torch.manual_seed(3)
    T, k, H, I = 9, 4, 320, 256
    x = torch.randn(T, H, device=DEV).bfloat16()
    pair_row = torch.randperm(T * k, device=DEV).int()
    pair_row[5] = -1
    out = mx.alloc_mx_act(T * k, H, DEV)
    out.data.view(torch.uint8).fill_(0x11)
    mx.quant_mx8(x, out=out, rows=T * k, K=H, pair_row=pair_row, kdiv=k)
    ref = mx.quant_mx8_ref(x)
    for p in range(T * k):
        r = int(pair_row[p])
        if r >= 0:
            assert torch.equal(out.data[r].view(torch.uint8), ref.data[p // k].view(torch.uint8))
            assert torch.equal(out.sf[r], ref.sf[p // k])
    untouched = 5
    gu = torch.randn(T, 2 * I, device=DEV).bfloat16() * 3
    for mode in (0, 1):
        got = mx.quant_mx8(gu, rows=T, K=I, glu_mode=mode, alpha=1.702, limit=7.0)
        g, u = gu[:, :I].float(), gu[:, I:].float()
        if mode == 0:
            act = torch.nn.functional.silu(g) * u
        else:
            gg, uu = g.clamp(max=7.0), u.clamp(-7.0, 7.0)
            act = gg * torch.sigmoid(1.702 * gg) * (1 + uu)
        back = mx.dequant_mx_act(got)
        err = ((back - act).abs().max() / act.abs().max()).item()
        assert err < 0.07, (mode, err)
    del untouched
    assert _status() == 0


@pytest.mark.parametrize("M,N,K", [(16, 256, 128), (1, 384, 320), (64, 2880, 2880), (40, 5760, 2880),
                                   (128, 1024, 4096), (100, 640, 96)])
def test_linear_mx_matches_fp32_of_the_same_operands(M, N, K):
    """The tensor core multiplies exactly the stored values (E2M1 x e4m3, exponents applied in
    hardware) and accumulates in fp32: against the fp32 product of the dequantised operands the
    difference is accumulation order only."""
    from loken_b200.ops import mx, quant

    torch.manual_seed(M * 3 + N)
    w = torch.randn(N, K, device=DEV) * 0.05
    qw = quant.quantize_weight_torch(w, "mxfp4")
    mw = mx.mx_weight(qw)
    x = (torch.randn(M, K, device=DEV) * 0.7).bfloat16()
    xa = mx.quant_mx8(x)
    bias = torch.randn(N, device=DEV)
    out = mx.linear_mx(xa, mw, bias=bias)
    torch.cuda.synchronize()
    assert _status() == 0
    ref = mx.dequant_mx_act(xa) @ quant.dequantize_weight(qw).t() + bias
    err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
    assert err < 6e-3, err            # bf16 output rounding
    # and against the product with unquantised activations: e4m3 keeps 3 mantissa bits (the reference
    # project's bar of 2e-2 is for int8 activations, which keep 7), so the worst element of a
    # K = 4096 dot product may be off by a few per cent of the largest output
    full = x.float() @ quant.dequantize_weight(qw).t() + bias
    assert ((out.float() - full).abs().max() / full.abs().max()).item() < 4e-2


def test_moe_layer_mx_against_the_dequantising_path():
    import dataclasses

    from loken_b200.models.config import get_config
    from loken_b200.models.moe import MoeRunner, dequant_experts, random_moe

    cfg = dataclasses.replace(get_config("gpt-oss-120b"), n_experts=8, top_k=2, hidden=320, expert_intermediate=256,
                              n_layers=1)
    gen = torch.Generator(device=DEV).manual_seed(0)
    moe = random_moe(cfg, gen, DEV, 0.05)

    class W:
        pass
    w = W()
    w.embed = torch.zeros(1, device=DEV)
    lay = W()
    lay.moe = moe
    w.layers = [lay]
    T = 37
    run = MoeRunner(cfg, w, T)
    assert run.use_mx
    h = torch.randn(T, cfg.hidden, device=DEV).bfloat16()
    out = torch.zeros(T, cfg.hidden, device=DEV, dtype=torch.bfloat16)
    run.forward(0, moe, h, out, T)
    torch.cuda.synchronize()
    assert _status() == 0
    # fp32 oracle of the layer
    gu, dn = dequant_experts(moe)
    logits = h.float() @ moe.router_w.float().t() + moe.router_b
    top = torch.topk(logits, cfg.top_k, dim=1)
    wts = torch.softmax(top.values, dim=1)
    want = torch.zeros(T, cfg.hidden, device=DEV)
    I = cfg.expert_intermediate
    for t in range(T):
        for j in range(cfg.top_k):
            e = int(top.indices[t, j])
            z = gu[e] @ h[t].float() + moe.gate_up_b[e]
            g, u = z[:I].clamp(max=cfg.glu_limit), z[I:].clamp(-cfg.glu_limit, cfg.glu_limit)
            a = g * torch.sigmoid(cfg.glu_alpha * g) * (1 + u)
            want[t] += wts[t, j] * (dn[e] @ a + moe.down_b[e])
    # two chained products with e4m3 activations: an e4m3 rounding is uniform within +-6.25 %, i.e.
    # 3.6 % rms per value, and in a sum of random-sign terms that does not average down: each product
    # carries ~3.6 % of a typical output as noise, two in a row ~5 %
    d = (out.float() - want).abs()
    assert (d.max() / want.abs().max()).item() < 0.1
    assert (d.mean() / want.abs().mean()).item() < 6e-2


@pytest.mark.parametrize("T,E", [(37, 128), (1, 32), (130, 128), (300, 60)])     # 1, 2 and 4 tokens per CTA; ragged ends
@pytest.mark.parametrize("mode", ["softmax_topk", "softmax", "sigmoid"])
def test_fused_router_matches_torch(mode, T, E):
    import ctypes as C

    from loken_b200.models.moe import ROUTER_MODE
    from loken_b200.ops._lib import cuda_lib, ptr, stream

    torch.manual_seed(5)
    H, k = 2880, 4
    h = torch.randn(T, H, device=DEV).bfloat16()
    w = (torch.randn(E, H, device=DEV) * 0.05).bfloat16()
    b = torch.randn(E, device=DEV) * 0.1
    ids = torch.zeros(T, k, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T, k, dtype=torch.float32, device=DEV)
    lg = torch.zeros(T, E, dtype=torch.float32, device=DEV)
    rc = cuda_lib().lk_moe_router(ptr(h), C.c_longlong(h.stride(0)), ptr(w), ptr(b), T, H, E, k, ROUTER_MODE[mode], 1,
                                  ptr(ids), ptr(wts), ptr(lg), C.c_longlong(E), stream())
    assert rc == 0
    torch.cuda.synchronize()
    ref = h.float() @ w.float().t() + b
    assert ((lg - ref).abs().max() / ref.abs().max()).item() < 1e-4
    sc = lg if mode == "softmax_topk" else torch.softmax(lg, 1) if mode == "softmax" else torch.sigmoid(lg)
    top = torch.topk(sc, k, dim=1)
    assert torch.equal(ids.long(), top.indices)
    want = torch.softmax(top.values, 1) if mode == "softmax_topk" else top.values / top.values.sum(1, keepdim=True)
    assert ((wts - want).abs().max()).item() < 1e-5
