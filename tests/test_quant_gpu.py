"""Dequant-fused GEMM over GGUF block formats against fp32 PyTorch on the decoded weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-9)).item()


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k", "q6_k", "mxfp4"])
@pytest.mark.parametrize("M,N,K", [(1, 256, 256), (5, 384, 1024), (40, 1000, 512), (130, 640, 768), (300, 2304, 256)])
def test_linear_gguf(fmt, M, N, K):
    from loken_b200.ops import quant
    from loken_b200.ops._lib import Workspace

    torch.manual_seed(M + N)
    w = torch.randn(N, K, device=DEV) * 0.05
    q = quant.quantize_weight(w, fmt)
    wd = quant.dequantize_weight(q)
    assert rel_err(wd, w) < {"q8_0": 0.01, "q4_k": 0.12, "q6_k": 0.04, "mxfp4": 0.3}[fmt]
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    bias = torch.randn(N, device=DEV)
    ref = x.float() @ wd.bfloat16().float().t() + bias     # the kernel rounds decoded weights to bf16
    wsp = Workspace.get(torch.device(DEV))
    if fmt == "mxfp4":
        # the default route: weights as stored on the block-scaled MMA, activations to e4m3 (3 mantissa
        # bits: a few per cent of the largest output on the worst element; tests/test_mx_gpu.py checks the
        # product of the quantised operands exactly)
        out = quant.linear_gguf(x, q, bias=bias)
        torch.cuda.synchronize()
        assert wsp.read_status() == 0
        assert rel_err(out, ref) < 5e-2
        quant.MX_NATIVE = False        # and the dequant-fused route below
    try:
        out = quant.linear_gguf(x, q, bias=bias)
        torch.cuda.synchronize()
        assert wsp.read_status() == 0
        assert rel_err(out, ref) < 1e-2
        out2 = quant.linear_gguf(x, q, bias=bias, splits=2)
        assert rel_err(out2, ref) < 1e-2
    finally:
        quant.MX_NATIVE = True


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k", "q6_k"])
@pytest.mark.parametrize("M", [1, 2, 3, 8])
# streaming form: ragged rows, two chunks, 1024-value chunks; register form: a tail chunk, one block
@pytest.mark.parametrize("N,K", [(300, 2048), (300, 4096), (2000, 3072), (4096, 1280), (1234, 256)])
def test_gemv_dp4a_matches_the_integer_product_and_the_gemm(fmt, M, N, K):
    """Up to eight token rows run as a GEMV on int8 activations: it equals the product of the activations as
    quantised (per 32 values, amax / 127) with the decoded weights, and stays within the int8 noise of the
    tensor-core route that larger batches take."""
    from loken_b200.ops import quant

    torch.manual_seed(N + K + M)
    w = torch.randn(N, K, device=DEV) * 0.05
    q = quant.quantize_weight(w, fmt)
    wd = quant.dequantize_weight(q)
    x = (torch.randn(M, K, device=DEV) * torch.rand(M, 1, device=DEV) * 2).bfloat16()
    bias = torch.randn(N, device=DEV) * 0.1
    g = x.float().view(M, K // 32, 32)
    d = g.abs().amax(2, keepdim=True) / 127.0
    xq = (torch.round(g / d.clamp_min(1e-30)).clamp(-127, 127) * d).view(M, K)
    exact = xq @ wd.t() + bias
    out = quant.linear_gguf(x, q, bias=bias)
    torch.cuda.synchronize()
    # bf16 rounding of the output; the Q4_K minimum term uses the sum of the unquantised activations (closer to
    # the true product than the sum of their codes), which this emulation does not
    assert rel_err(out, exact) < (2e-2 if fmt == "q4_k" else 1e-2)
    assert rel_err(out, x.float() @ wd.t() + bias) < 2e-2
    old = quant.GEMV_MAX_M
    try:
        quant.GEMV_MAX_M = 0
        gemm = quant.linear_gguf(x, q, bias=bias)
    finally:
        quant.GEMV_MAX_M = old
    assert rel_err(out, gemm) < 2e-2                   # the reference's bar for 8-bit activations
    again = quant.linear_gguf(x, q, bias=bias)
    assert torch.equal(out, again)
    # the register form (the only one for shapes the bulk-copy ring does not take) agrees up to summation order
    from loken_b200.ops._lib import Workspace, cuda_lib

    try:
        cuda_lib().lk_gemv_q_stream(0)
        reg = quant.linear_gguf(x, q, bias=bias)
    finally:
        cuda_lib().lk_gemv_q_stream(1)
    torch.cuda.synchronize()
    assert rel_err(out, reg) < 1e-2
    assert Workspace.get(torch.device(DEV)).read_status() == 0


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k", "q6_k"])
@pytest.mark.parametrize("M,N,K", [(129, 1000, 512), (700, 2304, 1024)])
def test_prompt_sized_gemm_decodes_the_matrix_once(fmt, M, N, K):
    """From 129 token rows on the planes are decoded to bf16 in row chunks and the bf16 GEMM multiplies:
    the decoded rows equal the reference decode, and the product equals the fused kernel's."""
    from loken_b200.ops import quant
    from loken_b200.ops._lib import Workspace

    torch.manual_seed(N + K)
    q = quant.quantize_weight(torch.randn(N, K, device=DEV) * 0.05, fmt)
    wd = quant.dequantize_weight(q)
    got = quant.dequant_rows(q, 128, N, torch.empty(N - 128, K, dtype=torch.bfloat16, device=DEV))
    assert (got.float() - wd[128:]).abs().max().item() <= wd.abs().max().item() * 2.0 ** -7
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    bias = torch.randn(N, device=DEV)
    ref = x.float() @ wd.bfloat16().float().t() + bias
    old = quant.DEQUANT_ONCE_MIN_M, quant.DEQUANT_CHUNK_BYTES
    try:
        quant.DEQUANT_CHUNK_BYTES = 256 * K * 2            # several chunks, the last one ragged
        once = quant.linear_gguf(x, q, bias=bias)
        once32 = quant.linear_gguf(x, q, bias=bias, out_fp32=True)
        quant.DEQUANT_ONCE_MIN_M = 0
        fused = quant.linear_gguf(x, q, bias=bias)
    finally:
        quant.DEQUANT_ONCE_MIN_M, quant.DEQUANT_CHUNK_BYTES = old
    torch.cuda.synchronize()
    assert Workspace.get(torch.device(DEV)).read_status() == 0
    assert once32.dtype == torch.float32
    assert rel_err(once, ref) < 1e-2 and rel_err(once32, ref) < 2e-3 and rel_err(once, fused) < 1e-2


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k", "q6_k"])
@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("ring", [1, 0])                    # the bulk-copy ring and the register form
def test_gemv_front_equals_the_separate_kernels(fmt, M, ring):
    """A GEMV can compute its activations from RMSNorm(x + pending update) or from a gated unit and fold an
    earlier update into the residual rows on the side: the result is that of the separate kernels."""
    from loken_b200.ops import quant, rows
    from loken_b200.ops._lib import Workspace, cuda_lib

    K, N = 2048, 520
    torch.manual_seed(M + K)
    cuda_lib().lk_gemv_q_stream(ring)
    try:
        _front_case(quant, rows, fmt, M, N, K)
    finally:
        cuda_lib().lk_gemv_q_stream(1)
    torch.cuda.synchronize()
    assert Workspace.get(torch.device(DEV)).read_status() == 0


def _front_case(quant, rows, fmt, M, N, K):
    q = quant.quantize_weight(torch.randn(N, K, device=DEV) * 0.05, fmt)
    x = torch.randn(M, K, device=DEV).bfloat16()
    delta = (torch.randn(M, K, device=DEV) * 0.3).bfloat16()
    gamma = 1 + 0.1 * torch.randn(K, device=DEV)
    # norm in front; x itself stays as it was
    x1 = x.clone()
    h = torch.empty_like(x)
    rows.add_rmsnorm(x1, gamma, 1e-5, delta=delta, out=h, rows=M)
    want = quant.linear_gguf(h, q)
    x2 = x.clone()
    got = quant.linear_gguf(x2, q, front=quant.GemvFront(norm=gamma, eps=1e-5, delta=delta))
    assert torch.equal(x2, x)
    assert rel_err(got, want) < 1e-2
    got0 = quant.linear_gguf(x1, q, front=quant.GemvFront(norm=gamma, eps=1e-5))        # nothing pending
    assert rel_err(got0, want) < 1e-2
    # gated unit in front, and the pending update folded into other rows on the side
    for mode, alpha, limit in ((0, 0.0, 0.0), (1, 1.702, 7.0)):
        gu = (torch.randn(M, 2 * K, device=DEV) * 2).bfloat16()
        act = torch.empty(M, K, device=DEV, dtype=torch.bfloat16)
        rows.glu(gu, mode=mode, alpha=alpha, limit=limit, out=act, rows=M)
        want = quant.linear_gguf(act, q)
        res = torch.randn(8, K, device=DEV).bfloat16()
        res0 = res.clone()
        got = quant.linear_gguf(gu, q, front=quant.GemvFront(glu=(mode, alpha, limit), update=(res, delta)))
        assert rel_err(got, want) < 1e-2
        assert torch.equal(res[:M], (res0[:M].float() + delta.float()).bfloat16()) and torch.equal(res[M:], res0[M:])
    with pytest.raises(ValueError):
        quant.linear_gguf(torch.zeros(9, K, device=DEV, dtype=torch.bfloat16), q, front=quant.GemvFront(norm=gamma))


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k_m"])
@pytest.mark.parametrize("arch", ["gpt-oss", "olmoe"])
@pytest.mark.parametrize("T", [1, 3, 8])
def test_decode_size_mixture_layers_run_their_experts_as_gemv_slots(arch, fmt, T):
    """Up to 64 (token, expert) pairs the experts of a GGUF mixture layer run as slots of the streaming GEMV (the
    expert of a slot read on the device, the gated unit in front of the down projection): same result as the
    planned grouped GEMMs, within the int8 noise of the activations, and as the fp32 definition."""
    import dataclasses

    from loken_b200.models.config import tiny
    from loken_b200.models.moe import MoeRunner, dequant_experts, random_moe
    from loken_b200.models.reference import moe_ref
    from loken_b200.ops._lib import Workspace

    cfg = dataclasses.replace(tiny(arch, weight_format=fmt), n_experts=8, top_k=4, hidden=512, expert_intermediate=256,
                              n_layers=1)
    gen = torch.Generator(device=DEV).manual_seed(T)
    moe = random_moe(cfg, gen, DEV, 0.05)

    class W:
        pass
    w, lay = W(), W()
    w.embed = torch.zeros(1, device=DEV)
    lay.moe = moe
    w.layers = [lay]
    run = MoeRunner(cfg, w, 16)
    assert run._slots_ok(moe, T) and not run._slots_ok(moe, 17)
    h = torch.randn(16, cfg.hidden, device=DEV).bfloat16()
    got = torch.zeros(16, cfg.hidden, device=DEV, dtype=torch.bfloat16)
    plan = torch.zeros_like(got)
    run.forward(0, moe, h, got, T)
    old = MoeRunner.SLOT_MAX_PAIRS
    try:
        MoeRunner.SLOT_MAX_PAIRS = 0
        run.forward(0, moe, h, plan, T)
    finally:
        MoeRunner.SLOT_MAX_PAIRS = old
    torch.cuda.synchronize()
    assert Workspace.get(torch.device(DEV)).read_status() == 0
    want = moe_ref(h[:T].float(), moe, cfg)
    scale = want.abs().max().item()
    # two chained products on int8 activations (the reference's bar for one is 2e-2 of the largest output)
    assert (got[:T].float() - want).abs().max().item() < 5e-2 * scale
    assert (got[:T].float() - plan[:T].float()).abs().max().item() < 5e-2 * scale
    assert (got[T:] == 0).all()


@pytest.mark.parametrize("N,K", [(520, 2048), (300, 1280)])
def test_awq_planes_run_the_gemv_and_the_decode_once_gemm(N, K):
    """AWQ's 4-bit weights (groups of 128: scale and zero point) as device planes: up to eight token rows on the
    dp4a GEMV (both forms), more rows decoded once per call for the bf16 GEMM."""
    from loken_b200.ops import quant
    from loken_b200.ops._lib import Workspace, cuda_lib

    g = torch.Generator(device=DEV).manual_seed(N)
    qv = torch.randint(0, 16, (N, K), generator=g, device=DEV, dtype=torch.int32)
    z = torch.randint(0, 16, (N, K // 128), generator=g, device=DEV, dtype=torch.int32)
    s = (torch.rand(N, K // 128, generator=g, device=DEV) * 0.02 + 0.001).half()
    w = quant.from_awq(qv, z, s, DEV)
    wd = quant.dequantize_weight(w)
    assert (wd - (qv - z.repeat_interleave(128, 1)).float() * s.float().repeat_interleave(128, 1)).abs().max() < 2e-3
    x = (torch.randn(300, K, device=DEV) * 0.5).bfloat16()
    bias = torch.randn(N, device=DEV) * 0.1
    ref = x.float() @ wd.t() + bias
    for M in (1, 3, 8):
        outs = []
        for ring in (1, 0):
            try:
                cuda_lib().lk_gemv_q_stream(ring)
                outs.append(quant.linear_gguf(x[:M], w, bias=bias))
            finally:
                cuda_lib().lk_gemv_q_stream(1)
        for o in outs:
            assert rel_err(o, ref[:M]) < 2e-2
        assert rel_err(outs[0], outs[1]) < 1e-2
    for M in (20, 300):
        assert rel_err(quant.linear_gguf(x[:M], w, bias=bias), ref[:M]) < 1e-2
    torch.cuda.synchronize()
    assert Workspace.get(torch.device(DEV)).read_status() == 0
