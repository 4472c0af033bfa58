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
