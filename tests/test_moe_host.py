"""Experts computed on the host cores over the device plane layouts, against the fp32 definition."""
import pytest
import torch

from loken_b200.cpu.moe_host import moe_pairs, plane_format
from loken_b200.ops import quant


@pytest.mark.parametrize("fmt", ["bf16", "q8_0", "q4_k", "q6_k", "mxfp4"])
@pytest.mark.parametrize("glu", [(0, 0.0, 0.0), (1, 1.702, 7.0)])
@pytest.mark.parametrize("level", [0, 2])
def test_host_expert_pairs_match_the_definition(fmt, glu, level):
    torch.manual_seed(3)
    E, H, I, T = 5, 256, 512, 3
    gu_f, dn_f = torch.randn(E * 2 * I, H) * 0.05, torch.randn(E * H, I) * 0.05
    if fmt == "bf16":
        gu, dn = gu_f.bfloat16(), dn_f.bfloat16()
        gud, dnd = gu.float(), dn.float()
    else:
        gu, dn = quant.quantize_weight_torch(gu_f, fmt), quant.quantize_weight_torch(dn_f, fmt)
        gud, dnd = quant.dequantize_weight(gu), quant.dequantize_weight(dn)
    assert plane_format(gu) is not None
    gub, dnb = torch.randn(E, 2 * I) * 0.1, torch.randn(E, H) * 0.1
    x = torch.randn(T, H)
    pairs = [(0, 4, 0.7), (0, 1, 0.3), (2, 4, 1.0), (1, 0, 0.25), (1, 3, 0.75)]
    out = torch.zeros(T, H)
    out[2] = 1.0                                                  # pairs add to what is there
    moe_pairs(gu, dn, x, [p[0] for p in pairs], [p[1] for p in pairs], [p[2] for p in pairs], H=H, I=I, out=out,
              gu_bias=gub, dn_bias=dnb, glu=glu, threads=3, max_level=level)
    want = torch.zeros(T, H)
    want[2] = 1.0
    for t, e, w in pairs:
        z = gud[e * 2 * I:(e + 1) * 2 * I] @ x[t] + gub[e]
        g, u = z[:I], z[I:]
        if glu[0] == 0:
            a = torch.nn.functional.silu(g) * u
        else:
            gg, uu = g.clamp(max=glu[2]), u.clamp(-glu[2], glu[2])
            a = gg * torch.sigmoid(glu[1] * gg) * (1 + uu)
        want[t] += w * (dnd[e * H:(e + 1) * H] @ a + dnb[e])
    # int8 activations twice in a row (none for bf16 weights)
    tol = 2e-3 if fmt == "bf16" else 4e-2
    if fmt == "mxfp4":
        assert gu.scales.stride(0) >= H // 32                    # the exponent plane may be padded: the pitch is passed
    assert (out - want).abs().max().item() < tol * want.abs().max().item()
