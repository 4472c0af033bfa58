"""Block-fp8 safetensors round trip on CPU: write, read whole and as tensor-parallel shards."""
import torch

from loken_b200.models import loader_hf
from loken_b200.models.config import tiny
from loken_b200.models.weights import dequant_linear, random_weights


def test_block_fp8_safetensors_round_trip(tmp_path):
    cfg = tiny("llama", weight_format="fp8_block", head_dim=128, n_q=4, n_kv=2, hidden=512, intermediate=1024)
    cfg.rope_pairing = 1
    w = random_weights(cfg, torch.device("cpu"), seed=2, std=0.05)
    loader_hf.save_hf_fp8(str(tmp_path), cfg, w)
    got, hf = loader_hf.load_hf(str(tmp_path), torch.device("cpu"))
    assert hf["quantization_config"]["weight_block_size"] == [128, 128]
    c2 = got.cfg
    assert (c2.n_layers, c2.hidden, c2.n_q, c2.n_kv, c2.head_dim, c2.weight_format) == \
        (cfg.n_layers, 512, 4, 2, 128, "fp8_block")
    for a, b in zip(w.layers, got.layers):
        for name in ("wqkv", "wo", "w_gate_up", "w_down"):
            la, lb = getattr(a, name), getattr(b, name)
            assert lb.kind == "fp8_block"
            assert torch.equal(la.weight.data.view(torch.uint8), lb.weight.data.view(torch.uint8))
            assert torch.equal(la.weight.scale, lb.weight.scale)
    shards = [loader_hf.load_hf(str(tmp_path), torch.device("cpu"), tp_rank=r, tp_size=2)[0] for r in range(2)]
    full = dequant_linear(got.layers[0].wo)
    assert torch.equal(torch.cat([dequant_linear(s.layers[0].wo) for s in shards], 1), full)
    gu = dequant_linear(got.layers[1].w_gate_up)
    I = cfg.intermediate
    assert torch.equal(torch.cat([dequant_linear(s.layers[1].w_gate_up)[:I // 2] for s in shards], 0), gu[:I])
    assert all(s.layers[0].wqkv.kind == "fp8_block" for s in shards)


def test_awq_tensors_expand_to_the_weights_they_encode():
    import torch

    from loken_b200.models.loader_hf import AWQ_ORDER, awq_dequant

    g = torch.Generator().manual_seed(4)
    n_in, n_out, group = 256, 64, 128
    q = torch.randint(0, 16, (n_in, n_out), generator=g, dtype=torch.int32)
    z = torch.randint(0, 16, (n_in // group, n_out), generator=g, dtype=torch.int32)
    s = (torch.rand(n_in // group, n_out, generator=g) * 0.02 + 0.001).half()

    def pack(t):
        out = torch.zeros(t.shape[0], t.shape[1] // 8, dtype=torch.int64)
        for i, col in enumerate(AWQ_ORDER):
            out |= t[:, col::8].to(torch.int64) << (4 * i)
        return out.to(torch.int32)          # wraps the top nibble into the sign bit, as the files do

    w = awq_dequant(pack(q), pack(z), s)
    want = ((q - z.repeat_interleave(group, 0)).float() * s.float().repeat_interleave(group, 0)).t()
    assert w.shape == (n_out, n_in) and torch.equal(w, want)


def test_awq_tensors_stay_4_bit_planes_on_one_rank():
    """Groups of 128: the codes keep their values in the plane format of the dp4a GEMV; decoding the planes gives
    exactly the weights the tensors encode."""
    from loken_b200.models.loader_hf import AWQ_ORDER, awq_dequant, awq_planes
    from loken_b200.ops import quant

    g = torch.Generator().manual_seed(7)
    n_in, n_out = 256, 64

    def pack(t):
        out = torch.zeros(t.shape[0], t.shape[1] // 8, dtype=torch.int64)
        for i, col in enumerate(AWQ_ORDER):
            out |= t[:, col::8].to(torch.int64) << (4 * i)
        return out.to(torch.int32)

    class Sh:
        def __init__(self):
            self.t = {}
            for stem in ("a", "b"):
                q = torch.randint(0, 16, (n_in, n_out), generator=g, dtype=torch.int32)
                z = torch.randint(0, 16, (n_in // 128, n_out), generator=g, dtype=torch.int32)
                s = (torch.rand(n_in // 128, n_out, generator=g) * 0.02 + 0.001).half()
                self.t.update({stem + ".qweight": pack(q), stem + ".qzeros": pack(z), stem + ".scales": s})

        def has(self, n):
            return n in self.t

        def get(self, n):
            return self.t[n]

    sh = Sh()
    lin = awq_planes(sh, ["a", "b"], [None, slice(16, 48)], torch.device("cpu"))
    assert lin.kind == "gguf" and lin.weight.aq_fmt == quant.AQ_W4G128 and (lin.weight.rows, lin.weight.K) == (96, 256)
    want = torch.cat([awq_dequant(sh.get("a.qweight"), sh.get("a.qzeros"), sh.get("a.scales")),
                      awq_dequant(sh.get("b.qweight"), sh.get("b.qzeros"), sh.get("b.scales"))[16:48]], 0)
    got = quant.dequantize_weight(lin.weight)
    # the minimum is stored as zero x scale in f16: one more rounding than (q - zero) * scale
    assert (got - want).abs().max().item() <= 2e-3 * want.abs().max().item()
    assert awq_planes(sh, ["a", "missing"], [None, None], torch.device("cpu")) is None
