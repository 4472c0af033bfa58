"""GGUF container and block codecs (CPU): the C++ decoders against a numpy restatement of the
format definitions, encoder error bounds, and a write -> read round trip."""
import os
import struct

import numpy as np
import pytest

from loken_b200.formats import gguf


def f16(b):
    return np.frombuffer(b, dtype=np.float16).astype(np.float32)


def np_dequant_q8_0(raw, n):
    blk = raw.reshape(-1, 34)
    d = f16(blk[:, :2].tobytes())
    q = blk[:, 2:].view(np.int8).astype(np.float32)
    return (q * d[:, None]).reshape(n)


def np_dequant_q4_k(raw, n):
    out = np.empty(n, dtype=np.float32)
    blk = raw.reshape(-1, 144)
    for i, b in enumerate(blk):
        d, dmin = f16(b[0:2].tobytes())[0], f16(b[2:4].tobytes())[0]
        sc = b[4:16]
        qs = b[16:144]
        y = []
        for j in range(8):
            if j < 4:
                s, m = sc[j] & 63, sc[j + 4] & 63
            else:
                s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4)
                m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)
            q = qs[(j // 2) * 32:(j // 2) * 32 + 32]
            v = (q & 0xF) if j % 2 == 0 else (q >> 4)
            y.append(d * s * v.astype(np.float32) - dmin * m)
        out[i * 256:(i + 1) * 256] = np.concatenate(y)
    return out


def np_dequant_q6_k(raw, n):
    out = np.empty(n, dtype=np.float32)
    blk = raw.reshape(-1, 210)
    for i, b in enumerate(blk):
        ql, qh, sc = b[:128], b[128:192], b[192:208].view(np.int8)
        d = f16(b[208:210].tobytes())[0]
        y = np.empty(256, dtype=np.float32)
        for half in range(2):
            l_ = ql[half * 64:half * 64 + 64].astype(np.int32)
            h_ = qh[half * 32:half * 32 + 32].astype(np.int32)
            s_ = sc[half * 8:half * 8 + 8].astype(np.float32)
            for l in range(32):
                isx = l // 16
                q1 = ((l_[l] & 0xF) | (((h_[l] >> 0) & 3) << 4)) - 32
                q2 = ((l_[l + 32] & 0xF) | (((h_[l] >> 2) & 3) << 4)) - 32
                q3 = ((l_[l] >> 4) | (((h_[l] >> 4) & 3) << 4)) - 32
                q4 = ((l_[l + 32] >> 4) | (((h_[l] >> 6) & 3) << 4)) - 32
                base = half * 128
                y[base + l] = d * s_[isx] * q1
                y[base + l + 32] = d * s_[isx + 2] * q2
                y[base + l + 64] = d * s_[isx + 4] * q3
                y[base + l + 96] = d * s_[isx + 6] * q4
        out[i * 256:(i + 1) * 256] = y
    return out


LUT = np.array([0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12], dtype=np.float32)


def np_dequant_mxfp4(raw, n):
    blk = raw.reshape(-1, 17)
    e = blk[:, 0].astype(np.int32)
    d = np.where(e == 0, 2.0 ** -127, np.exp2((e - 127).astype(np.float64))).astype(np.float64) * 0.5
    qs = blk[:, 1:]
    lo, hi = LUT[qs & 0xF], LUT[qs >> 4]
    return (np.concatenate([lo, hi], axis=1) * d[:, None]).astype(np.float32).reshape(n)


@pytest.mark.parametrize("ty,ref,tol", [(gguf.Q8_0, np_dequant_q8_0, 0.006), (gguf.Q4_K, np_dequant_q4_k, 0.08),
                                         (gguf.Q6_K, np_dequant_q6_k, 0.025), (gguf.MXFP4, np_dequant_mxfp4, 0.27)])
def test_codec_matches_definition_and_bounds(ty, ref, tol):
    rng = np.random.default_rng(ty)
    x = (rng.standard_normal((8, 1024)) * rng.uniform(0.01, 3.0, (8, 1))).astype(np.float32)
    raw = gguf.quantize(x, ty)
    bv, bb = gguf.block_info(ty)
    assert raw.size == x.size // bv * bb
    got = gguf.dequantize(raw, ty, x.shape)
    want = ref(raw, x.size).reshape(x.shape)
    assert np.array_equal(got, want)                      # decoder == definition, bit for bit
    err = np.abs(got - x).max(axis=1) / np.abs(x).max(axis=1)
    assert err.max() < tol                                # encoder stays inside the format's envelope
    # random bytes decode the same way in both (no code path depends on the encoder)
    junk = rng.integers(0, 256, raw.size, dtype=np.uint8)
    if ty in (gguf.Q8_0, gguf.Q4_K, gguf.Q6_K):           # keep the f16 scale fields finite
        blk = junk.reshape(-1, bb)
        for off in ({gguf.Q8_0: [0], gguf.Q4_K: [0, 2], gguf.Q6_K: [208]}[ty]):
            blk[:, off:off + 2] = np.frombuffer(np.float16(0.37).tobytes(), dtype=np.uint8)
    assert np.array_equal(gguf.dequantize(junk, ty, x.shape), ref(junk, x.size).reshape(x.shape))


def test_q8_0_known_answer():
    x = np.zeros(32, dtype=np.float32)
    x[0], x[1], x[2] = 127.0, -63.5, 1.0
    raw = gguf.quantize(x, gguf.Q8_0)
    assert struct.unpack("<e", raw[:2].tobytes())[0] == 1.0
    assert list(raw[2:5].view(np.int8)) == [127, -64, 1]       # round half away from zero
    assert np.all(gguf.quantize(np.zeros(32, np.float32), gguf.Q8_0) == 0)


def test_f16_bf16_conversion():
    x = np.array([0.0, 1.0, -2.5, 65504.0, 1e-8, 3.14159], dtype=np.float32)
    h = gguf.dequantize(gguf.quantize(x, gguf.F16), gguf.F16, x.shape)
    assert np.array_equal(h, x.astype(np.float16).astype(np.float32))
    b = gguf.dequantize(gguf.quantize(x, gguf.BF16), gguf.BF16, x.shape)
    import torch

    assert np.array_equal(b, torch.tensor(x).bfloat16().float().numpy())


def test_gguf_round_trip(tmp_path):
    p = str(tmp_path / "t.gguf")
    rng = np.random.default_rng(0)
    a = rng.standard_normal((6, 256)).astype(np.float32)
    b = rng.standard_normal((3, 64)).astype(np.float32)
    w = gguf.GGUFWriter(p, alignment=64)
    w.add_meta("general.architecture", "llama")
    w.add_meta("llama.block_count", 2)
    w.add_meta("llama.rope.freq_base", 500000.0)
    w.add_meta("llama.flag", True)
    w.add_meta("tokenizer.ggml.tokens", ["<s>", "a", "bc", ""])
    w.add_meta("tokenizer.ggml.scores", [0.0, -1.5, 2.25])
    w.add_meta("tokenizer.ggml.token_type", [1, 2, 3])
    w.add_meta("big", 1 << 40)
    w.add_tensor("blk.0.attn_q.weight", a, gguf.Q4_K)
    w.add_tensor("output_norm.weight", b, gguf.F32)
    w.add_tensor("blk.0.ffn_down.weight", a, gguf.Q6_K)
    w.close()
    with gguf.GGUFReader(p) as r:
        assert r.version == 3 and r.alignment == 64
        assert r.meta["general.architecture"] == "llama"
        assert r.meta["llama.block_count"] == 2
        assert abs(r.meta["llama.rope.freq_base"] - 500000.0) < 1e-3
        assert r.meta["llama.flag"] is True
        assert r.meta["tokenizer.ggml.tokens"] == ["<s>", "a", "bc", ""]
        assert r.meta["tokenizer.ggml.scores"] == [0.0, -1.5, 2.25]
        assert r.meta["tokenizer.ggml.token_type"] == [1, 2, 3]
        assert r.meta["big"] == 1 << 40
        t = r.tensor("blk.0.attn_q.weight")
        assert t.shape == (6, 256) and t.ggml_type == gguf.Q4_K and t.nbytes == 6 * 144
        assert np.array_equal(t.data, gguf.quantize(a, gguf.Q4_K))
        assert np.array_equal(r.tensor("output_norm.weight").to_float(), b)
        assert np.abs(r.tensor("blk.0.ffn_down.weight").to_float() - a).max() < 0.1
    raw = open(p, "rb").read()
    assert raw[:4] == b"GGUF"


def test_gguf_rejects_garbage(tmp_path):
    p = str(tmp_path / "bad.gguf")
    open(p, "wb").write(b"NOPE" + b"\0" * 64)
    with pytest.raises(IOError):
        gguf.GGUFReader(p)
    open(p, "wb").write(b"GGUF" + struct.pack("<IQQ", 3, 1 << 40, 0))
    with pytest.raises(IOError):
        gguf.GGUFReader(p)


@pytest.mark.parametrize("name", ["q8_0", "q4_k", "q6_k", "mxfp4"])
def test_device_repack_keeps_the_format_numerics(name):
    """The aligned device planes decode to exactly what the GGUF blocks decode to."""
    import torch

    from loken_b200.ops import quant

    ty = quant.TYPE_OF_NAME[name]
    rng = np.random.default_rng(7)
    rows, K = 12, 1024
    x = (rng.standard_normal((rows, K)) * rng.uniform(0.05, 2.0, (rows, 1))).astype(np.float32)
    raw = gguf.quantize(x, ty)
    want = gguf.dequantize(raw, ty, (rows, K))
    q = quant.from_blocks(raw, ty, rows, K, torch.device("cpu"))
    got = quant.dequantize_weight(q).numpy()
    assert np.array_equal(got, want)


def test_torch_encoders_write_valid_device_planes():
    """The round-to-nearest encoders in torch (used on the GPU for large random-init models) produce
    the same plane shapes as the host encoders and decode to within the format's own error."""
    import torch

    from loken_b200.ops import quant

    torch.manual_seed(0)
    w = torch.randn(8, 512) * 0.02
    for fmt in ("q8_0", "mxfp4", "q4_k", "q6_k"):
        a, b = quant.quantize_weight_torch(w, fmt), quant.quantize_weight(w, fmt)
        assert a.codes.shape == b.codes.shape and a.scales.shape == b.scales.shape and a.aq_fmt == b.aq_fmt
        ea = (quant.dequantize_weight(a) - w).abs().max().item()
        eb = (quant.dequantize_weight(b) - w).abs().max().item()
        assert ea <= 1.25 * eb + 1e-6, (fmt, ea, eb)
