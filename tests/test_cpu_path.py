"""The C++ CPU decode path: SIMD dots against the scalar definition, the pooled GEMV, and a whole
tiny model against the fp32 PyTorch oracle of the same file."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from loken_b200.cpu.engine import CpuModel, _lib
from loken_b200.formats import gguf as G


def test_q8_dot_levels_agree_with_scalar():
    rng = np.random.default_rng(0)
    L = _lib()
    have = L.lkc_cpu_level()
    for n in (32, 256, 4096):
        a = G.quantize(rng.standard_normal(n).astype(np.float32), G.Q8_0)
        b = G.quantize((rng.standard_normal(n) * 3).astype(np.float32), G.Q8_0)
        want = L.lkcpu_dot_q8_0(a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), n // 32, 0)
        fa = G.dequantize(a, G.Q8_0, (n,))
        fb = G.dequantize(b, G.Q8_0, (n,))
        assert abs(want - float(fa.astype(np.float64) @ fb.astype(np.float64))) < 1e-3 * max(1.0, abs(want))
        for level in (2, 4):
            if level <= have:
                got = L.lkcpu_dot_q8_0(a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), n // 32, level)
                assert abs(got - want) <= 2e-5 * max(1.0, abs(want)), (n, level)


@pytest.mark.parametrize("threads", [1, 4])
def test_pooled_gemv_matches_float(threads):
    rng = np.random.default_rng(1)
    N, K = 515, 768
    w = rng.standard_normal((N, K)).astype(np.float32) * 0.1
    x = rng.standard_normal(K).astype(np.float32)
    wq = G.quantize(w, G.Q8_0)
    out = np.zeros(N, dtype=np.float32)
    for _ in range(20):       # many short tasks exercise the pool's hand-off
        rc = _lib().lkcpu_gemv_q8_0(wq.ctypes.data_as(C.c_void_p), x.ctypes.data_as(C.c_void_p),
                                    out.ctypes.data_as(C.c_void_p), N, K, threads, 4)
        assert rc == 0
    ref = G.dequantize(wq, G.Q8_0, (N, K)) @ x
    assert np.abs(out - ref).max() < 0.02 * np.abs(ref).max()


@pytest.mark.parametrize("ty", [G.Q4_K, G.Q6_K])
def test_k_quant_rows_take_integer_dots(ty):
    """Q4_K and Q6_K rows against the Q8_0-quantised activation: the scalar definition equals the float product
    of the decoded weights with the decoded activation, and the AVX2 version equals the scalar one."""
    rng = np.random.default_rng(2)
    L = _lib()
    have = L.lkc_cpu_level()
    N, K = 67, 1024
    w = rng.standard_normal((N, K)).astype(np.float32) * 0.1
    x = (rng.standard_normal(K) * 2).astype(np.float32)
    wq = G.quantize(w, ty)
    xq = G.dequantize(G.quantize(x, G.Q8_0), G.Q8_0, (K,))               # what the integer dot multiplies by
    ref = G.dequantize(wq, ty, (N, K)).astype(np.float64) @ xq.astype(np.float64)
    outs = {}
    for level in (0, 2):
        if level > have:
            continue
        out = np.zeros(N, dtype=np.float32)
        rc = L.lkcpu_gemv_any(int(ty), wq.ctypes.data_as(C.c_void_p), x.ctypes.data_as(C.c_void_p),
                              out.ctypes.data_as(C.c_void_p), N, K, 3, level)
        assert rc == 0
        outs[level] = out
        assert np.abs(out - ref).max() < 1e-4 * max(1.0, np.abs(ref).max()), (level, np.abs(out - ref).max())
    if 2 in outs:
        assert np.abs(outs[2] - outs[0]).max() <= 2e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("arch,fmt", [("qwen3", "q8_0"), ("llama", "q8_0"), ("llama", "q4_k_m")])
def test_cpu_model_matches_oracle(tmp_path, arch, fmt):
    from loken_b200.models import loader
    from loken_b200.models.config import tiny
    from loken_b200.models.reference import forward_ref

    cfg = tiny(arch, weight_format=fmt, head_dim=64, n_q=4, n_kv=2, hidden=256, intermediate=512, vocab=512)
    path = os.path.join(tmp_path, "m.gguf")
    loader.export_random_gguf(path, cfg, seed=3, std=0.05)
    m = CpuModel.from_gguf(path, threads=2)
    assert m.simd_level >= 0 and m.threads == 2
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (23,), generator=g).tolist()
    got = torch.from_numpy(m.prefill(prompt).copy())
    w, _ = loader.load_gguf(path, torch.device("cpu"))
    ref = forward_ref(w, prompt)[-1]
    cos = torch.nn.functional.cosine_similarity(got, ref.float(), dim=0).item()
    assert cos > 0.998, cos
    # greedy generation is reproducible and position bookkeeping survives a reset
    a = m.generate(prompt, max_tokens=6)["tokens"]
    b = m.generate(prompt, max_tokens=6)["tokens"]
    assert a == b and len(a) == 6
    # a scalar-only run gives the same tokens
    m0 = CpuModel.from_gguf(path, threads=1, max_level=0)
    assert m0.generate(prompt, max_tokens=6)["tokens"] == a
    m.close()
    m0.close()
