"""Error-compensated quantisation: the bytes are the format's own, and the outputs over calibration-like
rows are closer than those of plain round-to-block quantisation."""
import numpy as np
import pytest

from loken_b200.formats import gguf as G
from loken_b200.formats.compensate import output_error, quantize_compensated


def _case(seed, N=96, K=1024, n=48, rank=12):
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    # activations live near a low-dimensional subspace plus a few loud channels, as a model's do
    basis = rng.standard_normal((rank, K)).astype(np.float32)
    X = rng.standard_normal((n, rank)).astype(np.float32) @ basis + 0.1 * rng.standard_normal((n, K)).astype(np.float32)
    X[:, rng.integers(0, K, 8)] *= 6.0
    Xtest = rng.standard_normal((n, rank)).astype(np.float32) @ basis + 0.1 * rng.standard_normal((n, K)).astype(np.float32)
    Xtest[:, :] *= 1.0
    return W, X, Xtest


@pytest.mark.parametrize("ty", [G.Q4_K, G.Q6_K, G.Q8_0])
def test_outputs_are_closer_and_bytes_are_the_formats_own(ty):
    W, X, Xtest = _case(ty)
    raw, dec = quantize_compensated(W, X, ty)
    bv, bb = G.block_info(ty)
    assert raw.dtype == np.uint8 and raw.size == W.size // bv * bb
    assert np.array_equal(G.dequantize(raw, ty, W.shape), dec)              # row-major blocks, decodable as any tensor
    plain = G.dequantize(G.quantize(W, ty), ty, W.shape)
    e_plain, e_comp = output_error(W, plain, X), output_error(W, dec, X)
    assert e_comp < 0.7 * e_plain, (e_plain, e_comp)                         # on the rows it was fitted to
    held = output_error(W, dec, Xtest), output_error(W, plain, Xtest)
    assert held[0] < held[1]                                                 # and on rows from the same source it never saw
    # weights themselves move further from the originals: the error went where activations do not look
    assert np.abs(dec - W).mean() >= np.abs(plain - W).mean() * 0.9


def test_refusals_and_dead_columns():
    W, X, _ = _case(1, N=8, K=512)
    with pytest.raises(ValueError):
        quantize_compensated(W[:, :500], X[:, :500], G.Q4_K)
    with pytest.raises(ValueError):
        quantize_compensated(W, X[:, :256], G.Q4_K)
    X[:, 100:140] = 0.0                                                      # channels no calibration row excites
    raw, dec = quantize_compensated(W, X, G.Q4_K)
    assert np.isfinite(dec).all()
