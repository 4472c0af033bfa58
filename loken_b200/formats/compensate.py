"""Quantise a matrix so that what one block of columns loses, the columns after it absorb.

A projection is judged by what it does to activations: the quantity to keep small is the error of W x over
the rows x the model really produces, not the error of W.  Given calibration rows X [n, K], the output error
of a quantised matrix Q is tr((W - Q) H (W - Q)^T) with H = X^T X / n.  Columns are quantised a block at a
time in their stored order; the error a block leaves is pushed into the columns that have not been
quantised yet by the least-squares correction, so they cancel as much of it as the calibration rows allow
(the family of methods that quantise some columns and repair the rest; reference:
`src/inference/load/compensate.rs:1-16`).

The block quantiser is not touched: each block is encoded by the format's own rule (`formats/gguf.py:
quantize`), this module only decides which values the rule is handed.  The output is the format's bytes.

Numerics: H gets a ridge of `damp` times its mean diagonal (calibration rows are fewer than columns, so H
is singular without it); the correction uses the upper Cholesky factor U of H^-1, block by block:

    E = (W_b - Q_b) U_bb^-1          W_rest -= E U_b,rest

in float64 on the host.  With the span equal to the format's block (256 for the K formats) one solve per
block suffices.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from . import gguf as G


def _factor(X: np.ndarray, damp: float) -> torch.Tensor:
    """Upper Cholesky factor of (X^T X / n + ridge)^-1, float64."""
    x = torch.from_numpy(np.ascontiguousarray(X, dtype=np.float64))
    H = x.T @ x / max(1, x.shape[0])
    d = torch.diagonal(H)
    dead = d <= 0
    H[dead, dead] = 1.0                               # a column no row excites: its weights cost nothing either way
    H += torch.eye(H.shape[0], dtype=torch.float64) * (damp * float(d.mean()) + 1e-12)
    L = torch.linalg.cholesky(H)
    Hinv = torch.cholesky_inverse(L)
    return torch.linalg.cholesky(Hinv, upper=True)


def output_error(W: np.ndarray, Q: np.ndarray, X: np.ndarray) -> float:
    """Mean squared error of the outputs over the calibration rows, relative to the outputs' mean square."""
    y = X.astype(np.float64) @ W.astype(np.float64).T
    e = X.astype(np.float64) @ (W.astype(np.float64) - Q.astype(np.float64)).T
    return float((e * e).mean() / max((y * y).mean(), 1e-30))


def quantize_compensated(W: np.ndarray, X: np.ndarray, ggml_type: int, *, damp: float = 0.01, span: Optional[int] = None,
                         threads: int = 8) -> Tuple[np.ndarray, np.ndarray]:
    """W [N, K] float, X [n, K] calibration rows of the projection's input -> (raw block bytes of the format for
    W in row-major order, the decoded matrix the bytes stand for)."""
    W = np.ascontiguousarray(W, dtype=np.float32)
    N, K = W.shape
    bv, bb = G.block_info(ggml_type)
    span = span or bv
    if K % bv or span % bv or X.shape[1] != K:
        raise ValueError("rows must be whole blocks of the format and match the calibration rows' width")
    U = _factor(X, damp)
    work = torch.from_numpy(W.astype(np.float64))
    decoded = np.empty((N, K), dtype=np.float32)
    raws = []
    for b0 in range(0, K, span):
        b1 = min(K, b0 + span)
        cur = work[:, b0:b1].to(torch.float32).numpy()
        raw = G.quantize(cur, ggml_type, threads=threads)
        q = G.dequantize(raw, ggml_type, cur.shape, threads=threads)
        decoded[:, b0:b1] = q
        raws.append(raw.reshape(N, (b1 - b0) // bv * bb))
        if b1 < K:
            err = work[:, b0:b1] - torch.from_numpy(q.astype(np.float64))
            # E = err U_bb^-1 (U_bb upper triangular), then the unquantised columns take E U_b,rest
            E = torch.linalg.solve_triangular(U[b0:b1, b0:b1], err, upper=True, left=False)
            work[:, b1:] -= E @ U[b0:b1, b1:]
    return np.ascontiguousarray(np.concatenate(raws, axis=1)).reshape(-1), decoded
