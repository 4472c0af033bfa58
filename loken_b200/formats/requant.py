"""Requantise a model file: read every tensor of a GGUF, decode it, encode it in the target format.

    requantize_gguf("llama-bf16.gguf", "llama-q4_k_m.gguf", "q4_k_m")

Which tensor gets which block type follows the roles llama.cpp's mixes use and `models/weights.py:
linear_format` reads back: in Q4_K_M the value projections and the down projections are Q6_K and the
rest Q4_K; embeddings and the output head keep one step more (Q6_K under a 4-bit mix, Q8_0 under Q8_0);
MXFP4 covers the experts only, attention stays bf16; norms, biases, sinks and router matrices are never
quantised.  A row length that is not a multiple of the block size falls back to the next type that
fits, then to bf16.

A calibration record (`calibrate()`: per-tensor sensitivity measured on text) lifts the most
sensitive tensors one step (Q4_K -> Q6_K -> Q8_0): the reference's convert takes a calibration the
same way (`docs/API.md:528-529`, `src/convert/`).  When the record also carries activation rows
(`<record>.rows.npz`, kept by `calibrate(keep_rows=...)`), the matrices those rows feed are encoded with
error compensation (`formats/compensate.py`): the format's own bytes, chosen so that the outputs over such
rows stay close.  The decode -> encode path runs in the C++ codecs
(`csrc/host/formats.cpp`), one tensor in memory at a time.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterable, Optional

import numpy as np

from . import gguf as G

FORMATS = ("q8_0", "q4_k_m", "q4_k", "q6_k", "mxfp4", "bf16", "f16")
_STEP_UP = {G.Q4_K: G.Q6_K, G.Q6_K: G.Q8_0, G.MXFP4: G.Q8_0}
_FILE_TYPE = {"f16": 1, "q8_0": 7, "q4_k": 14, "q4_k_m": 15, "q6_k": 18, "bf16": 32, "mxfp4": 38}


def role_of(name: str) -> str:
    """embed | head | v | down | expert | expert_down | router | linear | keep."""
    base = name.rsplit(".", 1)[0] if name.endswith((".weight", ".bias")) else name
    if not name.endswith(".weight"):
        return "keep"
    leaf = base.split(".")[-1]
    if leaf == "token_embd":
        return "embed"
    if leaf == "output":
        return "head"
    if leaf.endswith("_norm") or leaf in ("output_norm", "attn_sinks", "rope_freqs"):
        return "keep"
    if leaf == "ffn_gate_inp":
        return "router"
    if leaf.endswith("_exps"):
        return "expert_down" if "down" in leaf else "expert"
    if leaf == "attn_v":
        return "v"
    if leaf == "ffn_down":
        return "down"
    if leaf.startswith(("attn_", "ffn_")):
        return "linear"
    return "keep"


def target_type(role: str, fmt: str) -> Optional[int]:
    """ggml type of a tensor with this role under `fmt`; None = copy the tensor as it is stored."""
    if role in ("keep", "router"):
        return None
    if fmt in ("bf16", "f16"):
        return G.BF16 if fmt == "bf16" else G.F16
    if fmt == "mxfp4":
        return G.MXFP4 if role in ("expert", "expert_down") else G.BF16
    if fmt == "q8_0":
        return G.Q8_0
    if fmt == "q6_k":
        return G.Q6_K
    if fmt == "q4_k":
        return G.Q6_K if role in ("embed", "head") else G.Q4_K
    if fmt == "q4_k_m":
        return G.Q6_K if role in ("embed", "head", "v", "down", "expert_down") else G.Q4_K
    raise ValueError(f"unknown target format {fmt} (known: {', '.join(FORMATS)})")


def _fit(t: int, K: int) -> int:
    """The type itself when K is a multiple of its block, else the next one that fits."""
    for cand in (t, G.Q8_0, G.BF16):
        if cand in (G.F32, G.F16, G.BF16):
            return cand
        bv, _ = G.block_info(cand)
        if K % bv == 0:
            return cand
    return G.BF16


def plan(tensors: Iterable, fmt: str, sensitive: Optional[Dict[str, float]] = None, lift_fraction: float = 0.1):
    """name -> (target ggml type or None).  With a calibration record, the `lift_fraction` most sensitive
    quantised tensors go one step up."""
    out: Dict[str, Optional[int]] = {}
    infos = list(tensors)
    for ti in infos:
        role = role_of(ti.name)
        t = target_type(role, fmt) if len(ti.shape) >= 2 else None
        out[ti.name] = None if t is None else _fit(t, int(ti.shape[-1]))
    if sensitive:
        cand = sorted((n for n, t in out.items() if t in _STEP_UP and n in sensitive), key=lambda n: -sensitive[n])
        for n in cand[:max(1, int(len(cand) * lift_fraction))] if cand else []:
            K = next(int(ti.shape[-1]) for ti in infos if ti.name == n)
            out[n] = _fit(_STEP_UP[out[n]], K)
    return out


def requantize_gguf(src: str, dst: str, fmt: str, *, calibration: Optional[str] = None, threads: int = 8,
                    progress: Optional[Callable[[str, int, int], None]] = None) -> dict:
    """Writes `dst` with every matrix of `src` re-encoded for `fmt`; returns a summary.  The write goes to
    `dst + ".partial"` and is renamed when complete, so an interrupted conversion never leaves a file that
    looks whole."""
    if fmt not in FORMATS:
        raise ValueError(f"unknown target format {fmt} (known: {', '.join(FORMATS)})")
    sens = None
    rows = None
    if calibration:
        with open(calibration) as f:
            sens = json.load(f).get("sensitivity", {})
        if os.path.exists(calibration + ".rows.npz"):
            rows = np.load(calibration + ".rows.npz")
    compensated = 0
    r = G.GGUFReader(src)
    tmp = dst + ".partial"
    try:
        w = G.GGUFWriter(tmp)
        for k, v in r.meta.items():
            if k == "general.file_type":
                continue
            if isinstance(v, list) and not v:
                continue
            w.add_meta(k, v)
        if fmt in _FILE_TYPE:
            w.add_meta("general.file_type", _FILE_TYPE[fmt])
        w.add_meta("general.quantized_by", "loken")
        targets = plan(r.tensors.values(), fmt, sens)
        counts: Dict[str, int] = {}
        bytes_in = bytes_out = 0
        names = list(r.tensors)
        for i, name in enumerate(names):
            ti = r.tensors[name]
            t = targets[name]
            bytes_in += ti.nbytes
            shape_only = np.broadcast_to(np.zeros(1, np.float32), ti.shape)      # add_tensor reads the shape only
            if t is None or t == ti.ggml_type:
                w.add_tensor(name, shape_only, ti.ggml_type, raw=ti.data)
                out_t = ti.ggml_type
                bytes_out += ti.nbytes
            else:
                x = G.dequantize(ti.data, ti.ggml_type, ti.shape, threads=threads)
                if (rows is not None and name in rows.files and len(ti.shape) == 2 and t not in (G.F32, G.F16, G.BF16)
                        and rows[name].shape[1] == ti.shape[-1]):
                    from .compensate import quantize_compensated

                    raw, _ = quantize_compensated(x, rows[name].astype(np.float32), t, threads=threads)
                    compensated += 1
                else:
                    raw = G.quantize(x, t, threads=threads)
                w.add_tensor(name, shape_only, t, raw=raw)
                out_t = t
                bytes_out += raw.nbytes
                del x
            tn = G.TYPE_NAMES.get(out_t, str(out_t))
            counts[tn] = counts.get(tn, 0) + 1
            if progress is not None:
                progress(name, i + 1, len(names))
        w.close()
        os.replace(tmp, dst)
    finally:
        r.close()
        if os.path.exists(tmp):
            os.remove(tmp)
    return {"source": src, "output": dst, "format": fmt, "tensors": len(names), "types": counts,
            "bytes_in": bytes_in, "bytes_out": bytes_out, "calibrated": bool(sens), "compensated": compensated}


def sensitivity_from_activations(stats: Dict[str, Dict[str, float]]) -> Dict[str, float]:
    """Turns what `calibrate()` recorded (per tensor: mean square of the input activations, mean square
    of the weights, rows) into one number per tensor: the expected squared output error a unit of relative
    weight noise causes, normalised by the output's own size.  Larger = more sensitive."""
    out = {}
    for name, s in stats.items():
        out[name] = float(s.get("act_ms", 1.0)) * float(s.get("w_ms", 1.0)) * float(s.get("k", 1.0))
    tot = sum(out.values()) or 1.0
    return {k: v / tot for k, v in out.items()}


def write_calibration(path: str, name: str, model: str, stats: Dict[str, Dict[str, float]], texts: int, tokens: int,
                      rows: Optional[Dict[str, np.ndarray]] = None):
    """`rows`: tensor name -> activation rows [n, K] (float16) kept for error compensation; stored beside the
    record as `<path>.rows.npz`."""
    rec = {"name": name, "model": model, "texts": texts, "tokens": tokens, "stats": stats,
           "sensitivity": sensitivity_from_activations(stats), "rows": bool(rows)}
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    if rows:
        tmpz = path + ".rows.partial.npz"
        np.savez_compressed(tmpz, **{k: np.asarray(v, dtype=np.float16) for k, v in rows.items()})
        os.replace(tmpz, path + ".rows.npz")
    tmp = path + ".partial"
    with open(tmp, "w") as f:
        json.dump(rec, f)
    os.replace(tmp, path)
    return rec


# which stored tensors read the rows a probe role sees
_ROLE_TENSORS = {"qkv": ("attn_q", "attn_k", "attn_v", "attn_qkv"), "o": ("attn_output",),
                 "gate_up": ("ffn_gate", "ffn_up", "ffn_gate_exps", "ffn_up_exps"), "down": ("ffn_down",)}


def calibrate(weights, token_lists, *, max_tokens: int = 4096, keep_rows: int = 0, rows_out: Optional[dict] = None
              ) -> Dict[str, Dict[str, float]]:
    """Runs the fp32 forward of `weights` (a loaded model, one rank) over the given token lists and records,
    per stored tensor, the mean square of the activations it multiplies, the mean square of its own
    values and its row length: what `sensitivity_from_activations` turns into a ranking.  Returns the
    stats keyed by GGUF tensor name.  With `keep_rows` > 0, up to that many activation rows per tensor
    (evenly spaced over the text) are put into `rows_out` under the same names, for error compensation."""
    import torch

    from ..models.reference import dequant_linear, forward_ref

    acc: Dict[tuple, list] = {}

    kept: Dict[tuple, list] = {}

    def probe(il, role, x):
        s = acc.setdefault((il, role), [0.0, 0])
        s[0] += float(x.float().pow(2).sum())
        s[1] += x.numel()
        if keep_rows > 0:
            have = kept.setdefault((il, role), [])
            room = keep_rows - sum(r.shape[0] for r in have)
            if room > 0:
                xr = x.float().reshape(-1, x.shape[-1])
                step = max(1, xr.shape[0] // room)
                have.append(xr[::step][:room].to(torch.float16).cpu().numpy())

    seen = 0
    with torch.no_grad():
        for toks in token_lists:
            toks = list(toks)[:max(1, max_tokens - seen)]
            if len(toks) < 2:
                continue
            forward_ref(weights, toks, probe=probe)
            seen += len(toks)
            if seen >= max_tokens:
                break
    stats: Dict[str, Dict[str, float]] = {}
    for (il, role), (ss, n) in acc.items():
        lw = weights.layers[il]
        lin = {"qkv": lw.wqkv, "o": lw.wo, "gate_up": getattr(lw, "w_gate_up", None), "down": getattr(lw, "w_down", None)}[role]
        w_ms, k = 1.0, 1.0
        if lin is not None:
            wf = dequant_linear(lin).float()
            w_ms, k = float(wf.pow(2).mean()), float(wf.shape[1])
        for leaf in _ROLE_TENSORS[role]:
            stats[f"blk.{il}.{leaf}.weight"] = {"act_ms": ss / max(n, 1), "w_ms": w_ms, "k": k}
            if rows_out is not None and kept.get((il, role)):
                rows_out[f"blk.{il}.{leaf}.weight"] = np.concatenate(kept[(il, role)], 0)
    return stats
