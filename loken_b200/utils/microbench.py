"""The kernel micro-benchmark set: every single-kernel workload of `utils/prof_cases.py` at the shapes
of the benchmark models, one line per kernel with its time and the rate it implies.

    python -m loken_b200.utils.microbench                 # the whole set
    python -m loken_b200.utils.microbench --only gemm     # names containing "gemm"

Times are CUDA-graph replays bracketed by CUDA events (see `prof_cases._bracket`); buffers are rotated
or larger than the L2 so DRAM figures mean something.  The output of one run is the table to compare a
kernel change against.
"""
from __future__ import annotations

import argparse
import contextlib
import io
import json

SET = [
    # name, prof_cases arguments
    ("gemm_fp8 gate/up m64", ["gemm_fp8", "--m", "64"]),
    ("gemm_fp8 gate/up m16", ["gemm_fp8", "--m", "16"]),
    ("gemm_fp8 gate/up m1", ["gemm_fp8", "--m", "1"]),
    ("gemm_fp8 down m64", ["gemm_fp8", "--m", "64", "--n", "8192", "--k", "28672"]),
    ("gemm_fp8 qkv m64", ["gemm_fp8", "--m", "64", "--n", "10240", "--k", "8192"]),
    ("gemm_fp8 o m64", ["gemm_fp8", "--m", "64", "--n", "8192", "--k", "8192"]),
    ("gemm_fp8 prefill m4096", ["gemm_fp8", "--m", "4096", "--n", "8192", "--k", "8192"]),
    ("gemm_bf16 gate/up m64", ["gemm_bf16", "--m", "64"]),
    ("gemm_q8_0 gate/up m64", ["gemm_q8_0", "--m", "64"]),
    ("gemm_q6_k gate/up m64", ["gemm_q6_k", "--m", "64"]),
    ("gemm_q4_k gate/up m64", ["gemm_q4_k", "--m", "64"]),
    ("gemm_mxfp4 gate/up m64", ["gemm_mxfp4", "--m", "64"]),
    ("attn_decode b64 ctx1056", ["attn_decode", "--batch", "64", "--ctx", "1056"]),
    ("attn_decode b64 ctx8192", ["attn_decode", "--batch", "64", "--ctx", "8192"]),
    ("attn_decode b1 ctx8192", ["attn_decode", "--batch", "1", "--ctx", "8192"]),
    ("attn_prefill 8x2048", ["attn_prefill", "--seqs", "8", "--ctx", "2048"]),
    ("add_rmsnorm t64", ["add_rmsnorm", "--batch", "64"]),
    ("glu t64", ["glu", "--batch", "64"]),
    ("rope_kv t64", ["rope_kv", "--batch", "64"]),
    ("embed t64", ["embed", "--batch", "64"]),
    ("sampler b64", ["sampler", "--batch", "64"]),
    ("moe layer t128 mxfp4", ["moe", "--batch", "128", "--fmt", "mxfp4", "--experts", "128"]),
    ("moe layer t16 mxfp4", ["moe", "--batch", "16", "--fmt", "mxfp4", "--experts", "128"]),
]


def run_set(only: str = "") -> list:
    from . import prof_cases

    rows = []
    for name, argv in SET:
        if only and only not in name:
            continue
        buf = io.StringIO()
        try:
            with contextlib.redirect_stdout(buf):
                prof_cases.main(argv)
            rows.append({"kernel": name, "result": buf.getvalue().strip().splitlines()[-1] if buf.getvalue().strip() else ""})
        except Exception as e:          # one failing case does not hide the others
            rows.append({"kernel": name, "error": f"{type(e).__name__}: {e}"})
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="", help="run the cases whose name contains this")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    rows = run_set(a.only)
    if a.json:
        print(json.dumps(rows))
        return
    for r in rows:
        print(f"{r['kernel']:28s} {r.get('result') or r.get('error')}")


if __name__ == "__main__":
    main()
