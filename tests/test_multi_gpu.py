"""Multi-GPU tests: each starts one child process per GPU with torch.distributed.run on
127.0.0.1 and reads the JSON report the ranks leave.  Skipped with fewer than two GPUs."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run(worker: str, nproc: int, out: str, port: int, extra=(), timeout=300):
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, worker), out, *extra]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.load(open(out))


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
def test_peer_memory_allreduce(tmp_path):
    n = min(_ngpu(), 8)
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    rep = _run("mp_collectives_worker.py", n, str(tmp_path / "ar.json"), 29631)
    print(json.dumps(rep))          # the timing table, for `pytest -s`
    assert rep["ok"], rep
    assert rep["timeout_reported"] is True
    assert rep["recovers_after_timeout"] is True


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("fmt", ["bf16", "fp8_block"])
def test_tensor_parallel_matches_single_gpu(tmp_path, fmt):
    n = min(_ngpu(), 8)
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    rep = _run("mp_tp_worker.py", n, str(tmp_path / "tp.json"), 29641, (fmt,))
    print(json.dumps(rep))
    # every way of summing the row-parallel layers reproduces the degree-1 ENGINE (same kernels, same
    # numerics): bf16 weights to cosine >= 0.9995 with the same greedy tokens (one more bf16 rounding per
    # partial sum), block-scaled fp8 to the format's own noise (cosine >= 0.99)
    bound = 0.9995 if fmt == "bf16" else 0.99
    for name in ("nccl", "push", "fused", "sum_norm"):
        assert rep[f"match_{name}"], (name, rep)
        assert rep[f"logits_cos_min_{name}"] >= bound, (name, rep)
        assert rep[f"status_{name}"] == 0, (name, rep)
        assert rep[f"cos_vs_nccl_{name}"] >= bound, (name, rep)
    if rep["world"] == 2:      # a sum of two has one order: the same rounding places as NCCL
        assert rep["cos_vs_nccl_push"] >= 0.99999 and rep["cos_vs_nccl_fused"] >= 0.99999
    assert rep["sharded_steps_sum_norm"] > 0 and rep["sharded_steps_push"] == 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("fmt", ["bf16", "mxfp4"])
def test_expert_parallel_matches_single_gpu(tmp_path, fmt):
    """EP = N reproduces EP = 1, with the mixture layers run replicated + all-reduce and with the
    all-to-all dispatch / combine over peer memory on a token-sharded residual stream."""
    n = min(_ngpu(), 8)
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    rep = _run("mp_ep_worker.py", n, str(tmp_path / "ep.json"), 29661, (fmt,))
    print(json.dumps(rep))
    bound = 0.9995 if fmt == "bf16" else 0.99      # at nine positions in ten; the worker bounds the worst one
    for name in ("replicated", "dispatch"):
        assert rep[f"match_{name}"], (name, rep)
        assert rep[f"logits_cos_p10_{name}"] >= bound, (name, rep)
        assert rep[f"status_{name}"] == 0, (name, rep)
    assert rep["sharded_steps_dispatch"] > 0 and rep["sharded_steps_replicated"] == 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
def test_pipeline_parallel_matches_single_gpu(tmp_path):
    rep = _run("mp_pp_worker.py", 2, str(tmp_path / "pp.json"), 29651)
    assert rep["tokens_match_oracle"] and rep["ranks_agree"], rep
    assert rep["ranges"] == [[0, 2], [2, 4]] and rep["held_layers"] == [2]
    assert rep["status"] == 0
