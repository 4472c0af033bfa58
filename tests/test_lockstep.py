"""Tensor-parallel serving hand-shake on CPU (gloo processes): followers see every request and
every between-step call rank 0 makes and take exactly the same engine steps; a rank that leaves
between steps is noticed on the host by the others."""
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode, out, nproc, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "mp_lockstep_worker.py"),
           mode, out]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=300)


def test_followers_mirror_rank0(tmp_path):
    out = str(tmp_path / "rep")
    r = _run("mirror", out, 2, 29655)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    r0, r1 = json.load(open(out + ".0")), json.load(open(out + ".1"))
    assert r0["texts"] == ["locks", "lockstep reply"]
    assert r0["prompts"] == r1["prompts"] and len(r0["prompts"]) == 2
    assert r0["steps"] == r1["steps"] > 0
    # embeddings, the cache reset and the layer timing ran on every rank, in the same order
    assert r0["calls"] == r1["calls"] == [["embed", r0["embed_n"]], ["reset"], ["layer_perf", 2]]
    assert "not available under tensor parallelism" in r0["refused"]
    assert r1["rc"] == 0


def test_a_rank_that_leaves_between_steps_is_noticed_by_the_others(tmp_path):
    out = str(tmp_path / "rep")
    r = _run("leave", out, 3, 29657)
    reps = [json.load(open(f"{out}.{i}")) for i in range(3)]
    assert "rank(s) [2] left" in reps[0]["err"], (reps, r.stderr[-1500:])
    assert reps[0]["steps"] >= 3
    assert reps[1]["rc"] == 3 and reps[1]["waited_s"] < 30      # its receive ran out: it returned, did not hang
    assert reps[2] == {"left": True}
