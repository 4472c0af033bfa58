"""Child of test_lockstep: gloo ranks on CPU, a scripted engine each; rank 0 drives through the
LLM facade, the others follow.  Mode "mirror": every rank must have seen the same requests, the
same between-step calls (embed, cache reset, layer_perf) and taken the same steps.  Mode "leave":
the last rank leaves between two steps; rank 0's next step raises RankLeft and the remaining
follower's receive runs out, after which it returns."""
import json
import os
import sys
import time

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from loken_b200.engine.llm import LLM, GenerationParams  # noqa: E402
from loken_b200.parallel.follower import LockstepEngine, RankLeft, control_group, follow  # noqa: E402
from loken_b200.parallel.watchdog import RankWatchdog  # noqa: E402
from loken_b200.text.tokenizer import ByteTokenizer  # noqa: E402
from tests.fakes import FakeEngine  # noqa: E402


class CountingEngine(FakeEngine):
    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.calls = []

    def embed(self, tokens, pooling="last"):
        self.calls.append(("embed", len(tokens)))
        return super().embed(tokens, pooling)

    def layer_perf(self, n_tokens=1):
        self.calls.append(("layer_perf", n_tokens))
        return super().layer_perf(n_tokens)

    def reset_prefix_cache(self):
        self.calls.append(("reset",))
        return super().reset_prefix_cache()


def mirror(out):
    rank = dist.get_rank()
    grp = control_group(timeout_s=30)
    eng = CountingEngine("lockstep reply")
    if rank == 0:
        ls = LockstepEngine(eng, grp, keepalive_s=0)
        llm = LLM(ls, ByteTokenizer(260), "m")
        a = llm.generate("first", GenerationParams(max_tokens=5))
        vec, n = llm.embed("embed me")
        llm.on_engine_thread(lambda e: e.reset_prefix_cache())
        llm.on_engine_thread(lambda e: e.layer_perf(2))
        b = llm.generate("second prompt", GenerationParams(max_tokens=50))
        refused = ""
        try:
            llm.on_engine_thread(lambda e: e.some_unmirrored_mutation())
        except AttributeError as e:
            refused = str(e)
        llm.close()
        ls.shutdown()
        rep = {"texts": [a.text, b.text], "steps": eng.stats.steps, "prompts": eng.prompts, "calls": eng.calls,
               "embed_n": n, "refused": refused}
    else:
        rc = follow(eng, grp)
        rep = {"steps": eng.stats.steps, "prompts": eng.prompts, "calls": eng.calls, "rc": rc}
    with open(f"{out}.{rank}", "w") as f:
        json.dump(rep, f)
    dist.barrier()


def leave(out):
    rank, world = dist.get_rank(), dist.get_world_size()
    grp = control_group(timeout_s=4)
    store = dist.distributed_c10d._get_default_store()
    wd = RankWatchdog(store, rank, world, interval_s=0.1, timeout_s=1.0).start()
    eng = CountingEngine("x" * 40)
    rep = {}
    if rank == 0:
        ls = LockstepEngine(eng, grp, wd, keepalive_s=1.0)
        ls.add_request([1, 2, 3])
        for _ in range(3):
            ls.step()
        store.set("go_leave", "1")            # the last rank leaves now, between two steps
        t0 = time.monotonic()
        err = ""
        while time.monotonic() - t0 < 10:
            try:
                ls.step()
            except RankLeft as e:
                err = str(e)
                break
            time.sleep(0.05)
        rep = {"err": err, "steps": eng.stats.steps}
    elif rank == world - 1:
        # follows for three steps, then leaves in an orderly way (nothing in flight)
        import threading

        def leaver():
            store.wait(["go_leave"])
            wd.leave()
            wd.stop()
            with open(f"{out}.{rank}", "w") as f:
                json.dump({"left": True}, f)
            os._exit(0)

        threading.Thread(target=leaver, daemon=True).start()
        follow(eng, grp, wd)
        rep = {"left": True}
    else:
        t0 = time.monotonic()
        rc = follow(eng, grp, wd)
        rep = {"rc": rc, "waited_s": round(time.monotonic() - t0, 2), "steps": eng.stats.steps}
    wd.stop()
    with open(f"{out}.{rank}", "w") as f:
        json.dump(rep, f)
    os._exit(0)      # the group lost a member: no collective teardown


def main():
    mode, out = sys.argv[1], sys.argv[2]
    dist.init_process_group("gloo")
    if mode == "mirror":
        mirror(out)
        dist.destroy_process_group()
    else:
        leave(out)


if __name__ == "__main__":
    main()
