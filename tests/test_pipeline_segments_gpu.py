"""A model cut into two segments joined by TCP frames reproduces the whole model: prefill, decode,
a re-sent position (speculative reject), and the cache bookkeeping of a tail."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _models():
    from loken_b200.models.config import tiny
    from loken_b200.models.weights import random_weights

    dev = torch.device("cuda")
    cfg = tiny("llama", head_dim=64, n_q=4, n_kv=2, n_layers=4)
    full = random_weights(cfg, dev, seed=7, std=0.05)
    head = random_weights(cfg, dev, seed=7, std=0.05, layer_range=(0, 2))
    tail = random_weights(cfg, dev, seed=7, std=0.05, layer_range=(2, 4))
    return cfg, full, head, tail, dev


def test_two_segments_over_tcp_match_the_whole_model():
    from loken_b200.cluster.pipeline import SegmentError, SegmentLink, SegmentServer
    from loken_b200.cluster.segment import PipelineHead, SegmentRunner
    from loken_b200.models.reference import forward_ref

    cfg, full, head_w, tail_w, dev = _models()
    tail = SegmentRunner(cfg, tail_w, 2, 4, last=True, device=dev, max_ctx=256, max_requests=4)
    srv = SegmentServer(tail.run, cut=tail.cut).start()
    try:
        link = SegmentLink(srv.addr[0], srv.addr[1])
        head = PipelineHead(cfg, head_w, 2, link, device=dev, max_ctx=256, max_requests=4)
        g = torch.Generator().manual_seed(3)
        prompt = torch.randint(0, cfg.vocab, (37,), generator=g).tolist()
        ref = forward_ref(full, prompt)
        got = torch.from_numpy(head.forward(5, prompt, 0)).reshape(-1)
        cos = torch.nn.functional.cosine_similarity(got, ref[-1].float().cpu(), dim=0).item()
        assert cos > 0.998, cos
        # decode three tokens greedily and compare each step with the whole model's logits
        toks = list(prompt)
        for _ in range(3):
            toks.append(int(got.argmax()))
            got = torch.from_numpy(head.forward(5, toks[-1:], len(toks) - 1)).reshape(-1)
            ref = forward_ref(full, toks)
            assert torch.nn.functional.cosine_similarity(got, ref[-1].float().cpu(), dim=0).item() > 0.998
        # a rejected draft: the head re-sends from an earlier position and both caches trim back
        again = torch.from_numpy(head.forward(5, toks[-2:], len(toks) - 2)).reshape(-1)
        assert torch.allclose(again, got, atol=2e-2, rtol=0)
        assert tail.status()["requests"] == 1 and head.seg.alloc.length(head.seg.reqs[5].seq_id) == len(toks)
        # a second request is independent; rows that skip positions are refused with the reason
        assert len(head.generate(6, prompt[:9], 4)) == 4 and 6 not in tail.reqs
        with pytest.raises(SegmentError, match="unknown here"):
            link.boundary(99, np.zeros((1, cfg.hidden), np.float32), 7)
        with pytest.raises(SegmentError, match="width"):
            link.boundary(5, np.zeros((1, 3), np.float32), 0)
        head.release(5)
        assert tail.status()["requests"] == 0
        assert tail.runner.wsp.read_status() == 0
    finally:
        srv.stop()
