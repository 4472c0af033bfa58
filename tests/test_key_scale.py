"""Key lane scale folded into the Q / K norm weights: scores unchanged, int8 key blocks tighter."""
import torch

from loken_b200.models.key_scale import apply_key_scale, lane_scale, rotation_partner


def test_rotation_partner():
    assert rotation_partner(0, 8, True) == 1 and rotation_partner(5, 8, True) == 4
    assert rotation_partner(1, 8, False) == 5 and rotation_partner(6, 8, False) == 2
    assert rotation_partner(9, 8, False) is None        # a lane the rotation leaves alone


def test_scale_is_equal_on_a_rotation_pair():
    w = torch.tensor([1.0, -4.0, 0.5, 2.0, 3.0, 0.25, 1.0, 1.0])
    s = lane_scale(w, 8, adjacent=False)                 # pairs (0,4) (1,5) (2,6) (3,7)
    assert torch.equal(s, torch.tensor([3.0, 4.0, 1.0, 2.0, 3.0, 4.0, 1.0, 2.0]))
    s = lane_scale(w, 8, adjacent=True)                  # pairs (0,1) (2,3) (4,5) (6,7)
    assert torch.equal(s, torch.tensor([4.0, 4.0, 2.0, 2.0, 3.0, 3.0, 1.0, 1.0]))


def _rope(x, pos, theta=10000.0):
    hd = x.shape[-1]
    half = hd // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) / half)
    ang = pos[:, None].double() * inv[None]
    c, s = ang.cos(), ang.sin()
    a, b = x[..., :half].double(), x[..., half:].double()
    return torch.cat([a * c - b * s, a * s + b * c], -1)


def _q8_err(k):
    blocks = k.reshape(-1, 32)
    step = blocks.abs().amax(-1, keepdim=True) / 127.0
    deq = (blocks / step).round().clamp(-127, 127) * step
    return ((deq - blocks).pow(2).sum() / blocks.pow(2).sum()).sqrt().item()


def test_scores_are_unchanged_and_int8_keys_get_tighter():
    from loken_b200.models.config import tiny
    from loken_b200.models.weights import random_weights

    torch.manual_seed(0)
    cfg = tiny("qwen3", head_dim=64, n_q=4, n_kv=2, n_layers=2)
    w = random_weights(cfg, torch.device("cpu"), seed=3)
    for lw in w.layers:                                  # a few lanes with large K norm weights, as real checkpoints have
        lw.k_norm = lw.k_norm.clone()
        lw.k_norm[[3, 17, 40]] = torch.tensor([9.0, 14.0, 6.0])
    q_norm0, k_norm0 = w.layers[0].q_norm.clone(), w.layers[0].k_norm.clone()
    T, hd = 24, cfg.head_dim
    q = torch.randn(T, hd).double()
    k = torch.randn(T, hd).double()
    q = q / q.pow(2).mean(-1, keepdim=True).sqrt()
    k = k / k.pow(2).mean(-1, keepdim=True).sqrt()
    pos = torch.arange(T)
    before_k = _rope(k * k_norm0.double(), pos)
    scores0 = _rope(q * q_norm0.double(), pos) @ before_k.t()
    assert apply_key_scale(w) == cfg.n_layers
    assert apply_key_scale(w) == 0                       # folding twice would square the scale
    lw = w.layers[0]
    after_k = _rope(k * lw.k_norm.double(), pos)
    scores1 = _rope(q * lw.q_norm.double(), pos) @ after_k.t()
    assert torch.allclose(scores0, scores1, rtol=1e-5, atol=1e-5)
    assert lw.k_norm.abs().max() <= 1.0 + 1e-6
    assert _q8_err(after_k.float()) < 0.7 * _q8_err(before_k.float())
