"""torch.save checkpoints read without running them: values, views, wrappers, and files that try something."""
import collections
import os
import pickle
import zipfile

import pytest
import torch

from loken_b200.formats.pth import PthError, PthReader, read_state_dict


def test_state_dict_round_trip(tmp_path):
    g = torch.Generator().manual_seed(0)
    base = torch.randn(6, 8, generator=g)
    sd = collections.OrderedDict(
        a=torch.randn(4, 5, generator=g), b=torch.randn(3, 7, generator=g).bfloat16(), c=torch.randn(9, generator=g).half(),
        ids=torch.arange(12).reshape(3, 4), flags=torch.tensor([True, False, True]), bytes=torch.arange(200, dtype=torch.uint8),
        view=base[1:5, 2:6], transposed=base.t(), empty=torch.zeros(0, 3), scalar=torch.tensor(3.5),
        param=torch.nn.Parameter(torch.randn(2, 2, generator=g)))
    p = str(tmp_path / "m.bin")
    torch.save(sd, p)
    r = PthReader(p)
    assert set(r.keys()) == set(sd) and r.shape("view") == (4, 4) and r.dtype("b") == torch.bfloat16
    for k, v in sd.items():
        got = r.get_tensor(k)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v.detach()), k
    r.close()
    # wrappers are peeled, nesting is joined with dots, hyper-parameters are skipped
    torch.save({"state_dict": {"enc": {"w": sd["a"]}, "dec.w": sd["c"]}, "epoch": 3, "args": ["x", 1]}, p)
    got = read_state_dict(p)
    assert set(got) == {"enc.w", "dec.w"} and torch.equal(got["enc.w"], sd["a"])


class _Evil:
    def __reduce__(self):
        return (os.system, ("echo pwned > /dev/null",))


def test_anything_else_is_refused(tmp_path):
    p = str(tmp_path / "evil.bin")
    torch.save({"w": torch.zeros(2), "x": _Evil()}, p)
    with pytest.raises(PthError, match="system"):
        PthReader(p)
    with open(p, "wb") as f:
        f.write(b"not a zip")
    with pytest.raises(PthError):
        PthReader(p)
    # a tensor that claims more than its storage holds
    q = str(tmp_path / "short.bin")
    torch.save({"w": torch.arange(10.0)}, q)
    z = zipfile.ZipFile(q)
    names = z.namelist()
    pkl = [n for n in names if n.endswith("data.pkl")][0]
    blob = z.read(pkl).replace(pickle.dumps(10, protocol=2)[2:-1], pickle.dumps(99, protocol=2)[2:-1])
    out = str(tmp_path / "lying.bin")
    with zipfile.ZipFile(out, "w", zipfile.ZIP_STORED) as zo:
        for n in names:
            zo.writestr(n, blob if n == pkl else z.read(n))
    with pytest.raises(PthError):
        PthReader(out).get_tensor("w")


def test_hf_loader_reads_a_bin_checkpoint(tmp_path):
    """The same tiny model saved as safetensors and as pytorch_model.bin loads to the same weights."""
    from safetensors.torch import load_file

    from loken_b200.models import loader_hf
    from loken_b200.models.config import tiny
    from loken_b200.models.weights import random_weights

    cfg = tiny("llama", weight_format="fp8_block", head_dim=128, n_q=4, n_kv=2, hidden=512, intermediate=1024)
    cfg.rope_pairing = 1
    w = random_weights(cfg, torch.device("cpu"), seed=3, std=0.05)
    d1, d2 = tmp_path / "st", tmp_path / "bin"
    os.makedirs(d1)
    loader_hf.save_hf_fp8(str(d1), cfg, w)
    os.makedirs(d2)
    for f in os.listdir(d1):
        if f.endswith(".safetensors"):
            torch.save(load_file(str(d1 / f)), str(d2 / "pytorch_model.bin"))
        else:
            (d2 / f).write_bytes((d1 / f).read_bytes())
    a, _ = loader_hf.load_hf(str(d1), torch.device("cpu"))
    b, _ = loader_hf.load_hf(str(d2), torch.device("cpu"))
    assert torch.equal(a.embed, b.embed)
    for la, lb in zip(a.layers, b.layers):
        assert lb.wqkv.kind == "fp8_block"
        assert torch.equal(la.wqkv.weight.data.view(torch.uint8), lb.wqkv.weight.data.view(torch.uint8))
        assert torch.equal(la.w_down.weight.scale, lb.w_down.weight.scale)
