"""`prompt_embeds` payloads: loken's container, `torch.save` read without unpickling, bare f32,
the refusals, and the engine-side embedding override on CPU fakes."""
import base64
import io
import struct
import zlib

import numpy as np
import pytest
import torch

from loken_b200.text import prompt_embeds as pe


def test_loken_container_round_trip_and_refusals():
    rows = np.random.default_rng(0).standard_normal((5, 64)).astype("<f4")
    for dt, tol in (("f4", 0), ("f2", 2e-3), ("bf16", 1e-2)):
        b = pe.encode_loken(rows, dt)
        assert b[:8] == bytes.fromhex("0000c0ff4c4b454d") and len(b) == 28 + 5 * 64 * (4 if dt == "f4" else 2)
        got = pe.decode_one(base64.b64encode(b).decode(), 64, 4096)
        assert got.shape == (5, 64) and np.abs(got - rows).max() <= tol * max(1.0, np.abs(rows).max())
    b = pe.encode_loken(rows)
    with pytest.raises(ValueError, match="corrupted"):
        pe.decode_one(b[:30] + bytes([b[30] ^ 1]) + b[31:], 64, 4096)
    with pytest.raises(ValueError, match="truncated or padded"):
        pe.decode_one(b + b"\0", 64, 4096)
    with pytest.raises(ValueError, match="hidden size"):
        pe.decode_one(b, 128, 4096)
    with pytest.raises(ValueError, match="context window"):
        pe.decode_one(b, 64, 5)
    bad = rows.copy()
    bad[1, 2] = np.inf
    with pytest.raises(ValueError, match="not finite"):
        pe.decode_one(pe.encode_loken(bad), 64, 4096)
    with pytest.raises(ValueError, match="base64"):
        pe.decode_one("@@@", 64, 4096)


def test_torch_save_is_read_without_running_its_pickle():
    t = torch.randn(7, 32)
    for tensor in (t, t.half(), t.bfloat16(), t.double(), t.unsqueeze(0), torch.randn(9, 40)[1:8, 4:36]):
        buf = io.BytesIO()
        torch.save(tensor, buf)
        got = pe.decode_one(base64.b64encode(buf.getvalue()).decode(), 32, 4096)
        want = tensor.float().reshape(-1, 32).numpy()
        assert got.shape == want.shape and np.allclose(got, want, atol=1e-6)
    # an archive that names any other global is refused before anything of it runs
    buf = io.BytesIO()
    torch.save({"x": t, "fn": print}, buf)
    with pytest.raises(ValueError):
        pe.decode_one(buf.getvalue(), 32, 4096)
    buf = io.BytesIO()
    torch.save([t, t], buf)
    with pytest.raises(ValueError, match="one plain tensor"):
        pe.decode_one(buf.getvalue(), 32, 4096)


def test_bare_f32_and_row_arrays():
    rows = np.arange(3 * 16, dtype="<f4").reshape(3, 16)
    assert np.array_equal(pe.decode_one(rows.tobytes(), 16, 100), rows)
    assert np.array_equal(pe.decode_request(rows.tolist(), 16, 100)[0], rows)
    two = pe.decode_request([base64.b64encode(rows.tobytes()).decode(), base64.b64encode(pe.encode_loken(rows)).decode()],
                            16, 100)
    assert len(two) == 2 and np.array_equal(two[0], two[1])
    with pytest.raises(ValueError, match="whole number of rows"):
        pe.decode_one(rows.tobytes()[:-4], 16, 100)
    # the magic is an f32 NaN: a bare payload that starts with it would be taken for the container,
    # and a bare payload may not carry a NaN anyway
    assert np.isnan(struct.unpack("<f", pe.MAGIC[:4])[0])
    assert zlib.crc32(b"") == 0


def test_completions_route_takes_prompt_embeds():
    from fastapi.testclient import TestClient

    from loken_b200.api.common import ModelRegistry
    from loken_b200.api.server import create_app
    from tests.fakes import fake_llm

    reg = ModelRegistry()
    llm = fake_llm("from rows")
    reg.add(llm)
    c = TestClient(create_app(reg, None))
    H = llm.cfg.hidden
    rows = np.random.default_rng(1).standard_normal((6, H)).astype("<f4")
    r = c.post("/v1/completions", json={"prompt_embeds": base64.b64encode(pe.encode_loken(rows, "f2")).decode(),
                                        "max_tokens": 4})
    assert r.status_code == 200, r.text
    j = r.json()
    assert j["choices"][0]["text"] == "from" and j["usage"]["prompt_tokens"] == 6
    got = llm.engine.embeds[-1]
    assert got.shape == (6, H) and np.abs(got - rows).max() < 2e-2
    # two payloads: two prompts, two choices
    r2 = c.post("/v1/completions", json={"prompt_embeds": [base64.b64encode(rows.tobytes()).decode()] * 2,
                                         "max_tokens": 2}).json()
    assert len(r2["choices"]) == 2
    bad = c.post("/v1/completions", json={"prompt_embeds": base64.b64encode(rows[:, :-1].tobytes()).decode()})
    assert bad.status_code == 400 and "rows" in bad.text
