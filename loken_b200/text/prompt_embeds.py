"""`prompt_embeds`: a prompt given as embedding rows instead of text (`/v1/completions`).

Three payload forms, told apart by their first bytes as the reference does
(`docs/API.md:56-118`, `src/inference/prompt_embeds/{mod,torch}.rs`):

  loken's format   magic 00 00 C0 FF 'LKEM' (an f32 NaN followed by four letters, so a bare f32
                   payload can never collide), version 1, dtype, rows, width, values, CRC-32
  torch.save       the zip archive `torch.save(tensor, buffer)` writes ('PK\\x03\\x04'): read WITHOUT
                   running its pickle: the pickle stream is walked by a restricted reader that knows
                   only the globals, opcodes and persistent references of one plain tensor
  bare f32         little-endian float32 values, width = the model's hidden size

Every form is refused (ValueError naming the fault) when the rows are not the model's width or would
fill the context window: checked before any value is converted; and when a value is not finite:
checked after.
"""
from __future__ import annotations

import base64
import io
import pickle
import struct
import zipfile
import zlib
from typing import List, Sequence, Union

import numpy as np

MAGIC = b"\x00\x00\xc0\xffLKEM"
_DT = {0: ("<f4", 4), 1: ("<f2", 2), 2: ("bf16", 2)}


def _bf16_to_f32(raw: bytes, n: int) -> np.ndarray:
    u = np.frombuffer(raw, dtype="<u2", count=n).astype("<u4") << 16
    return u.view("<f4")


def encode_loken(rows: np.ndarray, dtype: str = "f4") -> bytes:
    """The loken container of a [rows, width] array; dtype f4 | f2 | bf16."""
    rows = np.ascontiguousarray(rows, dtype="<f4")
    code = {"f4": 0, "f2": 1, "bf16": 2}[dtype]
    if code == 0:
        body = rows.tobytes()
    elif code == 1:
        body = rows.astype("<f2").tobytes()
    else:
        body = (rows.view("<u4") >> 16).astype("<u2").tobytes()
    head = MAGIC + struct.pack("<HBBIII", 1, code, 0, rows.shape[0], rows.shape[1], 0)
    blob = head + body
    return blob + struct.pack("<I", zlib.crc32(blob))


def _check_shape(n_rows: int, width: int, hidden: int, max_rows: int):
    if width != hidden:
        raise ValueError(f"prompt_embeds rows are {width} wide; the model's hidden size is {hidden}")
    if n_rows < 1:
        raise ValueError("prompt_embeds holds no rows")
    if n_rows >= max_rows:
        raise ValueError(f"prompt_embeds holds {n_rows} rows; the served context window holds {max_rows}")


def _finite(a: np.ndarray) -> np.ndarray:
    if not np.isfinite(a).all():
        raise ValueError("prompt_embeds holds a value that is not finite")
    return a


def _decode_loken(b: bytes, hidden: int, max_rows: int) -> np.ndarray:
    if len(b) < 28:
        raise ValueError("prompt_embeds (loken format) is truncated")
    ver, code, _r0, n_rows, width, _r1 = struct.unpack_from("<HBBIII", b, 8)
    if ver != 1:
        raise ValueError(f"prompt_embeds (loken format) version {ver} is not supported")
    if code not in _DT:
        raise ValueError(f"prompt_embeds (loken format) dtype code {code} is unknown")
    _check_shape(n_rows, width, hidden, max_rows)
    size = _DT[code][1]
    if len(b) != 28 + n_rows * width * size:
        raise ValueError("prompt_embeds (loken format) is truncated or padded")
    (crc,) = struct.unpack_from("<I", b, len(b) - 4)
    if zlib.crc32(b[:-4]) != crc:
        raise ValueError("prompt_embeds (loken format) is corrupted (CRC-32 mismatch)")
    raw = b[24:-4]
    n = n_rows * width
    if code == 2:
        a = _bf16_to_f32(raw, n)
    else:
        a = np.frombuffer(raw, dtype=_DT[code][0], count=n).astype("<f4")
    return _finite(a.reshape(n_rows, width))


# ---- torch.save without unpickling -------------------------------------------------------------
class _Storage:
    def __init__(self, kind: str):
        self.kind = kind


_STORAGES = {"FloatStorage": ("<f4", 4), "HalfStorage": ("<f2", 2), "BFloat16Storage": ("bf16", 2),
             "DoubleStorage": ("<f8", 8)}


class _TensorStub:
    def __init__(self, storage, offset, size, stride):
        self.storage, self.offset, self.size, self.stride = storage, offset, tuple(size), tuple(stride)


def _rebuild_tensor_v2(storage, storage_offset, size, stride, requires_grad=False, backward_hooks=None, metadata=None):
    if backward_hooks:
        raise ValueError("prompt_embeds: a tensor carrying hooks is refused")
    if metadata:
        raise ValueError("prompt_embeds: a tensor carrying attributes is refused")
    return _TensorStub(storage, int(storage_offset), size, stride)


class _PlainTensorReader(pickle.Unpickler):
    """Knows exactly the globals of one plain tensor; everything else is refused, nothing is called
    but the inert stand-ins above."""

    def find_class(self, module, name):
        if module == "torch._utils" and name == "_rebuild_tensor_v2":
            return _rebuild_tensor_v2
        if module == "collections" and name == "OrderedDict":
            import collections

            return collections.OrderedDict
        if module == "torch" and name in _STORAGES:
            return _Storage(name)
        raise ValueError(f"prompt_embeds: the archive names {module}.{name}, which a plain tensor does not need")

    def persistent_load(self, pid):
        # ('storage', storage_type, key, location, numel)
        if not (isinstance(pid, tuple) and len(pid) == 5 and pid[0] == "storage" and isinstance(pid[1], _Storage)):
            raise ValueError("prompt_embeds: unexpected persistent reference in the archive")
        return (pid[1].kind, str(pid[2]), int(pid[4]))


def _decode_torch(b: bytes, hidden: int, max_rows: int) -> np.ndarray:
    try:
        z = zipfile.ZipFile(io.BytesIO(b))
    except zipfile.BadZipFile:
        raise ValueError("prompt_embeds: not a readable torch.save archive")
    names = z.namelist()
    pkl = [n for n in names if n.endswith("/data.pkl") or n == "data.pkl"]
    if len(pkl) != 1:
        raise ValueError("prompt_embeds: torch's legacy format or several objects are refused")
    for info in z.infolist():
        if info.compress_type != zipfile.ZIP_STORED:
            raise ValueError("prompt_embeds: compressed archives are refused")
    root = pkl[0][:-len("data.pkl")]
    if any(n.endswith("byteorder") and z.read(n).strip() != b"little" for n in names):
        raise ValueError("prompt_embeds: big-endian archives are refused")
    obj = _PlainTensorReader(io.BytesIO(z.read(pkl[0]))).load()       # zipfile checks each entry's CRC-32 on read
    if not isinstance(obj, _TensorStub):
        raise ValueError("prompt_embeds: the archive does not hold one plain tensor")
    kind, key, numel = obj.storage
    size = obj.size
    if len(size) == 3 and size[0] == 1:
        size, stride = size[1:], obj.stride[1:]
    else:
        stride = obj.stride
    if len(size) != 2:
        raise ValueError(f"prompt_embeds: tensor of shape {list(obj.size)}; (tokens, hidden) or (1, tokens, hidden) is expected")
    _check_shape(size[0], size[1], hidden, max_rows)
    dt, esz = _STORAGES[kind]
    raw = z.read(f"{root}data/{key}")
    if len(raw) < numel * esz:
        raise ValueError("prompt_embeds: the archive's storage is shorter than its tensor")
    flat = _bf16_to_f32(raw, numel) if dt == "bf16" else np.frombuffer(raw, dtype=dt, count=numel)
    last = obj.offset + (size[0] - 1) * stride[0] + (size[1] - 1) * stride[1]
    if obj.offset < 0 or min(stride) < 0 or last >= numel:
        raise ValueError("prompt_embeds: the tensor reaches outside its storage")
    a = np.lib.stride_tricks.as_strided(flat[obj.offset:], shape=size, strides=(stride[0] * flat.itemsize,
                                                                                   stride[1] * flat.itemsize))
    return _finite(np.ascontiguousarray(a, dtype="<f4"))


def decode_one(payload: Union[str, bytes, Sequence], hidden: int, max_rows: int) -> np.ndarray:
    """One prompt's embedding rows as float32 [rows, hidden]."""
    if isinstance(payload, (list, tuple)):
        rows = payload
        if not rows or not isinstance(rows[0], (list, tuple)):
            raise ValueError("prompt_embeds: an array of rows of numbers is expected")
        _check_shape(len(rows), len(rows[0]), hidden, max_rows)
        if any(len(r) != hidden for r in rows):
            raise ValueError("prompt_embeds: the rows differ in width")
        try:
            return _finite(np.asarray(rows, dtype="<f4"))
        except (TypeError, ValueError) as e:
            raise ValueError(f"prompt_embeds: rows of numbers are expected ({e})")
    if isinstance(payload, str):
        try:
            b = base64.b64decode(payload, validate=True)
        except Exception:
            raise ValueError("prompt_embeds is not valid base64")
    else:
        b = bytes(payload)
    if b[:8] == MAGIC:
        return _decode_loken(b, hidden, max_rows)
    if b[:4] == b"PK\x03\x04":
        return _decode_torch(b, hidden, max_rows)
    if len(b) == 0 or len(b) % (4 * hidden):
        raise ValueError(f"prompt_embeds (bare f32): {len(b)} bytes is not a whole number of rows of {hidden} values")
    n_rows = len(b) // (4 * hidden)
    _check_shape(n_rows, hidden, hidden, max_rows)
    return _finite(np.frombuffer(b, dtype="<f4").reshape(n_rows, hidden).copy())


def decode_request(value, hidden: int, max_rows: int) -> List[np.ndarray]:
    """`prompt_embeds` of a request body: a base64 string (one prompt), an array of base64 strings
    (one prompt each) or an array of rows of numbers (one prompt)."""
    if isinstance(value, str):
        return [decode_one(value, hidden, max_rows)]
    if isinstance(value, list) and value and all(isinstance(v, str) for v in value):
        return [decode_one(v, hidden, max_rows) for v in value]
    if isinstance(value, list):
        return [decode_one(value, hidden, max_rows)]
    raise ValueError("prompt_embeds takes a base64 string, an array of base64 strings or an array of rows of numbers")
