"""Checkpoints written by `torch.save` (`pytorch_model.bin`, `*.pth`, `*.pt`), read without running them.

A torch checkpoint is a zip archive: `data.pkl` is a pickle program that rebuilds a dict of tensors, the
tensors' bytes sit in `data/<key>` entries.  Unpickling a file from the network with the stock unpickler
executes whatever the file says.  This reader interprets the pickle with an unpickler that knows exactly
the handful of globals a state dict needs (ordered dicts, the tensor rebuild function, the storage types)
and maps each of them to an inert stand-in; any other global ends the read.  Tensor bytes are then read
straight from the archive, entry by entry, when a tensor is asked for (entries are stored uncompressed, so
one read per tensor; zipfile checks the entry's CRC)
(reference: `src/tensor/pth.rs`, "pickle subset without running it").

    r = PthReader("pytorch_model.bin")
    r.keys(); r.shape("model.embed_tokens.weight"); r.get_tensor("model.embed_tokens.weight")
"""
from __future__ import annotations

import collections
import io
import pickle
import zipfile
from typing import Dict, List, Tuple

import numpy as np
import torch

# storage class name -> (torch dtype, numpy dtype to read with, bytes per element)
STORAGES = {
    "FloatStorage": (torch.float32, "<f4", 4), "HalfStorage": (torch.float16, "<f2", 2),
    "BFloat16Storage": (torch.bfloat16, "<u2", 2), "DoubleStorage": (torch.float64, "<f8", 8),
    "LongStorage": (torch.int64, "<i8", 8), "IntStorage": (torch.int32, "<i4", 4), "ShortStorage": (torch.int16, "<i2", 2),
    "CharStorage": (torch.int8, "i1", 1), "ByteStorage": (torch.uint8, "u1", 1), "BoolStorage": (torch.bool, "u1", 1),
    "Float8_e4m3fnStorage": (torch.float8_e4m3fn, "u1", 1), "UntypedStorage": (torch.uint8, "u1", 1),
}
MAX_TENSORS = 1 << 20


class PthError(ValueError):
    pass


class _StorageType:
    def __init__(self, kind: str):
        self.kind = kind


class _Stub:
    """A tensor as the pickle describes it: which storage, where in it, what shape."""
    __slots__ = ("kind", "key", "numel", "offset", "size", "stride")

    def __init__(self, storage, offset, size, stride):
        self.kind, self.key, self.numel = storage
        self.offset, self.size, self.stride = int(offset), tuple(int(s) for s in size), tuple(int(s) for s in stride)


def _rebuild_tensor_v2(storage, storage_offset, size, stride, requires_grad=False, backward_hooks=None, metadata=None):
    return _Stub(storage, storage_offset, size, stride)


_DTYPE_STORAGE = {"float32": "FloatStorage", "float16": "HalfStorage", "bfloat16": "BFloat16Storage", "float64": "DoubleStorage",
                  "int64": "LongStorage", "int32": "IntStorage", "int16": "ShortStorage", "int8": "CharStorage",
                  "uint8": "ByteStorage", "bool": "BoolStorage", "float8_e4m3fn": "Float8_e4m3fnStorage"}


def _rebuild_tensor_v3(storage, storage_offset, size, stride, requires_grad, backward_hooks, dtype, metadata=None):
    """Dtypes without a storage class of their own (fp8): an untyped storage measured in bytes plus the dtype."""
    if dtype not in _DTYPE_STORAGE:
        raise PthError(f"tensors of dtype {dtype} are not read")
    kind = _DTYPE_STORAGE[dtype]
    _k, key, nbytes = storage
    return _Stub((kind, key, nbytes // STORAGES[kind][2]), storage_offset, size, stride)


def _rebuild_parameter(data, requires_grad=False, backward_hooks=None, *rest):
    return data


class _StateDictReader(pickle.Unpickler):
    def find_class(self, module, name):
        if module == "collections" and name == "OrderedDict":
            return collections.OrderedDict
        if module == "torch._utils" and name == "_rebuild_tensor_v2":
            return _rebuild_tensor_v2
        if module == "torch._utils" and name == "_rebuild_tensor_v3":
            return _rebuild_tensor_v3
        if module == "torch._utils" and name in ("_rebuild_parameter", "_rebuild_parameter_with_state"):
            return _rebuild_parameter
        if module == "torch" and name in STORAGES:
            return _StorageType(name)
        if module == "torch.storage" and name == "UntypedStorage":
            return _StorageType("UntypedStorage")
        if module == "torch" and name in _DTYPE_STORAGE:
            return name            # a dtype object: its name is all that is needed
        raise PthError(f"the checkpoint names {module}.{name}; a state dict needs no such object, so the file is refused")

    def persistent_load(self, pid):
        if not (isinstance(pid, tuple) and len(pid) >= 5 and pid[0] == "storage" and isinstance(pid[1], _StorageType)):
            raise PthError("unexpected persistent reference in the checkpoint")
        return (pid[1].kind, str(pid[2]), int(pid[4]))


def _flatten(obj, prefix: str, out: Dict[str, _Stub]):
    """State dicts nest (`{"model": {...}}`, `{"state_dict": {...}}`): names are joined with dots."""
    if isinstance(obj, _Stub):
        out[prefix] = obj
    elif isinstance(obj, dict):
        for k, v in obj.items():
            if not isinstance(k, (str, int)):
                continue
            _flatten(v, f"{prefix}.{k}" if prefix else str(k), out)
            if len(out) > MAX_TENSORS:
                raise PthError("the checkpoint names more tensors than any model has")
    # numbers, strings, lists of hyper-parameters: not tensors, not kept


class PthReader:
    def __init__(self, path: str):
        self.path = path
        try:
            self.zip = zipfile.ZipFile(path)
        except zipfile.BadZipFile:
            raise PthError(f"{path} is not a torch zip checkpoint (the legacy format before torch 1.6 is not read)")
        names = self.zip.namelist()
        pkl = [n for n in names if n.endswith("/data.pkl") or n == "data.pkl"]
        if len(pkl) != 1:
            raise PthError("the archive does not hold exactly one data.pkl")
        self.root = pkl[0][:-len("data.pkl")]
        for n in names:
            if n.endswith("byteorder") and self.zip.read(n).strip() != b"little":
                raise PthError("big-endian checkpoints are not read")
        obj = _StateDictReader(io.BytesIO(self.zip.read(pkl[0]))).load()
        self.tensors: Dict[str, _Stub] = {}
        _flatten(obj, "", self.tensors)
        # the common wrappers are peeled so names match what the model's loader expects
        for wrap in ("state_dict.", "model_state_dict.", "module."):
            if self.tensors and all(k.startswith(wrap) for k in self.tensors):
                self.tensors = {k[len(wrap):]: v for k, v in self.tensors.items()}

    def close(self):
        self.zip.close()

    def keys(self) -> List[str]:
        return list(self.tensors)

    def has(self, name: str) -> bool:
        return name in self.tensors

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.tensors[name].size

    def dtype(self, name: str) -> torch.dtype:
        return STORAGES[self.tensors[name].kind][0]

    def get_tensor(self, name: str) -> torch.Tensor:
        t = self.tensors[name]
        tdt, ndt, esz = STORAGES[t.kind]
        info = self.zip.getinfo(f"{self.root}data/{t.key}")
        if info.file_size < t.numel * esz:
            raise PthError(f"{name}: its storage is shorter than the checkpoint says")
        n = 1
        for s in t.size:
            n *= s
        # the reach of the view inside its storage, checked before anything is indexed
        last = t.offset + sum((s - 1) * st for s, st in zip(t.size, t.stride)) if n else t.offset
        if t.offset < 0 or any(st < 0 for st in t.stride) or (n and last >= t.numel):
            raise PthError(f"{name}: the tensor reaches outside its storage")
        raw = self.zip.read(info)
        flat = torch.from_numpy(np.frombuffer(raw, dtype=ndt, count=t.numel).copy())
        if tdt == torch.bfloat16:
            flat = flat.view(torch.int16).view(torch.bfloat16)
        elif tdt == torch.bool:
            flat = flat.bool()
        elif tdt == torch.float8_e4m3fn:
            flat = flat.view(torch.float8_e4m3fn)
        if n == 0:
            return torch.empty(t.size, dtype=tdt)
        return torch.as_strided(flat, t.size, t.stride, t.offset).contiguous()


def read_state_dict(path: str) -> Dict[str, torch.Tensor]:
    r = PthReader(path)
    try:
        return {k: r.get_tensor(k) for k in r.keys()}
    finally:
        r.close()
