"""Reading and writing the safetensors container, without any library for it.

Format (the reference reads the same, crates/safetensors/src/lib.rs:62-124):
an unsigned 64-bit little-endian header length `n`, `n` bytes of JSON that map
each tensor name to `{"dtype", "shape", "data_offsets": [begin, end]}` (the key
`__metadata__` is not a tensor), then the data, offsets relative to its start.
Unlike the reference, which trusts `data_offsets`, every entry is checked here:
the range must lie inside the file and its length must equal shape x item size.
Files are memory-mapped, so a tensor is only paged in when it is copied.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# dtype tag -> (torch dtype, numpy carrier dtype, item size)
_DTYPES = {
    "F32": (torch.float32, np.float32, 4),
    "F16": (torch.float16, np.float16, 2),
    "BF16": (torch.bfloat16, np.uint16, 2),
    "F64": (torch.float64, np.float64, 8),
    "I64": (torch.int64, np.int64, 8),
    "I32": (torch.int32, np.int32, 4),
    "I16": (torch.int16, np.int16, 2),
    "I8": (torch.int8, np.int8, 1),
    "U8": (torch.uint8, np.uint8, 1),
    "BOOL": (torch.bool, np.bool_, 1),
}
_TAG_OF = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One memory-mapped file; `tensor(name)` gives a CPU tensor that views the map."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (shorter than the 8-byte length field)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", None)
        self._data_start = 8 + n
        data_len = size - self._data_start
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                tag, shape, (b, en) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor '{name}'") from None
            if tag not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {tag}")
            numel = 1
            for s in shape:
                numel *= s
            if not (0 <= b <= en <= data_len):
                raise SafetensorsError(f"{path}: tensor '{name}' data_offsets [{b},{en}] lie outside the data ({data_len} bytes)")
            if en - b != numel * _DTYPES[tag][2]:
                raise SafetensorsError(f"{path}: tensor '{name}' has {en - b} bytes but shape {list(shape)} of {tag} needs {numel * _DTYPES[tag][2]}")
            self.entries[name] = (tag, shape, int(b), int(en))
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def tensor(self, name: str) -> torch.Tensor:
        tag, shape, b, en = self.entries[name]
        tdt, ndt, isz = _DTYPES[tag]
        count = (en - b) // isz
        arr = np.frombuffer(self._mm, dtype=ndt, count=count, offset=self._data_start + b)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)     # the view is read-only; callers copy, never write
            t = torch.from_numpy(arr.copy() if count == 0 else arr)
        if tag == "BF16":
            t = t.view(torch.bfloat16)
        return t.reshape(shape)

    def close(self):
        # tensors handed out keep the map alive through numpy; nothing to force here
        self._f.close()


def open_model_tensors(model_dir: str) -> Dict[str, Tuple[SafetensorsFile, str]]:
    """Map every tensor name of a model folder to (file, name).  A folder holds
    either `model.safetensors` or `model.safetensors.index.json` with its shards
    (the reference reads only the single file, crates/cuda/src/engine.rs:3201)."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    out: Dict[str, Tuple[SafetensorsFile, str]] = {}
    if os.path.exists(single):
        f = SafetensorsFile(single)
        for n in f.names():
            out[n] = (f, n)
        return out
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as fh:
            wm = json.load(fh).get("weight_map")
        if not isinstance(wm, dict):
            raise SafetensorsError(f"{index}: no 'weight_map' object")
        files: Dict[str, SafetensorsFile] = {}
        for name, shard in wm.items():
            if shard not in files:
                files[shard] = SafetensorsFile(os.path.join(model_dir, shard))
            if name not in files[shard].entries:
                raise SafetensorsError(f"{index}: tensor '{name}' is not in shard {shard}")
            out[name] = (files[shard], name)
        return out
    raise FileNotFoundError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata=None) -> None:
    """Write tensors (any device) in name order, data aligned as the format asks
    (header padded with spaces to a multiple of 8)."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TAG_OF:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of '{name}'")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            elif t.dtype == torch.bool:
                t = t.view(torch.uint8)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)
