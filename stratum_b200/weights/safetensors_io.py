"""Reading and writing the safetensors container, without any helper package.

Layout (as the reference's own parser reads it, stratum/native/stratum_st.h:232-336):
an 8-byte little-endian header length N, N bytes of JSON mapping each tensor
name to {"dtype", "shape", "data_offsets": [begin, end]} (offsets relative to
the first byte after the header), then the raw little-endian data.  The reader
maps the file and refuses anything inconsistent before a byte of data is used:
header length beyond the file, offsets out of range or out of order, a byte
count that disagrees with shape x dtype, duplicate names, unknown dtypes
(cf. the reference's hostile-file guards, stratum/native/stratum_gguf.h:273-287, :398-420).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I32": (torch.int32, 4), "I64": (torch.int64, 8),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int        # absolute byte offset in the file
    nbytes: int
    path: str


def _no_duplicates(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise SafetensorsError(f"duplicate tensor name {k!r} in header")
        seen[k] = v
    return seen


class SafetensorsFile:
    """One mapped file and its index; tensors are views of the mapping until copied."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError as e:
            raise SafetensorsError(f"{path}: {e.strerror}") from None
        if size < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a safetensors header")
        self._fh = open(path, "rb")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"), object_pairs_hook=_no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        data0 = 8 + hlen
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, TensorEntry] = {}
        spans: List[Tuple[int, int, str]] = []
        for name, info in header.items():
            if not isinstance(info, dict) or not {"dtype", "shape", "data_offsets"} <= set(info):
                raise SafetensorsError(f"{path}: entry {name!r} lacks dtype/shape/data_offsets")
            dt = info["dtype"]
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            shape = info["shape"]
            if not isinstance(shape, list) or any(isinstance(d, bool) or not isinstance(d, int) or d < 0
                                                  for d in shape):
                raise SafetensorsError(f"{path}: tensor {name!r} has a malformed shape {shape!r}")
            off = info["data_offsets"]
            if (not isinstance(off, list) or len(off) != 2
                    or any(isinstance(o, bool) or not isinstance(o, int) for o in off)):
                raise SafetensorsError(f"{path}: tensor {name!r} has malformed data_offsets {off!r}")
            b, e = off
            count = 1
            for d in shape:
                count *= d
            want = count * _DTYPES[dt][1]
            if b < 0 or e < b or data0 + e > size:
                raise SafetensorsError(f"{path}: tensor {name!r} data [{b}, {e}) lies outside the file")
            if e - b != want:
                raise SafetensorsError(f"{path}: tensor {name!r} holds {e - b} bytes, "
                                       f"shape {shape} x {dt} needs {want}")
            spans.append((b, e, name))
            self.entries[name] = TensorEntry(name, _DTYPES[dt][0], tuple(shape), data0 + b, want, path)
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{path}: tensors {n0!r} and {n1!r} overlap")

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapping (read-only memory: copy before writing)."""
        e = self.entries[name]
        if e.nbytes == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        count = e.nbytes // _DTYPES[_NAMES[e.dtype]][1]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # the mapping is read-only; nothing here writes to it
            t = torch.frombuffer(self._mm, dtype=e.dtype, count=count, offset=e.begin)
        return t.view(e.shape)

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass                                  # a tensor still views the mapping; the OS frees it at exit
        self._fh.close()


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """model.safetensors, or the shards model.safetensors.index.json names."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    if os.path.isfile(index):
        try:
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f)["weight_map"]
            shards = sorted(set(weight_map.values()))
        except (OSError, KeyError, TypeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{index}: cannot read the shard index ({e})") from None
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]
    raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write CPU tensors in name order, data aligned to 64 bytes after the header."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} (tensor {name!r})")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (-(8 + len(blob))) % 64
    blob += b" " * pad
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
