"""Reading and writing safetensors files, by tensor name.

File layout: 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``,
then the tensor bytes.  The header is validated with the rules the reference
applies (src/io/QuickNN.SafeTensors.pas:548-675): bounded header length, a JSON
object, string-valued ``__metadata__``, a known dtype, offsets inside the buffer,
byte count equal to shape x dtype size, no overlap, no gap, full coverage, no
duplicate names.  Shards are found through ``model.safetensors.index.json``'s
``weight_map`` (SafeTensors.pas:777-834).

Tensors come back as views of a read-only memory map in their stored dtype.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
MAX_HEADER_BYTES = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


def _no_duplicates(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise SafetensorsError(f"duplicate tensor name in header: {k!r}")
        seen[k] = v
    return seen


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end")

    def __init__(self, name, dtype, shape, begin, end):
        self.name, self.dtype, self.shape, self.begin, self.end = name, dtype, shape, begin, end


class SafetensorsFile:
    """One memory-mapped file with a validated directory."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: file is shorter than its 8-byte header length")
        self._fh = open(path, "rb")
        try:
            (hlen,) = struct.unpack("<Q", self._fh.read(8))
            if hlen < 2 or hlen > MAX_HEADER_BYTES or 8 + hlen > size:
                raise SafetensorsError(f"{path}: header length {hlen} is out of bounds "
                                       f"(file has {size} bytes)")
            raw = self._fh.read(hlen)
            try:
                header = json.loads(raw.decode("utf-8"), object_pairs_hook=_no_duplicates)
            except UnicodeDecodeError as e:
                raise SafetensorsError(f"{path}: header is not UTF-8: {e}") from None
            except json.JSONDecodeError as e:
                raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
            if not isinstance(header, dict):
                raise SafetensorsError(f"{path}: header is not a JSON object")
            self.data_start = 8 + hlen
            self.data_bytes = size - self.data_start
            self.metadata: Dict[str, str] = {}
            self.entries: Dict[str, TensorEntry] = {}
            self._parse(header)
            self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        except Exception:
            self._fh.close()
            raise

    def _parse(self, header: dict) -> None:
        path = self.path
        meta = header.get("__metadata__")
        if meta is not None:
            if not isinstance(meta, dict) or not all(isinstance(v, str) for v in meta.values()):
                raise SafetensorsError(f"{path}: __metadata__ must map strings to strings")
            self.metadata = dict(meta)
        spans: List[Tuple[int, int, str]] = []
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if not isinstance(info, dict):
                raise SafetensorsError(f"{path}: entry {name!r} is not an object")
            dt = info.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unknown dtype {dt!r}")
            shape = info.get("shape")
            if not isinstance(shape, list) or not all(isinstance(d, int) and d >= 0 for d in shape):
                raise SafetensorsError(f"{path}: tensor {name!r} has an invalid shape {shape!r}")
            off = info.get("data_offsets")
            if (not isinstance(off, list) or len(off) != 2
                    or not all(isinstance(o, int) for o in off)):
                raise SafetensorsError(f"{path}: tensor {name!r} has invalid data_offsets {off!r}")
            b, e = off
            if b < 0 or e < b or e > self.data_bytes:
                raise SafetensorsError(f"{path}: tensor {name!r} lies outside the data "
                                       f"({b}..{e} of {self.data_bytes} bytes; truncated file?)")
            count = 1
            for d in shape:
                count *= d
            if count * _DTYPES[dt][1] != e - b:
                raise SafetensorsError(f"{path}: tensor {name!r} has {e - b} bytes but its shape "
                                       f"{shape} x {dt} needs {count * _DTYPES[dt][1]}")
            self.entries[name] = TensorEntry(name, _DTYPES[dt][0], tuple(shape), b, e)
            spans.append((b, e, name))
        spans.sort()
        cursor = 0
        for b, e, name in spans:
            if b < cursor:
                raise SafetensorsError(f"{path}: tensor {name!r} overlaps the one before it")
            if b > cursor:
                raise SafetensorsError(f"{path}: {b - cursor} unused bytes before tensor {name!r}")
            cursor = e
        if cursor != self.data_bytes:
            raise SafetensorsError(f"{path}: {self.data_bytes - cursor} bytes after the last tensor "
                                   f"are not covered by the header")

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        count = 1
        for d in e.shape:
            count *= d
        if count == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        with warnings.catch_warnings():
            # the map is read-only on purpose; nothing here writes through the tensor
            warnings.filterwarnings("ignore", message="The given buffer is not writable")
            t = torch.frombuffer(self._mm, dtype=e.dtype, count=count, offset=self.data_start + e.begin)
        return t.view(e.shape)

    def close(self) -> None:
        # tensors handed out keep the map alive through the buffer protocol
        try:
            self._fh.close()
        except Exception:
            pass


class TensorDirectory:
    """All tensors of a model folder: one file or shards behind an index."""

    def __init__(self, files: Iterable[SafetensorsFile], where: Mapping[str, SafetensorsFile]):
        self.files = list(files)
        self._where = dict(where)

    @classmethod
    def open(cls, model_dir: str) -> "TensorDirectory":
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as fh:
                idx = json.load(fh)
            wm = idx.get("weight_map") if isinstance(idx, dict) else None
            if not isinstance(wm, dict):
                raise SafetensorsError(f"{index}: no weight_map")
            files: Dict[str, SafetensorsFile] = {}
            where: Dict[str, SafetensorsFile] = {}
            for name, shard in wm.items():
                if shard not in files:
                    files[shard] = SafetensorsFile(os.path.join(model_dir, shard))
                if name not in files[shard].entries:
                    raise SafetensorsError(f"{index}: tensor {name!r} is not in shard {shard!r}")
                where[name] = files[shard]
            for shard, f in files.items():
                for name in f.entries:
                    if where.get(name) is not f:
                        raise SafetensorsError(
                            f"{index}: shard {shard!r} holds {name!r} that the index does not map to it")
            return cls(files.values(), where)
        if os.path.isfile(single):
            f = SafetensorsFile(single)
            return cls([f], {n: f for n in f.entries})
        raise FileNotFoundError(f"no model.safetensors or model.safetensors.index.json in {model_dir}")

    def names(self) -> List[str]:
        return list(self._where)

    def shape_dtype(self, name: str) -> Tuple[Tuple[int, ...], torch.dtype]:
        e = self._where[name].entries[name]
        return e.shape, e.dtype

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write tensors in name order, contiguous, without gaps."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of {name!r}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                fh.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)
