"""Reader and writer for the safetensors container (own code; the format is small).

Layout: 8 bytes little-endian header length, a JSON header ``{name: {"dtype", "shape",
"data_offsets": [begin, end]}, "__metadata__": {...}}``, then the raw little-endian tensor
bytes. The reference reads such files through ``safe_load_file``
(src/transformers/modeling_utils.py:502-511), refusing archives whose ``format`` metadata is
not one of pt/tf/flax/mlx, and resolves sharded checkpoints through
``model.safetensors.index.json`` (src/transformers/utils/hub.py:1034-1085).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Iterator, List, Optional, Tuple

import numpy as np
import torch

SAFE_WEIGHTS_NAME = "model.safetensors"                   # src/transformers/utils/__init__.py:261
SAFE_WEIGHTS_INDEX_NAME = "model.safetensors.index.json"  # src/transformers/utils/__init__.py:262

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_CODES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors archive."""


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "path")

    def __init__(self, name, dtype, shape, begin, end, path):
        self.name, self.dtype, self.shape, self.begin, self.end, self.path = name, dtype, shape, begin, end, path

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class SafetensorsFile:
    """One archive, memory-mapped; tensors are materialised one at a time."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header ({size} bytes)")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes); truncated file?")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: the header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: the header is not a JSON object")
        self.metadata: Dict[str, str] = header.pop("__metadata__", None) or {}
        self._data_start = 8 + hlen
        payload = size - self._data_start
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                code, shape, (begin, end) = info["dtype"], [int(s) for s in info["shape"]], info["data_offsets"]
            except (KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}: {info!r}") from e
            if code not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has dtype {code!r}, which is not supported "
                                       f"(supported: {', '.join(sorted(_DTYPES))})")
            entry = TensorEntry(name, _DTYPES[code][0], tuple(shape), int(begin), int(end), path)
            want = entry.numel * _DTYPES[code][1]
            if begin < 0 or end < begin or end - begin != want:
                raise SafetensorsError(f"{path}: tensor {name!r} of shape {shape} and dtype {code} needs {want} "
                                       f"bytes but its offsets give {end - begin}")
            if end > payload:
                raise SafetensorsError(f"{path}: tensor {name!r} ends at byte {end} of a payload of {payload} "
                                       f"bytes; truncated file?")
            self.entries[name] = entry
        self._mm: Optional[mmap.mmap] = None
        if payload > 0:
            self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A host tensor that owns its memory (copied out of the mapping)."""
        e = self.entries[name]
        if e.numel == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = bytearray(self._mm[self._data_start + e.begin:self._data_start + e.end])
        return torch.frombuffer(buf, dtype=e.dtype).reshape(e.shape)

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass  # a view is still alive; the mapping goes with it
            self._mm = None
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def checkpoint_files(folder: str) -> List[str]:
    """The archive(s) of a model folder: the single file, else the shards that the index names."""
    single = os.path.join(folder, SAFE_WEIGHTS_NAME)
    if os.path.isfile(single):
        return [single]
    index = os.path.join(folder, SAFE_WEIGHTS_INDEX_NAME)
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map", {})
        files = sorted(set(weight_map.values()))
        missing = [f for f in files if not os.path.isfile(os.path.join(folder, f))]
        if missing:
            raise FileNotFoundError(f"{index} names shard files that are not in the folder: {missing}")
        return [os.path.join(folder, f) for f in files]
    others = [f for f in os.listdir(folder) if f.endswith(".bin")] if os.path.isdir(folder) else []
    hint = f" (found {others}: convert them to safetensors first)" if others else ""
    raise FileNotFoundError(f"no {SAFE_WEIGHTS_NAME} or {SAFE_WEIGHTS_INDEX_NAME} in model folder {folder!r}{hint}")


def open_checkpoint(folder: str) -> Tuple[List[SafetensorsFile], Dict[str, SafetensorsFile]]:
    """Open every archive of a folder; returns the files and a map tensor name -> file.
    A name that two shards hold is an error."""
    files = [SafetensorsFile(p) for p in checkpoint_files(folder)]
    where: Dict[str, SafetensorsFile] = {}
    for f in files:
        fmt = f.metadata.get("format")
        if fmt is not None and fmt not in ("pt", "tf", "flax", "mlx"):
            raise SafetensorsError(f"{f.path}: metadata format {fmt!r} is not one of pt, tf, flax, mlx")
        for name in f.keys():
            if name in where:
                raise SafetensorsError(f"tensor {name!r} is stored in both {where[name].path} and {f.path}")
            where[name] = f
    return files, where


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Optional[dict] = None,
                      plan: Optional[List[Tuple[str, torch.dtype, Tuple[int, ...]]]] = None) -> None:
    """Write an archive. ``tensors`` yields (name, host tensor) in the order of ``plan`` (a list of
    (name, dtype, shape)); without a plan the tensors are gathered first. With a plan they are
    streamed, so a model larger than host memory's spare room can be written tensor by tensor."""
    if plan is None:
        items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
        plan = [(n, t.dtype, tuple(t.shape)) for n, t in items]
        tensors = iter(items)
    header: Dict[str, dict] = {}
    if metadata is not None:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, dtype, shape in plan:
        if dtype not in _CODES:
            raise SafetensorsError(f"tensor {name!r}: dtype {dtype} cannot be stored")
        n = 1
        for s in shape:
            n *= s
        nbytes = n * _DTYPES[_CODES[dtype]][1]
        header[name] = {"dtype": _CODES[dtype], "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for (name, dtype, shape), (tname, t) in zip(plan, tensors):
            if tname != name or t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(f"tensor {tname!r} {t.dtype} {tuple(t.shape)} does not follow the plan "
                                       f"({name!r} {dtype} {tuple(shape)})")
            t = t.detach().cpu().contiguous()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dtype == torch.bfloat16
                        else t.numpy().tobytes())
    os.replace(tmp, path)
