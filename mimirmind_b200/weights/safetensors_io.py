"""safetensors container: reader (single file or sharded folder) and writer.

Format and checks follow the reference's container code: an 8-byte little-endian
header length, a JSON object ``{name: {dtype, shape, data_offsets}}`` with
``__metadata__`` skipped, offsets relative to the data region, byte length equal to
``prod(shape) * width``, ``begin <= end``, no negative dimension, no region past the
file (src/core/safetensors/SafetensorsHeader.cpp:33-153); a folder holds either a
shard index ``model.safetensors.index.json`` with a ``weight_map`` or a single
``model.safetensors`` (src/core/safetensors/SafetensorsModel.cpp:32-56), every mapped
tensor must exist in its shard and no tensor may appear in two shards (:100-129).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# dtype tag → (width in bytes, numpy carrier dtype, torch dtype)
_DTYPES = {
    "F64": (8, np.float64, torch.float64),
    "F32": (4, np.float32, torch.float32),
    "F16": (2, np.float16, torch.float16),
    "BF16": (2, np.uint16, torch.bfloat16),
    "I64": (8, np.int64, torch.int64),
    "I32": (4, np.int32, torch.int32),
    "I16": (2, np.int16, torch.int16),
    "I8": (1, np.int8, torch.int8),
    "U8": (1, np.uint8, torch.uint8),
    "BOOL": (1, np.bool_, torch.bool),
}
_TAG_OF_TORCH = {
    torch.float64: "F64",
    torch.float32: "F32",
    torch.float16: "F16",
    torch.bfloat16: "BF16",
    torch.int64: "I64",
    torch.int32: "I32",
    torch.int16: "I16",
    torch.int8: "I8",
    torch.uint8: "U8",
    torch.bool: "BOOL",
}

_MAX_HEADER = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorRecord:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int  # byte offsets inside the data region
    end: int
    shard: str  # file path


def parse_header(blob: bytes, file_size: int, where: str) -> Tuple[Dict[str, TensorRecord], int]:
    """Parse the first bytes of a safetensors file. Returns (records, data region start)."""
    if len(blob) < 8:
        raise SafetensorsError(f"{where}: file shorter than the 8-byte length prefix")
    (hlen,) = struct.unpack("<Q", blob[:8])
    if hlen == 0 or hlen > _MAX_HEADER:
        raise SafetensorsError(f"{where}: header length {hlen} is not plausible")
    if 8 + hlen > file_size:
        raise SafetensorsError(f"{where}: header ({hlen} bytes) runs past the end of the file")
    if len(blob) < 8 + hlen:
        raise SafetensorsError(f"{where}: header truncated")
    try:
        pairs = json.loads(blob[8 : 8 + hlen].decode("utf-8"), object_pairs_hook=list)
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"{where}: header is not valid JSON ({e})") from None
    if not isinstance(pairs, list):
        raise SafetensorsError(f"{where}: header is not a JSON object")
    data_start = 8 + hlen
    data_size = file_size - data_start
    records: Dict[str, TensorRecord] = {}
    for name, entry_pairs in pairs:
        if name == "__metadata__":
            continue
        if name in records:
            raise SafetensorsError(f"{where}: tensor '{name}' appears twice in the header")
        entry = dict(entry_pairs) if isinstance(entry_pairs, list) else None
        if entry is None or not all(k in entry for k in ("dtype", "shape", "data_offsets")):
            raise SafetensorsError(f"{where}: tensor '{name}' lacks dtype, shape or data_offsets")
        tag = entry["dtype"]
        if tag not in _DTYPES:
            raise SafetensorsError(f"{where}: tensor '{name}' has unknown dtype '{tag}'")
        shape = entry["shape"]
        if not isinstance(shape, list) or any((not isinstance(d, int)) or isinstance(d, bool) or d < 0 for d in shape):
            raise SafetensorsError(f"{where}: tensor '{name}' has an invalid shape {shape!r}")
        offs = entry["data_offsets"]
        if (
            not isinstance(offs, list)
            or len(offs) != 2
            or any((not isinstance(o, int)) or isinstance(o, bool) or o < 0 for o in offs)
        ):
            raise SafetensorsError(f"{where}: tensor '{name}' has invalid data_offsets {offs!r}")
        begin, end = offs
        if begin > end:
            raise SafetensorsError(f"{where}: tensor '{name}' has begin {begin} > end {end}")
        if end > data_size:
            raise SafetensorsError(f"{where}: tensor '{name}' ends at {end}, past the data region ({data_size} bytes)")
        count = 1
        for d in shape:
            count *= d
        want = count * _DTYPES[tag][0]
        if end - begin != want:
            raise SafetensorsError(
                f"{where}: tensor '{name}' holds {end - begin} bytes but shape {shape} of {tag} needs {want}"
            )
        records[name] = TensorRecord(name, tag, tuple(shape), begin, end, where)
    return records, data_start


class _Shard:
    def __init__(self, path: str):
        self.path = path
        self.size = os.path.getsize(path)
        self.file = open(path, "rb")
        head = self.file.read(8)
        if len(head) < 8:
            self.file.close()
            raise SafetensorsError(f"{path}: file shorter than the 8-byte length prefix")
        (hlen,) = struct.unpack("<Q", head)
        if hlen == 0 or hlen > _MAX_HEADER or 8 + hlen > self.size:
            self.file.close()
            raise SafetensorsError(f"{path}: header length {hlen} runs past the end of the file or is not plausible")
        blob = head + self.file.read(hlen)
        self.records, self.data_start = parse_header(blob, self.size, path)
        self.map = mmap.mmap(self.file.fileno(), 0, access=mmap.ACCESS_READ) if self.size > 0 else None

    def tensor(self, rec: TensorRecord) -> torch.Tensor:
        width, np_dtype, torch_dtype = _DTYPES[rec.dtype]
        count = (rec.end - rec.begin) // width
        arr = np.frombuffer(self.map, dtype=np_dtype, count=count, offset=self.data_start + rec.begin)
        # copy: the result must outlive the mapping and be writable for torch
        t = torch.from_numpy(arr.copy())
        if rec.dtype == "BF16":
            t = t.view(torch.bfloat16)
        return t.reshape(rec.shape)

    def close(self) -> None:
        if self.map is not None:
            self.map.close()
            self.map = None
        self.file.close()


class SafetensorsFolder:
    """All tensors of a model folder under one namespace."""

    INDEX = "model.safetensors.index.json"
    SINGLE = "model.safetensors"

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._shards: Dict[str, _Shard] = {}
        self.records: Dict[str, TensorRecord] = {}
        index_path = os.path.join(model_dir, self.INDEX)
        single_path = os.path.join(model_dir, self.SINGLE)
        if os.path.isfile(index_path):
            self._open_sharded(index_path)
        elif os.path.isfile(single_path):
            sh = self._shard(single_path)
            self.records = dict(sh.records)
        else:
            raise SafetensorsError(f"{model_dir}: neither {self.INDEX} nor {self.SINGLE} found")

    def _shard(self, path: str) -> _Shard:
        if path not in self._shards:
            if not os.path.isfile(path):
                raise SafetensorsError(f"{path}: shard named by the index does not exist")
            self._shards[path] = _Shard(path)
        return self._shards[path]

    def _open_sharded(self, index_path: str) -> None:
        try:
            with open(index_path, "r", encoding="utf-8") as f:
                idx = json.load(f)
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{index_path}: not valid JSON ({e})") from None
        wm = idx.get("weight_map") if isinstance(idx, dict) else None
        if not isinstance(wm, dict) or not wm:
            raise SafetensorsError(f"{index_path}: no 'weight_map' object")
        for name, fname in wm.items():
            if not isinstance(fname, str):
                raise SafetensorsError(f"{index_path}: weight_map['{name}'] is not a file name")
            sh = self._shard(os.path.join(self.model_dir, fname))
            if name not in sh.records:
                raise SafetensorsError(f"{index_path}: tensor '{name}' is mapped to {fname} but is not in it")
            self.records[name] = sh.records[name]
        # a tensor present in two shards is ambiguous even if the index picks one
        seen: Dict[str, str] = {}
        for path, sh in self._shards.items():
            for name in sh.records:
                if name in seen:
                    raise SafetensorsError(f"tensor '{name}' appears in two shards: {seen[name]} and {path}")
                seen[name] = path

    def names(self) -> List[str]:
        return list(self.records)

    def __contains__(self, name: str) -> bool:
        return name in self.records

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.records[name].shape

    def dtype_tag(self, name: str) -> str:
        return self.records[name].dtype

    def tensor(self, name: str) -> torch.Tensor:
        rec = self.records.get(name)
        if rec is None:
            raise SafetensorsError(f"tensor '{name}' not in model")
        return self._shards[rec.shard].tensor(rec)

    def close(self) -> None:
        for sh in self._shards.values():
            sh.close()
        self._shards.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write tensors (CPU, any listed dtype) to one safetensors file, names sorted."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        tag = _TAG_OF_TORCH.get(t.dtype)
        if tag is None:
            raise SafetensorsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": tag, "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - len(blob) % 8) % 8
    blob += b" " * pad
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)
