"""safetensors container: reader (single file or sharded folder) and writer.

The container code is C++ (``csrc/host/safetensors.cpp``, in the host runtime library); this module is its Python
face and turns the bytes it reads into torch tensors.  Format and checks follow the reference's container code: an
8-byte little-endian header length, a JSON object ``{name: {dtype, shape, data_offsets}}`` with ``__metadata__``
skipped, offsets relative to the data region, byte length equal to ``prod(shape) * width``, ``begin <= end``, no
negative dimension, no region past the file (src/core/safetensors/SafetensorsHeader.cpp:33-153); a folder holds
either a shard index ``model.safetensors.index.json`` with a ``weight_map`` or a single ``model.safetensors``
(src/core/safetensors/SafetensorsModel.cpp:32-56), every mapped tensor must exist in its shard and no tensor may
appear in two shards (:100-129).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..cache import host


class SafetensorsError(ValueError):
    pass


# dtype tag → torch dtype (bfloat16 travels as its 16 bits)
_TORCH_OF_TAG = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
    "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_TAG_OF_TORCH = {v: k for k, v in _TORCH_OF_TAG.items()}


@dataclass(frozen=True)
class TensorRecord:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int  # byte offsets inside the data region
    end: int
    shard: str  # file path


def _records(lib, h) -> Dict[str, TensorRecord]:
    out: Dict[str, TensorRecord] = {}
    dims = (ctypes.c_longlong * 16)()
    for i in range(lib.mmh_st_count(h)):
        nd = lib.mmh_st_shape(h, i, dims, 16)
        if nd > 16:
            raise SafetensorsError(f"tensor '{lib.mmh_st_name(h, i).decode()}' has more than 16 dimensions")
        name = lib.mmh_st_name(h, i).decode("utf-8")
        out[name] = TensorRecord(name, lib.mmh_st_dtype(h, i).decode(), tuple(int(dims[k]) for k in range(nd)),
                                 int(lib.mmh_st_offset(h, i, 0)), int(lib.mmh_st_offset(h, i, 1)), lib.mmh_st_shard(h, i).decode("utf-8"))
    return out


def parse_header(blob: bytes, file_size: int, where: str) -> Tuple[Dict[str, TensorRecord], int]:
    """Parse the first bytes of a safetensors file. Returns (records, data region start)."""
    lib = host.load()
    h = lib.mmh_st_parse_header(blob, len(blob), int(file_size), where.encode("utf-8"))
    if not h:
        raise SafetensorsError(host.last_error())
    try:
        records = _records(lib, h)
        # every record of a header alone lies in the same file: its data region starts right after the header
        (hlen,) = __import__("struct").unpack("<Q", blob[:8])
        return records, 8 + hlen
    finally:
        lib.mmh_st_close(h)


class SafetensorsFolder:
    """All tensors of a model folder under one namespace."""

    INDEX = "model.safetensors.index.json"
    SINGLE = "model.safetensors"

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._lib = host.load()
        self._h = self._lib.mmh_st_open_folder(model_dir.encode("utf-8"))
        if not self._h:
            raise SafetensorsError(host.last_error())
        self.records: Dict[str, TensorRecord] = _records(self._lib, self._h)
        self._index = {name: i for i, name in enumerate(self.records)}

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
        if self._h is None:
            raise SafetensorsError("the folder is closed")
        t = torch.empty(rec.shape, dtype=_TORCH_OF_TAG[rec.dtype])
        nbytes = rec.end - rec.begin
        if nbytes and self._lib.mmh_st_read(self._h, self._index[name], t.data_ptr(), nbytes) != 0:
            raise SafetensorsError(host.last_error())
        return t

    def mismatch(self, want: Mapping[str, Tuple[Tuple[int, ...], bool]], where: str) -> Optional[str]:
        """``want``: name -> (shape, may be absent).  None when the folder holds exactly these tensors, else the one
        message that lists every missing tensor, every unexpected one and every wrong shape."""
        names = list(want)
        n = len(names)
        c_names = (ctypes.c_char_p * max(1, n))(*[s.encode("utf-8") for s in names])
        ndims = (ctypes.c_int * max(1, n))(*[len(want[s][0]) for s in names])
        flat = [int(d) for s in names for d in want[s][0]]
        shapes = (ctypes.c_longlong * max(1, len(flat)))(*flat)
        optional = (ctypes.c_int * max(1, n))(*[int(bool(want[s][1])) for s in names])
        if self._lib.mmh_st_check(self._h, where.encode("utf-8"), n, c_names, ndims, shapes, optional) == 0:
            return None
        return host.last_error()

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.mmh_st_close(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write tensors (CPU, any listed dtype) to one safetensors file, names sorted."""
    lib = host.load()
    order = sorted(tensors)
    n = len(order)
    keep = []
    names = (ctypes.c_char_p * max(1, n))()
    dtypes = (ctypes.c_char_p * max(1, n))()
    ndims = (ctypes.c_int * max(1, n))()
    data = (ctypes.c_void_p * max(1, n))()
    nbytes = (ctypes.c_longlong * max(1, n))()
    flat: List[int] = []
    for i, name in enumerate(order):
        t = tensors[name]
        tag = _TAG_OF_TORCH.get(t.dtype)
        if tag is None:
            raise SafetensorsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        c = t.detach().contiguous().cpu()
        keep.append(c)
        names[i], dtypes[i], ndims[i] = name.encode("utf-8"), tag.encode(), c.dim()
        data[i], nbytes[i] = c.data_ptr(), c.numel() * c.element_size()
        flat.extend(int(d) for d in c.shape)
    shapes = (ctypes.c_longlong * max(1, len(flat)))(*flat)
    meta_items = [str(x).encode("utf-8") for kv in (metadata or {}).items() for x in kv]
    meta = (ctypes.c_char_p * max(1, len(meta_items)))(*meta_items)
    if lib.mmh_st_write(path.encode("utf-8"), n, names, dtypes, ndims, shapes, data, nbytes, len(meta_items) // 2, meta) != 0:
        raise SafetensorsError(host.last_error())
