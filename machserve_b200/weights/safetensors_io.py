"""Reading and writing the safetensors container, without any library for it.

Format, as the reference parses it (crates/mach-model/src/loader.rs:141-188,
:289-314 of gqf2008/machserve): eight bytes of little-endian header length, a
JSON object {name: {dtype, shape, data_offsets}} (the `__metadata__` entry is
skipped), then raw little-endian data; offsets are relative to the data section.
The same checks are made: header length within the file and at most 64 MiB,
offsets inside the data section and of the size the shape and dtype give, no
name twice.  A folder may hold several `*.safetensors` shards; they are read in
sorted order and a name may appear in one only (:877-910).
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

MAX_HEADER_BYTES = 64 << 20

# container dtype -> (bytes per element, numpy dtype to view the bytes as, torch dtype of that view)
_DTYPES = {
    "F32": (4, "<f4", torch.float32),
    "F16": (2, "<f2", torch.float16),
    "BF16": (2, "<u2", torch.bfloat16),
    "F64": (8, "<f8", torch.float64),
    "I64": (8, "<i8", torch.int64),
    "I32": (4, "<i4", torch.int32),
    "I16": (2, "<i2", torch.int16),
    "I8": (1, "i1", torch.int8),
    "U8": (1, "u1", torch.uint8),
    "BOOL": (1, "u1", torch.bool),
}
_TORCH_TO_NAME = {
    torch.float32: "F32",
    torch.float16: "F16",
    torch.bfloat16: "BF16",
    torch.float64: "F64",
    torch.int64: "I64",
    torch.int32: "I32",
    torch.int16: "I16",
    torch.int8: "I8",
    torch.uint8: "U8",
    torch.bool: "BOOL",
}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


def _no_duplicates(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise SafetensorsError(f"tensor name '{k}' appears twice in the header")
        seen[k] = v
    return seen


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name, dtype, shape, begin, end, file):
        self.name, self.dtype, self.shape, self.begin, self.end, self.file = name, dtype, shape, begin, end, file


class SafetensorsFile:
    """One memory-mapped file.  `entries` maps names to where their bytes lie."""

    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to hold a header length ({size} bytes)")
        self._fh = open(self.path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen > MAX_HEADER_BYTES:
            raise SafetensorsError(f"{self.path}: header of {hlen} bytes is larger than {MAX_HEADER_BYTES}")
        if 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: header of {hlen} bytes runs past the end of the file ({size} bytes)")
        try:
            header = json.loads(self._map[8 : 8 + hlen].decode("utf-8"), object_pairs_hook=_no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header must be a JSON object")
        self.data_start = 8 + hlen
        data_len = size - self.data_start
        self.entries: Dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (begin, end) = meta["dtype"], list(meta["shape"]), meta["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: entry '{name}' lacks dtype, shape or data_offsets") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has unsupported dtype {dtype}")
            if any((not isinstance(d, int)) or d < 0 for d in shape):
                raise SafetensorsError(f"{self.path}: tensor '{name}' has a bad shape {shape}")
            want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dtype][0] if shape else _DTYPES[dtype][0]
            if not (isinstance(begin, int) and isinstance(end, int) and 0 <= begin <= end <= data_len):
                raise SafetensorsError(
                    f"{self.path}: tensor '{name}' has offsets [{begin}, {end}) outside the data section of {data_len} bytes"
                )
            if end - begin != want:
                raise SafetensorsError(
                    f"{self.path}: tensor '{name}' of shape {shape} and dtype {dtype} needs {want} bytes, "
                    f"its offsets give {end - begin}"
                )
            self.entries[name] = TensorEntry(name, dtype, tuple(shape), begin, end, self)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor with the stored dtype, copied out of the map."""
        e = self.entries[name]
        _, np_dtype, t_dtype = _DTYPES[e.dtype]
        raw = np.frombuffer(self._map, dtype=np.uint8, count=e.end - e.begin, offset=self.data_start + e.begin)
        arr = raw.view(np_dtype).reshape(e.shape).copy()
        if e.dtype == "BF16":
            return torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16)
        if e.dtype == "BOOL":
            return torch.from_numpy(arr).to(torch.bool)
        return torch.from_numpy(arr)

    def close(self):
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass
        self._fh.close()


INDEX_NAME = "model.safetensors.index.json"


def read_shard_index(folder: Path) -> Optional[Tuple[Dict[str, str], Optional[int]]]:
    """(tensor name -> shard file name, the total size it states or None) from a folder's
    `model.safetensors.index.json`, or None if there is none.
    A shard must be a `.safetensors` file that lies in the folder itself (no path may lead out of it) and exists
    (crates/mach-model/src/loader.rs:327-384 of gqf2008/machserve)."""
    path = folder / INDEX_NAME
    if not path.is_file():
        return None
    try:
        raw = json.loads(path.read_text())
    except (OSError, ValueError) as e:
        raise SafetensorsError(f"{path}: cannot be read as JSON: {e}") from None
    weight_map = raw.get("weight_map") if isinstance(raw, dict) else None
    if not isinstance(weight_map, dict):
        raise SafetensorsError(f"{path}: 'weight_map' is missing or is not an object")
    out = {}
    for name, shard in weight_map.items():
        if not isinstance(shard, str) or not shard.endswith(".safetensors") or Path(shard).name != shard or shard in (".", ".."):
            raise SafetensorsError(f"{path}: weight_map['{name}'] must name a .safetensors file of this folder, found {shard!r}")
        if not (folder / shard).is_file():
            raise SafetensorsError(f"{path}: the shard {shard} that it names is missing")
        out[name] = shard
    total = raw.get("metadata", {}).get("total_size") if isinstance(raw.get("metadata"), dict) else None
    if total is not None and (isinstance(total, bool) or not isinstance(total, (int, float)) or total < 0 or total != int(total)):
        raise SafetensorsError(f"{path}: metadata.total_size must be a non-negative integer, found {total!r}")
    return out, (None if total is None else int(total))


def open_model_files(model_dir) -> Tuple[Dict[str, TensorEntry], List[SafetensorsFile]]:
    """All tensors of a folder's `*.safetensors` files (or of one file), by name.  With an index file in the
    folder, the shards are those it names and every tensor must lie where it says: a shard that the index does
    not know, a tensor that the index does not know or places elsewhere, an indexed tensor that no shard holds, or
    a total size that differs from the shards' payload is an error (crates/mach-model/src/loader.rs:390-502)."""
    p = Path(model_dir)
    index, total_size = (None if p.is_file() else read_shard_index(p)) or (None, None)
    if index is not None:
        named = sorted(set(index.values()))
        stray = sorted(f.name for f in p.glob("*.safetensors") if f.name not in named)
        if stray:
            raise SafetensorsError(f"{p}: files that {INDEX_NAME} does not name: {', '.join(stray)}")
        paths = [p / n for n in named]
    else:
        paths = [p] if p.is_file() else sorted(p.glob("*.safetensors"))
    if not paths:
        raise SafetensorsError(f"{p}: no *.safetensors file found")
    files, entries = [], {}
    try:
        for path in paths:
            f = SafetensorsFile(path)
            files.append(f)
            for name, e in f.entries.items():
                if name in entries:
                    raise SafetensorsError(f"tensor '{name}' is in both {entries[name].file.path.name} and {path.name}")
                if index is not None and index.get(name) != path.name:
                    where = f"is indexed in {index[name]}" if name in index else "is absent from the index"
                    raise SafetensorsError(f"{path.name}: tensor '{name}' {where}")
                entries[name] = e
        if index is not None:
            lost = sorted(n for n in index if n not in entries)
            if lost:
                raise SafetensorsError(f"{p / INDEX_NAME}: indexed tensors that no shard holds: {', '.join(lost[:8])}")
            payload = sum(e.end - e.begin for e in entries.values())
            if total_size is not None and payload != total_size:
                raise SafetensorsError(f"{p / INDEX_NAME}: metadata.total_size is {total_size}, the shards hold {payload} bytes")
    except SafetensorsError:
        for f in files:
            f.close()
        raise
    return entries, files


def write_safetensors(path, tensors: Dict[str, torch.Tensor] | Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Writes CPU tensors under their names, in the order given."""
    items = list(tensors.items()) if isinstance(tensors, dict) else list(tensors)
    header, offset = {}, 0
    for name, t in items:
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for _, t in items:
            c = t.detach().contiguous().cpu()
            if c.dtype == torch.bfloat16:
                c = c.view(torch.int16)
            elif c.dtype == torch.bool:
                c = c.to(torch.uint8)
            fh.write(c.numpy().tobytes())
