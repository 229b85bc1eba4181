"""Reader and writer of the safetensors container, written for this engine.

The format: eight bytes (little-endian length n of the header), n bytes of JSON
(tensor name -> dtype, shape, data_offsets relative to the end of the header), then the
data.  vt-transformer reads the same container with ``SafeTensorFile``
(vt-transformer/core/safetensors.hpp:80-281: a single file ``open_single`` :159-201, or
shards through ``*.index.json`` ``open_index`` :204-267, ``read_raw`` :125-140); like
it, this reader refuses a header above 1 GiB and a tensor named in two shards.
Tensors are memory-mapped and handed out in the dtype they are stored in.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}
_MAX_HEADER = 1 << 30


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    file: str
    begin: int      # absolute byte offsets in the file
    end: int


def _read_header(path: str) -> Tuple[Dict, int]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: shorter than the 8-byte length of a safetensors header")
        (n,) = struct.unpack("<Q", head)
        if n > _MAX_HEADER or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} is not plausible for a file of {size} bytes")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: the header is not valid JSON: {e}") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: the header is not a JSON object")
    return header, 8 + n


def read_index(path: str) -> Dict[str, TensorEntry]:
    """name -> entry for one safetensors file."""
    header, data_start = _read_header(path)
    size = os.path.getsize(path)
    out: Dict[str, TensorEntry] = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype = _DTYPES[info["dtype"]]
            shape = tuple(int(s) for s in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: tensor '{name}' has a malformed or unknown entry {info!r}") from None
        numel = 1
        for s in shape:
            numel *= s
        if e - b != numel * dtype.itemsize or b < 0 or data_start + e > size:
            raise SafetensorsError(f"{path}: tensor '{name}' of shape {list(shape)} and dtype {info['dtype']} "
                                   f"does not fit its bytes [{b}, {e}) in a file of {size} bytes")
        out[name] = TensorEntry(name, dtype, shape, path, data_start + b, data_start + e)
    return out


def index_folder(folder: str) -> Dict[str, TensorEntry]:
    """name -> entry for a model folder: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` lists."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(single):
        return read_index(single)
    if os.path.isfile(index):
        with open(index) as f:
            try:
                weight_map = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise SafetensorsError(f"{index}: not a shard index (no 'weight_map')") from None
        out: Dict[str, TensorEntry] = {}
        for shard in sorted(set(weight_map.values())):
            part = read_index(os.path.join(folder, shard))
            for name, entry in part.items():
                if name in out:
                    raise SafetensorsError(f"{folder}: tensor '{name}' is stored in two shards")
                out[name] = entry
        return out
    raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json is there")


class MappedFiles:
    """Memory maps of safetensors files, opened when a tensor is first read."""

    def __init__(self):
        self._maps: Dict[str, mmap.mmap] = {}

    def tensor(self, entry: TensorEntry) -> torch.Tensor:
        mm = self._maps.get(entry.file)
        if mm is None:
            with open(entry.file, "rb") as f:
                mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)   # private pages: torch wants writable memory
            self._maps[entry.file] = mm
        if entry.end == entry.begin:
            return torch.empty(entry.shape, dtype=entry.dtype)
        flat = torch.frombuffer(mm, dtype=entry.dtype, count=(entry.end - entry.begin) // entry.dtype.itemsize,
                                offset=entry.begin)
        return flat.view(entry.shape)

    def close(self) -> None:
        self._maps.clear()


def write_file(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], layout: List[Tuple[str, torch.dtype, Tuple[int, ...]]],
               metadata: Dict[str, str] = None) -> None:
    """Writes ``layout`` (name, dtype, shape in file order) and then the tensors that the
    iterable yields in the same order, one at a time."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, dtype, shape in layout:
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * dtype.itemsize
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        expected = iter(layout)
        for name, t in tensors:
            want_name, want_dtype, want_shape = next(expected)
            if name != want_name or t.dtype != want_dtype or tuple(t.shape) != tuple(want_shape):
                raise SafetensorsError(f"write_file: got '{name}' {t.dtype} {list(t.shape)} where the layout has "
                                       f"'{want_name}' {want_dtype} {list(want_shape)}")
            t = t.detach().cpu().contiguous()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() < (1 << 24)
                        else memoryview(t.view(torch.uint8).numpy()))
        if next(expected, None) is not None:
            raise SafetensorsError("write_file: fewer tensors than the layout lists")
    os.replace(tmp, path)
