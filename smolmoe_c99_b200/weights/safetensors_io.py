"""Reading and writing the safetensors container: an 8-byte little-endian header length,
a JSON header ``{name: {dtype, shape, data_offsets}}`` and the raw tensor bytes.

The reference reads the same container in its converter and checks the same things:
header length, JSON, dtype, shape, byte extents, overlap (scripts/hf/safetensors.ts:54-111);
its run-time counterpart is the sorted tensor directory of src/modelfile.c:47-87.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "F64": (torch.float64, 8),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int  # byte offsets into the file
    end: int


class SafetensorsFile:
    """One mapped file; tensors are views of the mapping until they are copied."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._file = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: {e.strerror or e}") from None
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        if header_len > _MAX_HEADER or 8 + header_len > size:
            raise SafetensorsError(f"{path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        data_start = 8 + header_len
        self.entries: Dict[str, TensorEntry] = {}
        extents: List[Tuple[int, int, str]] = []
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype_name, shape, (begin, end) = info["dtype"], info["shape"], info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor {name}") from None
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {dtype_name}")
            dtype, width = _DTYPES[dtype_name]
            if not isinstance(shape, list) or any(isinstance(d, bool) or not isinstance(d, int) or d < 0 for d in shape):
                raise SafetensorsError(f"{path}: tensor {name} has a malformed shape")
            count = 1
            for d in shape:
                count *= d
            if not (isinstance(begin, int) and isinstance(end, int)) or begin < 0 or end - begin != count * width:
                raise SafetensorsError(f"{path}: tensor {name}: byte extent does not match shape and dtype")
            if data_start + end > size:
                raise SafetensorsError(f"{path}: tensor {name} reaches past the end of the file (truncated?)")
            self.entries[name] = TensorEntry(name, dtype, tuple(shape), data_start + begin, data_start + end)
            if end > begin:
                extents.append((begin, end, name))
        extents.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(extents, extents[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{path}: tensors {n0} and {n1} overlap")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapping (read-only memory: copy before writing)."""
        e = self.entries[name]
        count = 1
        for d in e.shape:
            count *= d
        if count == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)  # the mapping is read-only; nobody writes to it
            flat = torch.frombuffer(self._map, dtype=e.dtype, count=count, offset=e.begin)
        return flat.view(e.shape)

    def close(self) -> None:
        # tensors handed out keep the mapping alive through the buffer protocol
        self._file.close()


def open_checkpoint(model_dir: str) -> Dict[str, Tuple[SafetensorsFile, TensorEntry]]:
    """All tensors of a model folder: ``model.safetensors``, or the shards listed in
    ``model.safetensors.index.json`` (scripts/hf/safetensors.ts:113-149)."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    files: List[str] = []
    if os.path.exists(single):
        files = [single]
    elif os.path.exists(index):
        with open(index, "r", encoding="utf-8") as f:
            try:
                weight_map = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise SafetensorsError(f"{index}: no weight_map") from None
        files = sorted({os.path.join(model_dir, v) for v in weight_map.values()})
    else:
        raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")
    out: Dict[str, Tuple[SafetensorsFile, TensorEntry]] = {}
    for path in files:
        st = SafetensorsFile(path)
        for name, entry in st.entries.items():
            if name in out:
                raise SafetensorsError(f"tensor {name} appears in {out[name][0].path} and in {path}")
            out[name] = (st, entry)
    return out


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Writes CPU tensors in sorted name order; the file is complete or absent (written
    beside the target, then renamed, like the reference's writers: src/prefixcache.c:129-154)."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-(8 + len(blob)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
