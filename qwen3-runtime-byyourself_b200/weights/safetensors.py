"""Reading and writing the safetensors container, and a model folder made of it.

Format: 8-byte little-endian header length, a JSON header (name -> dtype, shape,
data_offsets relative to the end of the header), then the raw little-endian data.

Parity with the reference (RicardoMin/Qwen3-Runtime-ByYourself):
  header checks   src/io/safetensors_file.cpp:31-74 (length <= 100,000,000, starts with '{')
  metadata checks src/io/safetensors_metadata.cpp:64-168 (dtypes BF16/F32/I32, offsets
                  inside the data, shape x dtype == byte count, `__metadata__` skipped)
  model folder    src/io/safetensors_checkpoint.cpp:126-155 (model.safetensors xor
                  model.safetensors.index.json), :182-286 (index and shards checked both
                  ways, total_size), :91-110 (shard names are plain files of the folder)
The reference maps files with mmap and uploads through pinned staging
(src/io/safetensors_loader.cpp:141-248); here the file is mapped, each tensor is a
zero-copy view of the mapping and torch does the upload.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Optional

import numpy as np
import torch

MAX_HEADER_BYTES = 100_000_000

_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F32": (torch.float32, 4),
    "I32": (torch.int32, 4),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFormatError(ValueError):
    """The file is not a well-formed safetensors container of supported dtypes."""


class TensorInfo:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name, dtype, shape, begin, end, file):
        self.name, self.dtype, self.shape, self.begin, self.end, self.file = name, dtype, shape, begin, end, file


class SafetensorsFile:
    """One mapped .safetensors file; `tensor(name)` is a CPU view of the mapping."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as e:
            raise SafetensorsFormatError(f"cannot open {path}: {e}") from None
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsFormatError(f"{path}: shorter than the 8-byte header length")
        (header_len,) = struct.unpack("<Q", self._fh.read(8))
        if header_len > MAX_HEADER_BYTES or 8 + header_len > size:
            raise SafetensorsFormatError(f"{path}: header length {header_len} is not plausible")
        raw = self._fh.read(header_len)
        if not raw.startswith(b"{"):
            raise SafetensorsFormatError(f"{path}: header does not start with '{{'")
        try:
            header = json.loads(raw.decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsFormatError(f"{path}: header is not JSON: {e}") from None
        self.data_start = 8 + header_len
        data_size = size - self.data_start
        self.metadata = header.pop("__metadata__", None)
        self.tensors: Dict[str, TensorInfo] = {}
        for name, entry in header.items():
            try:
                dtype_name, shape, (begin, end) = entry["dtype"], entry["shape"], entry["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsFormatError(f"{path}: malformed entry for {name!r}") from None
            if dtype_name not in _DTYPES:
                raise SafetensorsFormatError(
                    f"{path}: tensor {name!r} has dtype {dtype_name}; supported: {sorted(_DTYPES)}")
            dtype, item = _DTYPES[dtype_name]
            if not all(isinstance(s, int) and s >= 0 for s in shape):
                raise SafetensorsFormatError(f"{path}: tensor {name!r} has a bad shape {shape}")
            numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if not (0 <= begin <= end <= data_size) or end - begin != numel * item:
                raise SafetensorsFormatError(
                    f"{path}: tensor {name!r} claims bytes [{begin},{end}) for shape {shape} {dtype_name} "
                    f"in a data section of {data_size} bytes")
            self.tensors[name] = TensorInfo(name, dtype, tuple(shape), begin, end, self)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY) if size else None

    def tensor(self, name: str) -> torch.Tensor:
        info = self.tensors[name]
        count = int(np.prod(info.shape, dtype=np.int64)) if info.shape else 1
        if count == 0:
            return torch.empty(info.shape, dtype=info.dtype)
        flat = torch.frombuffer(self._map, dtype=info.dtype, count=count, offset=self.data_start + info.begin)
        return flat.view(info.shape)

    def close(self):
        # Views handed out keep the mapping alive; closing is left to the garbage collector.
        self._fh.close()


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> int:
    """Write `tensors` (CPU or device, bfloat16/float32/int32) to `path`; returns the data bytes."""
    header = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsFormatError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-(8 + len(raw)) % 16)  # the data section starts on a 16-byte boundary
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in tensors.values():
            c = t.detach().to("cpu").contiguous()
            f.write(c.view(torch.uint8).numpy().tobytes() if c.numel() else b"")
    return offset


SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"


def _check_shard_name(name) -> str:
    if (not isinstance(name, str) or not name.endswith(".safetensors") or name in (".safetensors",)
            or "/" in name or "\\" in name or name.startswith(".") or os.path.basename(name) != name):
        raise SafetensorsFormatError(f"shard name {name!r} is not a plain .safetensors file of the model folder")
    return name


class Checkpoint:
    """A model folder: one `model.safetensors`, or an index with its shards."""

    def __init__(self, folder: str):
        self.folder = folder
        single = os.path.join(folder, SINGLE_FILE)
        index = os.path.join(folder, INDEX_FILE)
        has_single, has_index = os.path.isfile(single), os.path.isfile(index)
        if has_single and has_index:
            raise SafetensorsFormatError(f"{folder}: both {SINGLE_FILE} and {INDEX_FILE} exist; keep one")
        if not has_single and not has_index:
            raise SafetensorsFormatError(f"{folder}: neither {SINGLE_FILE} nor {INDEX_FILE} found")
        self.files: Dict[str, SafetensorsFile] = {}
        self.tensors: Dict[str, TensorInfo] = {}
        if has_single:
            f = SafetensorsFile(single)
            self.files[SINGLE_FILE] = f
            self.tensors = dict(f.tensors)
            return
        try:
            with open(index, "r", encoding="utf-8") as fh:
                root = json.load(fh)
            weight_map = root["weight_map"]
            assert isinstance(weight_map, dict)
        except (OSError, json.JSONDecodeError, KeyError, AssertionError, TypeError) as e:
            raise SafetensorsFormatError(f"{index}: not a usable index: {e}") from None
        for shard in sorted({_check_shard_name(s) for s in weight_map.values()}):
            path = os.path.join(folder, shard)
            if not os.path.isfile(path):
                raise SafetensorsFormatError(f"{folder}: shard {shard} named by the index is missing")
            self.files[shard] = SafetensorsFile(path)
        for name, shard in weight_map.items():
            if name not in self.files[shard].tensors:
                raise SafetensorsFormatError(f"{index}: {name!r} is not in shard {shard}")
            self.tensors[name] = self.files[shard].tensors[name]
        for shard, f in self.files.items():
            for name in f.tensors:
                if weight_map.get(name) != shard:
                    raise SafetensorsFormatError(f"{folder}: shard {shard} holds {name!r}, which the index does not map there")
        total = (root.get("metadata") or {}).get("total_size")
        if total is not None:
            actual = sum(t.end - t.begin for t in self.tensors.values())
            if total != actual:
                raise SafetensorsFormatError(f"{index}: total_size {total} != {actual} bytes in the shards")

    def names(self) -> Iterable[str]:
        return self.tensors.keys()

    def tensor(self, name: str) -> torch.Tensor:
        info = self.tensors.get(name)
        if info is None:
            raise KeyError(f"checkpoint tensor not found: {name}")
        return info.file.tensor(name)
