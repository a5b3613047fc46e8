"""Reading and writing the safetensors container, by tensor name.

The format is small: eight bytes (little-endian) with the length of a JSON header,
the header mapping each tensor name to ``{"dtype", "shape", "data_offsets"}``, then
the raw little-endian data.  The reference has no reader of its own (it goes through
a model library, worker/src/inference/torch_engine.py:135-147); this one maps the
file and hands out tensors without copying until they are converted or moved.

A model folder holds either ``model.safetensors`` or ``model.safetensors.index.json``
whose ``weight_map`` names the shard of every tensor.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Iterable, Mapping

import numpy as np
import torch

_NUMPY_OF = {
    "F64": np.float64,
    "F32": np.float32,
    "F16": np.float16,
    "BF16": np.uint16,  # viewed as bfloat16 afterwards
    "I64": np.int64,
    "I32": np.int32,
    "I16": np.int16,
    "I8": np.int8,
    "U8": np.uint8,
    "BOOL": np.bool_,
}
_TORCH_OF = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAME_OF = {v: k for k, v in _TORCH_OF.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped ``.safetensors`` file."""

    def __init__(self, path: str) -> None:
        self.path = path
        with open(path, "rb") as handle:
            head = handle.read(8)
            if len(head) != 8:
                raise SafetensorsError(f"{path}: too short to be a safetensors file")
            (length,) = struct.unpack("<Q", head)
            size = os.fstat(handle.fileno()).st_size
            if length > size - 8:
                raise SafetensorsError(f"{path}: header length {length} exceeds the file")
            try:
                header = json.loads(handle.read(length).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as exc:
                raise SafetensorsError(f"{path}: header is not JSON") from exc
            self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        self.metadata: Mapping[str, str] = header.pop("__metadata__", {}) or {}
        self._entries: dict[str, dict] = header
        self._base = 8 + length
        for name, entry in header.items():
            begin, end = entry["data_offsets"]
            if entry["dtype"] not in _TORCH_OF:
                raise SafetensorsError(f"{path}: tensor {name!r} has unknown dtype {entry['dtype']}")
            count = int(np.prod(entry["shape"], dtype=np.int64)) if entry["shape"] else 1
            width = torch.empty((), dtype=_TORCH_OF[entry["dtype"]]).element_size()
            if end - begin != count * width or self._base + end > size:
                raise SafetensorsError(f"{path}: tensor {name!r} has inconsistent offsets")

    def keys(self) -> Iterable[str]:
        return self._entries.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self._entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _TORCH_OF[self._entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only: convert or copy before writing)."""
        entry = self._entries[name]
        begin, _ = entry["data_offsets"]
        shape = tuple(entry["shape"])
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if count == 0:
            return torch.empty(shape, dtype=_TORCH_OF[entry["dtype"]])
        array = np.frombuffer(self._map, dtype=_NUMPY_OF[entry["dtype"]], count=count, offset=self._base + begin)
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the mapped array is not writable
            flat = torch.from_numpy(array)
        if entry["dtype"] == "BF16":
            flat = flat.view(torch.bfloat16)
        return flat.reshape(shape)


class ModelTensors:
    """All tensors of a model folder, whichever shard they live in."""

    def __init__(self, folder: str) -> None:
        self.folder = folder
        single = os.path.join(folder, "model.safetensors")
        index = os.path.join(folder, "model.safetensors.index.json")
        self._where: dict[str, SafetensorsFile] = {}
        if os.path.exists(index):
            with open(index, "r", encoding="utf-8") as handle:
                weight_map = json.load(handle)["weight_map"]
            files: dict[str, SafetensorsFile] = {}
            for name, shard in weight_map.items():
                if shard not in files:
                    files[shard] = SafetensorsFile(os.path.join(folder, shard))
                if name not in files[shard]:
                    raise SafetensorsError(f"{index}: {name!r} is not in shard {shard}")
                self._where[name] = files[shard]
        elif os.path.exists(single):
            handle = SafetensorsFile(single)
            self._where = {name: handle for name in handle.keys()}
        else:
            raise FileNotFoundError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")

    def keys(self):
        return self._where.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str) -> tuple[int, ...]:
        return self._where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._where[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)


def save_file(tensors: Mapping[str, torch.Tensor], path: str, metadata: Mapping[str, str] | None = None) -> None:
    """Write tensors (CPU, any listed dtype) under their names, sorted, 8-byte aligned header."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        tensor = tensors[name]
        if tensor.dtype not in _NAME_OF:
            raise SafetensorsError(f"cannot store {name!r} of dtype {tensor.dtype}")
        size = tensor.numel() * tensor.element_size()
        header[name] = {
            "dtype": _NAME_OF[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + size],
        }
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name in order:
            tensor = tensors[name].detach().contiguous().cpu()
            if tensor.numel() == 0:
                continue
            raw = tensor.view(torch.uint8) if tensor.dtype != torch.bool else tensor.to(torch.uint8)
            handle.write(raw.reshape(-1).numpy().tobytes())
    os.replace(tmp, path)
