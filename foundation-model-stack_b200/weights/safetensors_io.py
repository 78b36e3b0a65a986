"""Reading and writing safetensors files by tensor name.

The format: 8 bytes little-endian header length N, N bytes of JSON mapping each name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the header), then the
raw little-endian data.  The reader maps the file into memory and materialises a tensor only when it is
asked for, as the reference's lazy loader does (fms/utils/serialization.py:319-336).
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    def __init__(self, path: str) -> None:
        self.path = path
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{path}: shorter than a safetensors header")
            (n,) = struct.unpack("<Q", head)
            if n <= 0 or 8 + n > size:
                raise SafetensorsError(f"{path}: header length {n} does not fit the file's {size} bytes")
            try:
                header = json.loads(f.read(n).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._data_start = 8 + n
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            if e["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {e['dtype']}")
            begin, end = e["data_offsets"]
            dtype = _DTYPES[e["dtype"]]
            shape = tuple(int(s) for s in e["shape"])
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * torch.empty((), dtype=dtype).element_size() or self._data_start + end > size:
                raise SafetensorsError(f"{path}: tensor {name} has inconsistent offsets")
            self.entries[name] = (dtype, shape, begin, end)
        self._mm = None

    def keys(self) -> List[str]:
        return list(self.entries)

    def spec(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def get(self, name: str) -> torch.Tensor:
        """A tensor that reads from the mapped file; copy it (``.to``) before the file object goes away."""
        dtype, shape, begin, end = self.entries[name]
        if self._mm is None:
            with open(self.path, "rb") as f:
                self._mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        count = (end - begin) // torch.empty((), dtype=dtype).element_size()
        t = torch.frombuffer(self._mm, dtype=dtype, count=count, offset=self._data_start + begin)
        return t.view(shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name} has unsupported dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def find_checkpoint_files(model_path: str) -> List[str]:
    """A file, a glob, or a folder whose ``*.safetensors`` are the shards of one checkpoint
    (``consolidated.safetensors`` is skipped as the reference does, fms/utils/serialization.py:390-411)."""
    if os.path.isfile(model_path):
        return [model_path]
    if os.path.isdir(model_path):
        files = sorted(glob.glob(os.path.join(model_path, "*.safetensors")))
        files = [f for f in files if os.path.basename(f) != "consolidated.safetensors"]
    else:
        files = sorted(glob.glob(model_path))
    if not files:
        raise FileNotFoundError(f"Can't find the requested checkpoint data at {model_path}")
    return files
