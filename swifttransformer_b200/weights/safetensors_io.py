"""Reading and writing ``.safetensors`` files by tensor name.

File layout: 8 bytes little-endian header length ``n``, ``n`` bytes of JSON
(``name -> {dtype, shape, data_offsets}`` plus an optional ``__metadata__``),
then the raw little-endian tensor bytes.  Tensors are memory-mapped and handed
out as torch views, so a multi-gigabyte checkpoint is never copied on the host.

The reference stores one TorchScript file per tensor instead
(scripts/lib/converter_lib.py:123-131) and reports a missing file, a wrong
element count or a wrong dtype one tensor at a time
(src/csrc/model/gpt/gpt_weight.cc:193-250).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class TensorInfo:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "path")

    def __init__(self, name, dtype, shape, begin, end, path):
        self.name, self.dtype, self.shape = name, dtype, tuple(shape)
        self.begin, self.end, self.path = begin, end, path


class SafetensorsFile:
    """One memory-mapped ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.tensors: Dict[str, TensorInfo] = {}
        for name, rec in header.items():
            try:
                dt, shape, (b, e) = rec["dtype"], rec["shape"], rec["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for '{name}'") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            numel = 1
            for s in shape:
                numel *= int(s)
            want = numel * _DTYPES[dt].itemsize
            if b < 0 or e < b or e > data_len or e - b != want:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' ({dt} {list(shape)}) claims bytes [{b},{e}) "
                    f"but needs {want} and the file holds {data_len} (truncated file?)")
            self.tensors[name] = TensorInfo(name, _DTYPES[dt], shape, b, e, path)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.tensors)

    def get(self, name: str) -> torch.Tensor:
        """A read-only CPU view of tensor ``name`` (shares the file mapping)."""
        info = self.tensors[name]
        n = info.end - info.begin
        if n == 0:
            return torch.empty(info.shape, dtype=info.dtype)
        buf = memoryview(self._mm)[self._data_start + info.begin:self._data_start + info.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            t = torch.frombuffer(buf, dtype=info.dtype)
        return t.view(info.shape)

    def close(self) -> None:
        # views handed out keep the mapping alive through the buffer protocol
        try:
            self._f.close()
        except Exception:
            pass


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """All ``*.safetensors`` of a model folder (one file, or shards)."""
    if not os.path.isdir(model_dir):
        raise SafetensorsError(f"model folder '{model_dir}' does not exist")
    paths = sorted(p for p in os.listdir(model_dir) if p.endswith(".safetensors"))
    if not paths:
        raise SafetensorsError(f"no .safetensors file in '{model_dir}'")
    return [SafetensorsFile(os.path.join(model_dir, p)) for p in paths]


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata=None) -> None:
    """Write named CPU tensors; data is laid out in the given order, 8-byte aligned header."""
    items = [(n, t.detach().contiguous().cpu()) for n, t in tensors]
    header = {}
    off = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ('{name}')")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
