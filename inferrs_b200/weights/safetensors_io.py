"""Reading and writing the safetensors container.

The file is: an unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` and the raw
little-endian tensor bytes.  Files are memory-mapped; a tensor's bytes are only
touched when it is asked for (the reference maps its weight files the same way,
candle-core/src/safetensors.rs:454-480).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

# safetensors dtype string -> (torch dtype, numpy dtype used to map the bytes, bytes per element)
_DTYPES = {
    "F32": (torch.float32, np.dtype("<f4"), 4),
    "F16": (torch.float16, np.dtype("<f2"), 2),
    "BF16": (torch.bfloat16, np.dtype("<i2"), 2),
    "F64": (torch.float64, np.dtype("<f8"), 8),
    "I64": (torch.int64, np.dtype("<i8"), 8),
    "I32": (torch.int32, np.dtype("<i4"), 4),
    "I16": (torch.int16, np.dtype("<i2"), 2),
    "I8": (torch.int8, np.dtype("i1"), 1),
    "U8": (torch.uint8, np.dtype("u1"), 1),
    "BOOL": (torch.bool, np.dtype("u1"), 1),
}
_TORCH_TO_NAME = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int
    path: str


class SafetensorsFile:
    """One mapped file; ``info`` lists its tensors, ``read`` gives one as a torch tensor."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        self._data_start = 8 + hlen
        self.metadata = header.pop("__metadata__", {}) or {}
        self.info: Dict[str, TensorInfo] = {}
        for name, d in header.items():
            try:
                dtype, shape, (b, e) = d["dtype"], tuple(int(x) for x in d["shape"]), d["data_offsets"]
            except (KeyError, TypeError, ValueError) as err:
                raise SafetensorsError(f"{path}: malformed entry for tensor '{name}': {d!r}") from err
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype}")
            n = 1
            for s in shape:
                n *= s
            if e - b != n * _DTYPES[dtype][2] or b < 0 or self._data_start + e > size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' ({dtype}{list(shape)}) does not fit its byte range [{b}, {e})")
            self.info[name] = TensorInfo(name, dtype, shape, b, e, path)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def read(self, name: str, private: bool = True) -> torch.Tensor:
        """The tensor, in its stored dtype, on the CPU: a private copy, or (``private=False``) a read-only view of
        the mapped file for a caller that copies it elsewhere at once and drops the view before the file is
        closed."""
        ti = self.info[name]
        tdt, ndt, _ = _DTYPES[ti.dtype]
        n = 1
        for s in ti.shape:
            n *= s
        arr = np.frombuffer(self._mm, dtype=ndt, count=n, offset=self._data_start + ti.begin)
        if private:
            t = torch.from_numpy(arr.copy())
        else:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")       # torch warns that the array cannot be written to: nobody writes
                t = torch.from_numpy(arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        elif tdt == torch.bool:
            t = t.to(torch.bool)
        return t.reshape(ti.shape)

    def close(self):
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:      # a view from read(private=False) is still alive: the mapping goes when it does
                pass
            self._mm = None
        self._f.close()


def _raw_bytes(name: str, t: torch.Tensor) -> bytes:
    if t.dtype not in _TORCH_TO_NAME:
        raise SafetensorsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
    t = t.detach().to("cpu").contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    if t.dtype == torch.bool:
        return t.to(torch.uint8).numpy().tobytes()
    return t.numpy().tobytes()


def write_safetensors_streamed(path: str, entries, metadata: Dict[str, str] = None):
    """Write tensors that are made one at a time: ``entries`` is a list of (name, shape, dtype, make), where
    ``make()`` returns the tensor when its turn has come.  Only one tensor is held at a time, so a model larger
    than the host's memory can be written.  The data section starts on an 8-byte boundary."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, shape, dtype, _ in entries:
        if dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"cannot store tensor '{name}' of dtype {dtype}")
        n = 1
        for d in shape:
            n *= int(d)
        size = n * _DTYPES[_TORCH_TO_NAME[dtype]][2]
        header[name] = {"dtype": _TORCH_TO_NAME[dtype], "shape": [int(d) for d in shape],
                        "data_offsets": [offset, offset + size]}
        offset += size
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for name, shape, dtype, make in entries:
            t = make()
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise SafetensorsError(f"tensor '{name}' was announced as {dtype} {tuple(shape)} and came as "
                                       f"{t.dtype} {tuple(t.shape)}")
            raw = _raw_bytes(name, t)
            lo, hi = header[name]["data_offsets"]
            if len(raw) != hi - lo:
                raise SafetensorsError(f"tensor '{name}': {len(raw)} bytes where {hi - lo} were announced")
            f.write(raw)
    os.replace(tmp, path)


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Dict[str, str] = None):
    """Write tensors in the order given; the data section starts on an 8-byte boundary."""
    entries = [(name, tuple(t.shape), t.dtype, (lambda t=t: t)) for name, t in tensors]
    write_safetensors_streamed(path, entries, metadata)
