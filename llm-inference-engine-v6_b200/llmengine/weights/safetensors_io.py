"""Reading and writing safetensors files, by hand.

Format: 8-byte little-endian header length, a JSON header, then the data section; each tensor has
`dtype`, `shape` and `data_offsets` relative to the data section. The reader memory-maps the file
and makes the same checks as the reference's loader (src/weights.cpp:151-242): file shorter than 8
bytes, header running past the file, negative dimension, offsets outside the data section, byte
count not equal to shape x dtype, dtype not one of F32/F16/BF16/I8/I32.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Tuple

import numpy as np
import torch


class SafetensorsError(RuntimeError):
    pass


_DTYPES: Dict[str, Tuple[torch.dtype, int]] = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I8": (torch.int8, 1), "I32": (torch.int32, 4),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """Name -> tensor view over a memory-mapped file. Views stay valid while this object lives."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"safetensors file too small: {path}")
        with open(path, "rb") as f:
            self._mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen + 8 > size:
            raise SafetensorsError(f"safetensors header overruns file: {path}")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"safetensors header is not valid JSON: {path}: {e}") from None
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, spec in header.items():
            if name == "__metadata__":
                continue
            try:
                dt, shape, (b, e) = spec["dtype"], tuple(int(d) for d in spec["shape"]), spec["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"safetensors entry malformed for {name}") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"unsupported safetensors dtype {dt} for {name}")
            if any(d < 0 for d in shape):
                raise SafetensorsError(f"safetensors negative shape dim for {name}")
            numel = 1
            for d in shape:
                numel *= d
            expected = numel * _DTYPES[dt][1]
            if e < b or e > data_len or b < 0:
                raise SafetensorsError(f"safetensors offsets out of range for {name}")
            if e - b != expected:
                raise SafetensorsError(f"safetensors byte-count mismatch for {name}: header says shape*dtype = "
                                       f"{expected} bytes but data_offsets cover {e - b}")
            self.entries[name] = (dt, shape, int(b), int(e))

    def names(self) -> List[str]:
        return sorted(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that aliases the mapped file (read-only memory: copy before writing)."""
        dt, shape, b, e = self.entries[name]
        tdt = _DTYPES[dt][0]
        if e == b:
            return torch.empty(shape, dtype=tdt)
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self._data_start + b)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the array is not writable
            t = torch.from_numpy(buf)
        return t.view(tdt).reshape(shape)


def list_safetensors(model_dir: str) -> List[str]:
    """Files ending in .safetensors directly in the folder, sorted (src/weights.cpp:37-51)."""
    if not os.path.isdir(model_dir):
        raise SafetensorsError(f"model folder does not exist: {model_dir}")
    files = sorted(os.path.join(model_dir, f) for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not files:
        raise SafetensorsError(f"no .safetensors files in {model_dir}")
    return files


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    header = {}
    blobs = []
    off = 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot write dtype {t.dtype} of {name}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
