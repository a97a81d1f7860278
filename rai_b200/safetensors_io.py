"""Host-side view of .safetensors files through the library's reader (rb_safetensors_*), plus a writer
for the same format.  The reader is what rb_model_load_safetensors uses; it needs no GPU."""
from __future__ import annotations

import ctypes
import json
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import _lib

_DTYPE_TAG = {0: "U8", 1: "U32", 2: "I64", 3: "F16", 4: "BF16", 5: "F32", 6: "F64"}
_NP = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "I64": np.int64, "U32": np.uint32, "U8": np.uint8}


class SafetensorsFile:
    """with SafetensorsFile(path) as f: f.entries -> [(name, dtype name or None, shape, bytes)], f.read(name)"""

    def __init__(self, path: str):
        self._h = ctypes.c_void_p()
        _lib.call("rb_safetensors_open", str(path).encode(), ctypes.byref(self._h))
        self.entries: List[Tuple[str, Optional[str], Tuple[int, ...], int]] = []
        self._data: Dict[str, Tuple[int, int]] = {}
        for i in range(_lib.lib().rb_safetensors_count(self._h)):
            name, dtype, rank = ctypes.c_char_p(), ctypes.c_int32(), ctypes.c_int32()
            shape, data, nbytes = (ctypes.c_int64 * 8)(), ctypes.c_void_p(), ctypes.c_uint64()
            _lib.call("rb_safetensors_entry", self._h, i, ctypes.byref(name), ctypes.byref(dtype), ctypes.byref(rank), shape,
                      ctypes.byref(data), ctypes.byref(nbytes))
            n = name.value.decode()
            self.entries.append((n, _DTYPE_TAG.get(dtype.value), tuple(shape[:rank.value]), int(nbytes.value)))
            self._data[n] = (data.value or 0, int(nbytes.value))

    def read_bytes(self, name: str) -> bytes:
        addr, n = self._data[name]
        return ctypes.string_at(addr, n) if n else b""

    def close(self) -> None:
        if self._h:
            _lib.lib().rb_safetensors_close(self._h)
            self._h = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def bf16_bytes(a: np.ndarray) -> bytes:
    """float32 -> bfloat16 bit patterns, round to nearest even (NaN kept quiet)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(np.asarray(a, dtype=np.float32))
    r[nan.reshape(r.shape)] = 0x7FC0
    return r.tobytes()


def write_safetensors(path: str, tensors: Dict[str, np.ndarray], dtype: str = "F32", metadata: Optional[dict] = None) -> None:
    """Writes float arrays as one .safetensors file with every tensor stored as `dtype`
    (F64, F32, F16 or BF16), names in the given order."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, a in tensors.items():
        a = np.asarray(a)
        blob = bf16_bytes(a) if dtype == "BF16" else np.ascontiguousarray(a, dtype=_NP[dtype]).tobytes()
        header[name] = {"dtype": dtype, "shape": [int(s) for s in a.shape], "data_offsets": [off, off + len(blob)]}
        blobs.append(blob)
        off += len(blob)
    js = json.dumps(header, separators=(",", ":")).encode()
    js += b" " * ((8 - len(js) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for b in blobs:
            f.write(b)
