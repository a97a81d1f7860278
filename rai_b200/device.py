"""`Cuda(id)`: the device object the backend binds to (rai-core/src/device.rs:161-196).  It owns the
library context (stream, tensor-map cache, status word) of one GPU of this process."""
from __future__ import annotations

import ctypes
from typing import Dict

from . import _lib


class Cuda:
    _cache: Dict[int, "Cuda"] = {}

    def __new__(cls, id: int = 0):
        # one context per (process, GPU), like the device cache of candle.rs:141-175
        if id in cls._cache:
            return cls._cache[id]
        self = super().__new__(cls)
        self.id = id
        self._ctx = ctypes.c_void_p()
        _lib.call("rb_init", id, ctypes.byref(self._ctx))
        cls._cache[id] = self
        return self

    @property
    def ctx(self) -> ctypes.c_void_p:
        return self._ctx

    def __eq__(self, other):  # rai-core/tests/device.rs:4-18
        return isinstance(other, Cuda) and other.id == self.id

    def __hash__(self):
        return hash(("cuda", self.id))

    def __repr__(self):
        return f"Cuda({self.id})"

    def use_torch_stream(self) -> None:
        """Enqueue library work on torch's current stream for this device, so that torch tensors
        produced before a call are ready when it runs and vice versa."""
        import torch
        _lib.call("rb_set_stream", self._ctx, ctypes.c_void_p(torch.cuda.current_stream(self.id).cuda_stream))

    def synchronize(self) -> None:
        """Waits for the stream and raises if a kernel recorded a device-side failure."""
        _lib.call("rb_sync", self._ctx)

    def sm_count(self) -> int:
        return _lib.lib().rb_sm_count(self._ctx)

    def launch_count(self) -> int:
        return int(_lib.lib().rb_launch_count(self._ctx))


def cuda_if_available(id: int = 0) -> Cuda:
    """rai-core/src/device.rs:198-204 — here there is no Cpu to fall back to: it raises instead."""
    return Cuda(id)
