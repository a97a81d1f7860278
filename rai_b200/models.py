"""Host-side mirror of rai-models' decoders over the C ABI: `Model::new`, `update_by_safetensors`,
`Model::fwd(tokens, seqlen_offset)`, `clear_kv_cache` (rai-models/src/llm/qwen2.rs:287-366 and the
phi2 / phi3 / gemma twins).  torch is used for device memory of inputs and outputs only."""
from __future__ import annotations

import ctypes
from typing import Dict, Iterable, Optional

import numpy as np
import torch

from . import _lib, configs
from .device import Cuda

_TORCH_DTYPE = {_lib.BF16: torch.bfloat16, _lib.F32: torch.float32}


def _shape_array(shape):
    return (ctypes.c_int64 * max(1, len(shape)))(*[int(s) for s in shape])


class Model:
    """One decoder on one GPU (or one tensor-parallel rank).

    cfg         a configuration dict (see rai_b200.configs)
    dtype       _lib.BF16 or _lib.F32, the `dtype` argument of Model::new
    device      Cuda(id)
    max_batch / max_seq   KV-cache capacity;  max_tokens  largest batch*seq of one forward call
    """

    def __init__(self, cfg: dict, dtype: int, device: Cuda, max_batch: int, max_seq: int,
                 max_tokens: Optional[int] = None, tp_rank: int = 0, tp_size: int = 1):
        self.cfg, self.dtype, self.device = cfg, dtype, device
        self.max_batch, self.max_seq = max_batch, max_seq
        self.max_tokens = max_tokens or max_batch * max_seq
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self._struct = configs.to_struct(cfg, dtype, max_batch, max_seq, self.max_tokens, tp_rank, tp_size)
        self._m = ctypes.c_void_p()
        device.use_torch_stream()
        _lib.call("rb_model_create", device.ctx, ctypes.byref(self._struct), ctypes.byref(self._m))
        self._finalized = False

    # ---- parameters -----------------------------------------------------------------------
    def param_names(self):
        L = _lib.lib()
        return [L.rb_model_param_name(self._m, i).decode() for i in range(L.rb_model_param_count(self._m))]

    def update_param(self, name: str, value) -> None:
        """Tensor::update_by_name (rai-core/src/nn.rs:192-205): cast to the model dtype and copy.
        `value` is a numpy float32 array, or a torch tensor (float32 / bfloat16, host or this GPU)."""
        if isinstance(value, np.ndarray):
            arr = np.ascontiguousarray(value, dtype=np.float32)
            _lib.call("rb_model_load_param", self._m, name.encode(), ctypes.c_void_p(arr.ctypes.data), 0, _lib.F32,
                      arr.ndim, _shape_array(arr.shape))
            return
        t = value.contiguous()
        if t.dtype not in (torch.float32, torch.bfloat16):
            t = t.float()
        src = _lib.F32 if t.dtype == torch.float32 else _lib.BF16
        if t.is_cuda:
            self.device.use_torch_stream()
        _lib.call("rb_model_load_param", self._m, name.encode(), ctypes.c_void_p(t.data_ptr()), int(t.is_cuda), src,
                  t.dim(), _shape_array(t.shape))
        if t.is_cuda:
            self.device.synchronize()  # `t` may be freed by the caller right after

    def update_params(self, named: Dict[str, object]) -> None:
        """Module::update_named_params for a whole name -> tensor map."""
        for k, v in named.items():
            self.update_param(k, v)
        self.finalize()

    def update_by_safetensors(self, files: Iterable[str]) -> None:
        """Module::update_by_safetensors (rai-core/src/nn.rs:39-55) through the library's own reader: the
        files are mapped and streamed to the GPU, each parameter cast to the model dtype on the device."""
        paths = [str(f).encode() for f in files]
        arr = (ctypes.c_char_p * len(paths))(*paths)
        self.device.use_torch_stream()
        _lib.call("rb_model_load_safetensors", self._m, arr, len(paths))
        self._finalized = True

    def finalize(self) -> None:
        _lib.call("rb_model_finalize", self._m)
        self._finalized = True

    def tp_init(self, unique_id: bytes) -> None:
        buf = ctypes.create_string_buffer(unique_id, 128)
        _lib.call("rb_model_tp_init", self._m, buf, 128)

    # ---- forward ---------------------------------------------------------------------------
    def _tokens_dev(self, tokens) -> torch.Tensor:
        if isinstance(tokens, np.ndarray):
            tokens = torch.from_numpy(tokens.astype(np.int64))
        return tokens.to(device=f"cuda:{self.device.id}", dtype=torch.int32).contiguous()

    def forward(self, tokens, seqlen_offset: int) -> torch.Tensor:
        """Model::fwd: tokens [B, S] -> logits of the last position, [B, 1, V] ([B, V] for phi2,
        which squeezes, phi2.rs:346)."""
        ids = self._tokens_dev(tokens)
        b, s = ids.shape
        self.device.use_torch_stream()
        logits = torch.empty((b, self.cfg["vocab_size"]), dtype=_TORCH_DTYPE[self.dtype], device=ids.device)
        _lib.call("rb_model_forward", self._m, ctypes.c_void_p(ids.data_ptr()), b, s, int(seqlen_offset),
                  ctypes.c_void_p(logits.data_ptr()))
        self.device.synchronize()
        return logits if self.cfg["arch"] == "phi2" else logits.unsqueeze(1)

    def forward_ragged(self, tokens, lens, seqlen_offset: int = 0) -> torch.Tensor:
        """Model::fwd for a right-padded batch: tokens [B, S], lens[b] valid tokens in row b.  Logits [B, V] of each
        sequence's last valid position; the cache keeps lens[b] tokens of sequence b."""
        ids = self._tokens_dev(tokens)
        b, s = ids.shape
        lens_arr = np.ascontiguousarray(np.asarray(lens, dtype=np.int32))
        self.device.use_torch_stream()
        logits = torch.empty((b, self.cfg["vocab_size"]), dtype=_TORCH_DTYPE[self.dtype], device=ids.device)
        _lib.call("rb_model_forward_ragged", self._m, ctypes.c_void_p(ids.data_ptr()), b, s, int(seqlen_offset),
                  lens_arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(logits.data_ptr()))
        self.device.synchronize()
        return logits

    def generate_ragged(self, prompts, steps: int) -> np.ndarray:
        """Generation for prompts of different lengths in one batch (a list of 1-D token arrays): right-pad, one
        ragged prompt call, then the device-side decode loop with every sequence at its own length.  [B, steps]."""
        b = len(prompts)
        lens = np.asarray([len(p) for p in prompts], dtype=np.int32)
        s = int(lens.max())
        ids = np.zeros((b, s), dtype=np.int32)
        for i, p in enumerate(prompts):
            ids[i, : len(p)] = np.asarray(p, dtype=np.int32)
        tok_in = torch.from_numpy(ids).pin_memory()
        first = torch.empty((b,), dtype=torch.int32).pin_memory()
        self.clear_kv_cache()
        _lib.call("rb_model_generate_ragged", self._m, ctypes.c_void_p(tok_in.data_ptr()), b, s,
                  lens.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(first.data_ptr()))
        out = [first.numpy().astype(np.int64).reshape(b, 1)]
        if steps > 1:
            rest = self.decode_loop(first.to(f"cuda:{self.device.id}"), -1, steps - 1)
            self.device.synchronize()
            out.append(rest.cpu().numpy().astype(np.int64).T)
        return np.concatenate(out, axis=1)

    def generate_step(self, tokens_host: torch.Tensor, seqlen_offset: int, out_host: torch.Tensor) -> None:
        """One iteration of the examples' generation loop with greedy sampling on the device:
        tokens_host [B, S] int32 (pinned) -> out_host [B] int32 (pinned).  Synchronous."""
        b, s = tokens_host.shape
        _lib.call("rb_model_generate_step", self._m, ctypes.c_void_p(tokens_host.data_ptr()), b, s, int(seqlen_offset),
                  ctypes.c_void_p(out_host.data_ptr()))

    def decode_loop(self, tokens_dev: torch.Tensor, pos: int, steps: int) -> torch.Tensor:
        """`steps` greedy single-token steps kept on the device; returns [steps, B] int32 (asynchronous)."""
        b = tokens_dev.numel()
        out = torch.empty((steps, b), dtype=torch.int32, device=tokens_dev.device)
        self.device.use_torch_stream()
        _lib.call("rb_model_decode_loop", self._m, ctypes.c_void_p(tokens_dev.data_ptr()), b, int(pos), int(steps),
                  ctypes.c_void_p(out.data_ptr()))
        return out

    def greedy_generate(self, prompt, steps: int, collect_logits: bool = False):
        """Prefill once, then one token per step (examples/qwen2/src/main.rs:78-99 without the
        repeat penalty).  Returns [B, steps] int64 on the host (and [steps, B, V] float32 logits)."""
        self.clear_kv_cache()
        ids = self._tokens_dev(prompt)
        b = ids.shape[0]
        toks, all_logits, pos = [], [], 0
        argmax = torch.empty((b,), dtype=torch.int32, device=ids.device)
        for _ in range(steps):
            logits = self.forward(ids, pos).reshape(b, -1)
            pos += ids.shape[1]
            _lib.call("rb_argmax_rows", self.device.ctx, ctypes.c_void_p(logits.data_ptr()), self.dtype, b,
                      logits.shape[1], ctypes.c_void_p(argmax.data_ptr()))
            self.device.synchronize()
            toks.append(argmax.clone())
            if collect_logits:
                all_logits.append(logits.float().cpu())
            ids = argmax.reshape(b, 1).clone()
        out = torch.stack(toks, dim=1).cpu().long()
        return (out, torch.stack(all_logits)) if collect_logits else out

    def clear_kv_cache(self) -> None:
        _lib.call("rb_model_clear_kv_cache", self._m)

    def set_sampling(self, repeat_penalty: float = 1.10, repeat_last_n: int = 64, eos_token: int = -1) -> None:
        """The sampling of the examples' loops (examples/qwen2/src/main.rs:74-76,84-96) for generate_step and
        decode_loop: repeat penalty over the last `repeat_last_n` tokens, then argmax, then the stop rule."""
        _lib.call("rb_model_set_sampling", self._m, float(repeat_penalty), int(repeat_last_n), int(eos_token))

    def finished(self, batch: int) -> np.ndarray:
        """Which sequences have produced the end-of-sequence token."""
        flags = np.zeros((batch,), dtype=np.uint8)
        _lib.call("rb_model_finished", self._m, int(batch), flags.ctypes.data_as(ctypes.c_void_p))
        return flags.astype(bool)

    def generate(self, prompt, steps: int) -> np.ndarray:
        """The examples' generation loop through the library's own entry points: one generate_step for the
        prompt (host tokens in, sampled token out), then the device-side decode loop.  [B, steps] int64."""
        ids = np.ascontiguousarray(np.asarray(prompt, dtype=np.int32))
        b = ids.shape[0]
        tok_in = torch.from_numpy(ids).pin_memory()
        first = torch.empty((b,), dtype=torch.int32).pin_memory()
        self.clear_kv_cache()
        self.generate_step(tok_in, 0, first)
        out = [first.numpy().astype(np.int64).reshape(b, 1)]
        if steps > 1:
            rest = self.decode_loop(first.to(f"cuda:{self.device.id}"), ids.shape[1], steps - 1)
            self.device.synchronize()
            out.append(rest.cpu().numpy().astype(np.int64).T)
        return np.concatenate(out, axis=1)

    def kv_read(self, layer: int, seq: int, kv_head: int, t0: int, n: int):
        """Test hook: K and V of tokens [t0, t0+n) as float32 [n, head_dim] host tensors."""
        d = configs.head_dim(self.cfg)
        dt = _TORCH_DTYPE[self.dtype]
        k = torch.empty((n, d), dtype=dt)
        v = torch.empty((n, d), dtype=dt)
        cache = ctypes.c_void_p(_lib.lib().rb_model_kv_cache(self._m))
        _lib.call("rb_kv_cache_read", cache, layer, seq, kv_head, t0, n, ctypes.c_void_p(k.data_ptr()),
                  ctypes.c_void_p(v.data_ptr()))
        return k.float(), v.float()

    def read_param(self, name: str) -> torch.Tensor:
        """One named parameter back on the host, in the model dtype and the parameter's full shape (a tensor-parallel
        rank returns the rectangle it keeps, zeros elsewhere)."""
        from . import synth
        shapes = {n: sh for n, sh, _ in synth.param_shapes(self.cfg)}
        t = torch.empty(shapes[name], dtype=_TORCH_DTYPE[self.dtype])
        _lib.call("rb_model_read_param", self._m, name.encode(), ctypes.c_void_p(t.data_ptr()), t.numel() * t.element_size())
        return t

    def to_safetensors(self, path: str) -> None:
        """Module::to_safetensors (rai-core/src/nn.rs:31-37): every named parameter, in the model dtype."""
        from . import safetensors_io
        named = {n: self.read_param(n) for n in self.param_names()}
        if self.dtype == _lib.BF16:
            safetensors_io.write_safetensors(path, {k: v.float().numpy() for k, v in named.items()}, "BF16")
        else:
            safetensors_io.write_safetensors(path, {k: v.numpy() for k, v in named.items()}, "F32")

    def param_bytes(self) -> int:
        return int(_lib.lib().rb_model_param_bytes(self._m))

    def close(self) -> None:
        if self._m:
            _lib.call("rb_model_destroy", self._m)
            self._m = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
