"""Decode parity at large batch and long context without a long CPU prefill.  TEST INFRASTRUCTURE, like the rest of
this directory: imported by tests/ and by the parity leg of bench.py (outside its timed region), never by the
product package.

A float32 CPU prefill of 64 x 2048 tokens through a full-width model takes minutes, so the cached prefix is
*injected* instead: the same random, bf16-rounded K and V rows go into the CPU oracle's cache
(`model.kv`, what rai keeps in `Attention::kv_cache`, rai-models/src/llm/qwen2.rs:127,193-204) and into the
GPU model's paged cache (through the library's own append kernel with a rotary width of 0, i.e. rows stored as
given).  The decode steps that follow run the whole model on both sides - embedding, norms, projections, RoPE,
the cache append, attention over the long cache, MLP, head - teacher-forced with the oracle's tokens.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Tuple

import numpy as np
import torch

import adapter
import rai_cpu


def rounded_params(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """N(0, 0.02) weights (norm weights 1, gemma 0; norm biases 0) rounded to bf16 and held as float32: the values
    both sides compute with."""
    from rai_b200 import synth
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape, kind in synth.param_shapes(cfg):
        if kind == "norm_w":
            t = torch.zeros(shape) if cfg["arch"] == "gemma" else torch.ones(shape)
        elif kind == "norm_b":
            t = torch.zeros(shape)
        else:
            t = (torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16).float()
        out[name] = t
    return out


def random_cache(cfg: dict, batch: int, ctx: int, seed: int) -> List[Tuple[torch.Tensor, torch.Tensor]]:
    """Per layer (k, v), each [batch, kv_heads, ctx, head_dim] float32 holding bf16-representable values."""
    from rai_b200 import configs
    nkv = cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    d = configs.head_dim(cfg)
    g = torch.Generator().manual_seed(seed)
    return [((torch.randn(batch, nkv, ctx, d, generator=g)).to(torch.bfloat16).float(),
             (torch.randn(batch, nkv, ctx, d, generator=g)).to(torch.bfloat16).float())
            for _ in range(cfg["num_hidden_layers"])]


def inject_gpu_cache(model, cfg: dict, kv, batch: int, ctx: int) -> None:
    """Writes `kv` into the GPU model's paged cache as the first `ctx` tokens of sequences 0..batch-1 (bf16 model,
    single GPU)."""
    from rai_b200 import _lib, configs
    nkv = cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    d = configs.head_dim(cfg)
    dev = model.device
    dev.use_torch_stream()
    cache = ctypes.c_void_p(_lib.lib().rb_model_kv_cache(model._m))
    _lib.call("rb_kv_cache_set_len", cache, batch, ctx)
    dummy = torch.zeros(64, dtype=torch.float32, device="cuda")
    q_out = torch.empty(batch * ctx, nkv * d, dtype=torch.bfloat16, device="cuda")
    for layer, (k, v) in enumerate(kv):
        # rows of [zero q heads | k heads | v heads] per token; rotary width 0 = stored as given
        kk = k.transpose(1, 2).reshape(batch * ctx, nkv * d).to(torch.bfloat16)
        vv = v.transpose(1, 2).reshape(batch * ctx, nkv * d).to(torch.bfloat16)
        rows = torch.cat([torch.zeros_like(kk), kk, vv], dim=1).cuda()
        _lib.call("rb_rope_kv_append", dev.ctx, ctypes.c_void_p(rows.data_ptr()), None, 0, None,
                  ctypes.c_void_p(dummy.data_ptr()), ctypes.c_void_p(dummy.data_ptr()), 0, batch, ctx, nkv, cache, layer,
                  ctypes.c_void_p(q_out.data_ptr()), _lib.BF16)
        dev.synchronize()
        del rows


def decode_parity(cfg: dict, params: Dict[str, torch.Tensor], model, batch: int, ctx: int, steps: int, seed: int,
                  tol: float = 2e-2) -> dict:
    """`steps` teacher-forced decode steps of `model` (GPU, bf16, weights already loaded from `params`) against the
    oracle built from the same `params`, both starting from the same injected `ctx`-token cache.  Returns the worst
    logit error (relative to the logit range), the number of greedy tokens that differ and how many of those are
    NOT excused by a reference top-1/top-2 margin below the tolerance."""
    oracle = rai_cpu.build(adapter.oracle_config(cfg), adapter.oracle_params(cfg, params))
    kv = random_cache(cfg, batch, ctx, seed)
    oracle.kv = [(k.clone(), v.clone()) for k, v in kv]
    inject_gpu_cache(model, cfg, kv, batch, ctx)
    del kv
    g = torch.Generator().manual_seed(seed + 1)
    ids = torch.randint(0, cfg["vocab_size"], (batch, 1), generator=g)
    worst, flips, unexcused = 0.0, 0, 0
    for t in range(steps):
        ref = oracle.forward(ids, ctx + t).reshape(batch, -1)
        got = model.forward(ids.numpy().astype(np.int32), ctx + t).reshape(batch, -1).float().cpu()
        rng = float(ref.max() - ref.min())
        worst = max(worst, float((got - ref).abs().max()) / max(rng, 1e-12))
        want = ref.argmax(-1)
        pick = got.argmax(-1)
        for b in range(batch):
            if int(pick[b]) != int(want[b]):
                flips += 1
                top = ref[b].topk(2).values
                row_rng = float(ref[b].max() - ref[b].min())
                if float(top[0] - top[1]) >= tol * row_rng:
                    unexcused += 1
        ids = want.reshape(batch, 1)
    return {"max_logit_err_of_range": worst, "tolerance": tol, "steps": steps, "batch": batch, "context": ctx,
            "greedy_tokens_differing": flips, "of_which_not_near_ties": unexcused,
            "layers": cfg["num_hidden_layers"]}
