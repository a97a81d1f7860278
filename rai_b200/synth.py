"""Parameter names/shapes of the four decoders and seeded synthetic weights and prompts.

Names follow the derive rule of rai-core/src/nn.rs:256-269 (field path joined by '.', Vec index as
'.i') with the `#[param(rename = ...)]` attributes of qwen2.rs:276-282, phi2.rs:307-313,
phi3.rs:260-266 and gemma.rs:309-318, i.e. the keys of a Hugging Face safetensors checkpoint.

Synthetic weights stand in for real checkpoints (none are available offline): every Linear and
Embedding matrix ~ N(0, 0.02), biases ~ N(0, 0.02), norm weights 1 + N(0, 0.05) (0 + N(0, 0.05) for
gemma, whose norm applies 1 + w; the noise keeps a kernel that forgets the weight from passing), LayerNorm
biases ~ N(0, 0.02); token ids uniform on [0, vocab).
"""
from __future__ import annotations

from typing import Dict, Iterator, List, Tuple

import numpy as np

from . import configs


def param_shapes(cfg: dict) -> List[Tuple[str, Tuple[int, ...], str]]:
    """[(name, shape, kind)] in checkpoint order; kind is 'matrix', 'bias', 'norm_w' or 'norm_b'."""
    a = cfg["arch"]
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nq
    d = configs.head_dim(cfg)
    out: List[Tuple[str, Tuple[int, ...], str]] = [("model.embed_tokens.weight", (V, H), "matrix")]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        if a == "phi3":
            out.append((p + "self_attn.qkv_proj.weight", ((nq + 2 * nkv) * d, H), "matrix"))
            out.append((p + "self_attn.o_proj.weight", (H, nq * d), "matrix"))
            out.append((p + "mlp.gate_up_proj.weight", (2 * I, H), "matrix"))
            out.append((p + "mlp.down_proj.weight", (H, I), "matrix"))
        else:
            bias = a in ("qwen2", "phi2")
            for n, rows in (("q_proj", nq * d), ("k_proj", nkv * d), ("v_proj", nkv * d)):
                out.append((p + f"self_attn.{n}.weight", (rows, H), "matrix"))
                if bias:
                    out.append((p + f"self_attn.{n}.bias", (rows,), "bias"))
            if a == "phi2":
                out.append((p + "self_attn.dense.weight", (H, nq * d), "matrix"))
                out.append((p + "self_attn.dense.bias", (H,), "bias"))
                out.append((p + "mlp.fc1.weight", (I, H), "matrix"))
                out.append((p + "mlp.fc1.bias", (I,), "bias"))
                out.append((p + "mlp.fc2.weight", (H, I), "matrix"))
                out.append((p + "mlp.fc2.bias", (H,), "bias"))
            else:
                out.append((p + "self_attn.o_proj.weight", (H, nq * d), "matrix"))
                out.append((p + "mlp.gate_proj.weight", (I, H), "matrix"))
                out.append((p + "mlp.up_proj.weight", (I, H), "matrix"))
                out.append((p + "mlp.down_proj.weight", (H, I), "matrix"))
        out.append((p + "input_layernorm.weight", (H,), "norm_w"))
        if a == "phi2":
            out.append((p + "input_layernorm.bias", (H,), "norm_b"))
        else:
            out.append((p + "post_attention_layernorm.weight", (H,), "norm_w"))
    if a == "phi2":
        out.append(("model.final_layernorm.weight", (H,), "norm_w"))
        out.append(("model.final_layernorm.bias", (H,), "norm_b"))
    else:
        out.append(("model.norm.weight", (H,), "norm_w"))
    if not configs.tied(cfg):
        out.append(("lm_head.weight", (V, H), "matrix"))
        if a == "phi2":
            out.append(("lm_head.bias", (V,), "bias"))
    return out


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16 -> float32 (so the CPU oracle and the GPU see the same values)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)


def iter_weights(cfg: dict, seed: int, round_bf16: bool = True) -> Iterator[Tuple[str, np.ndarray]]:
    """Yields (name, float32 array) in checkpoint order from numpy PCG64(seed)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    gemma = cfg["arch"] == "gemma"
    for name, shape, kind in param_shapes(cfg):
        if kind in ("matrix", "bias"):
            w = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
            # norm-like perturbation keeps the test weights from being trivially 1/0 everywhere
        elif kind == "norm_w":
            base = 0.0 if gemma else 1.0
            w = (base + rng.standard_normal(shape, dtype=np.float32) * np.float32(0.05)).astype(np.float32)
        else:
            w = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        yield name, (bf16_round(w) if round_bf16 else w)


def weights(cfg: dict, seed: int, round_bf16: bool = True) -> Dict[str, np.ndarray]:
    return dict(iter_weights(cfg, seed, round_bf16))


def prompt(cfg: dict, batch: int, seq: int, seed: int) -> np.ndarray:
    """[batch, seq] uint32 token ids, uniform on [0, vocab)."""
    rng = np.random.Generator(np.random.PCG64(seed + 1))
    return rng.integers(0, cfg["vocab_size"], size=(batch, seq), dtype=np.int64).astype(np.uint32)
