"""Decoder configurations.

Field names follow the reference `Config` structs (rai-models/src/llm/qwen2.rs:8-24, phi2.rs:9-24,
phi3.rs:9-24, gemma.rs:12-27) as they appear in a Hugging Face config.json, plus `arch`.
`BASELINE` holds the five benchmark configurations; `TINY` holds small models of the same four
architectures for parity tests.
"""
from __future__ import annotations

import copy
from typing import Dict

from . import _lib

ARCH_IDS = {"qwen2": _lib.ARCH_QWEN2, "phi2": _lib.ARCH_PHI2, "phi3": _lib.ARCH_PHI3, "gemma": _lib.ARCH_GEMMA}
# serde names of rai-nn/src/activations.rs:5-17
ACT_IDS = {"silu": _lib.ACT_SILU, "gelu_new": _lib.ACT_GELU_TANH, "newgelu": _lib.ACT_GELU_TANH,
           "gelu": _lib.ACT_GELU_ERF, "relu": _lib.ACT_RELU}

BASELINE: Dict[str, dict] = {
    # C1: Qwen2-0.5B architecture; batch 1, 128-token prompt, 128 greedy steps
    "qwen2-0.5b": dict(arch="qwen2", vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                       num_attention_heads=14, num_key_value_heads=2, max_position_embeddings=4096,
                       sliding_window=32768, rope_theta=1e6, rms_norm_eps=1e-6, hidden_act="silu",
                       tie_word_embeddings=True),
    # C2: Phi-2 architecture; batch 8, 512-token prompts, 256 greedy steps
    "phi2": dict(arch="phi2", vocab_size=51200, hidden_size=2560, intermediate_size=10240, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=32, max_position_embeddings=2048, rope_theta=1e4,
                 layer_norm_eps=1e-5, hidden_act="gelu_new", partial_rotary_factor=0.4, qk_layernorm=False,
                 tie_word_embeddings=False),
    # C3: Phi-3-mini architecture; batch 4 x 2048-token prompts, 64 decode steps
    "phi3-mini": dict(arch="phi3", vocab_size=32064, hidden_size=3072, intermediate_size=8192, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=32, max_position_embeddings=4096, rope_theta=1e4,
                      rms_norm_eps=1e-5, hidden_act="silu"),
    # C4: Gemma-2B architecture; batch 32 decode from a 1024-token cache, 128 greedy steps
    "gemma-2b": dict(arch="gemma", vocab_size=256000, hidden_size=2048, intermediate_size=16384, num_hidden_layers=18,
                     num_attention_heads=8, num_key_value_heads=1, head_dim=256, max_position_embeddings=8192,
                     rope_theta=1e4, rms_norm_eps=1e-6, hidden_act="gelu_new", attention_bias=False),
    # C5: Qwen2-7B architecture; prefill 8 x 4096, then batch-64 decode at 2048-token context, 256 steps
    "qwen2-7b": dict(arch="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                     num_attention_heads=28, num_key_value_heads=4, max_position_embeddings=8192, sliding_window=131072,
                     rope_theta=1e6, rms_norm_eps=1e-6, hidden_act="silu", tie_word_embeddings=False),
}

TINY: Dict[str, dict] = {
    "tiny-qwen2": dict(arch="qwen2", vocab_size=512, hidden_size=256, intermediate_size=320, num_hidden_layers=2,
                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256, sliding_window=4096,
                  rope_theta=1e6, rms_norm_eps=1e-6, hidden_act="silu", tie_word_embeddings=False),
    "tiny-qwen2-tied": dict(arch="qwen2", vocab_size=384, hidden_size=128, intermediate_size=192, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=256, sliding_window=4096,
                       rope_theta=1e6, rms_norm_eps=1e-6, hidden_act="silu", tie_word_embeddings=True),
    # 7 query heads per KV head and head_dim 128, the grouping of the 7B benchmark configuration
    "tiny-qwen2-g7": dict(arch="qwen2", vocab_size=640, hidden_size=896, intermediate_size=768, num_hidden_layers=2,
                     num_attention_heads=7, num_key_value_heads=1, max_position_embeddings=512, sliding_window=4096,
                     rope_theta=1e6, rms_norm_eps=1e-6, hidden_act="silu", tie_word_embeddings=False),
    # narrow shapes: K = 40 and 64 (less than one 64-wide K slice), N = 40, a 64-row vocabulary
    "tiny-qwen2-narrow": dict(arch="qwen2", vocab_size=64, hidden_size=128, intermediate_size=40, num_hidden_layers=2,
                              num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=256,
                              sliding_window=4096, rope_theta=1e6, rms_norm_eps=1e-6, hidden_act="silu",
                              tie_word_embeddings=False),
    # the head layout of the 7B benchmark configuration (28 query heads over 4 KV heads) at small width
    "tiny-qwen2-28h": dict(arch="qwen2", vocab_size=1024, hidden_size=1792, intermediate_size=1024, num_hidden_layers=2,
                           num_attention_heads=28, num_key_value_heads=4, max_position_embeddings=256,
                           sliding_window=4096, rope_theta=1e6, rms_norm_eps=1e-6, hidden_act="silu",
                           tie_word_embeddings=False),
    "tiny-phi2": dict(arch="phi2", vocab_size=320, hidden_size=160, intermediate_size=640, num_hidden_layers=2,
                 num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=256, rope_theta=1e4,
                 layer_norm_eps=1e-5, hidden_act="gelu_new", partial_rotary_factor=0.4, qk_layernorm=False,
                 tie_word_embeddings=False),
    "tiny-phi3": dict(arch="phi3", vocab_size=448, hidden_size=192, intermediate_size=512, num_hidden_layers=2,
                 num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=256, rope_theta=1e4,
                 rms_norm_eps=1e-5, hidden_act="silu"),
    "tiny-gemma": dict(arch="gemma", vocab_size=640, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                  num_attention_heads=2, num_key_value_heads=1, head_dim=256, max_position_embeddings=256,
                  rope_theta=1e4, rms_norm_eps=1e-6, hidden_act="gelu_new", attention_bias=False),
}


def get(name: str) -> dict:
    src = BASELINE.get(name) or TINY.get(name)
    if src is None:
        raise KeyError(f"unknown configuration {name!r}")
    return copy.deepcopy(src)


def head_dim(cfg: dict) -> int:
    return cfg["hidden_size"] // cfg["num_attention_heads"]


def rotary_dim(cfg: dict) -> int:
    # phi2.rs:47: (partial_rotary_factor * head_dim) as usize
    return int(cfg.get("partial_rotary_factor", 1.0) * head_dim(cfg))


def norm_eps(cfg: dict) -> float:
    return cfg["layer_norm_eps"] if cfg["arch"] == "phi2" else cfg["rms_norm_eps"]


def tied(cfg: dict) -> bool:
    return cfg["arch"] == "gemma" or bool(cfg.get("tie_word_embeddings", False))


def to_struct(cfg: dict, dtype: int, max_batch: int, max_seq: int, max_tokens: int, tp_rank: int = 0,
              tp_size: int = 1) -> "_lib.ModelConfig":
    if cfg["arch"] == "phi2" and cfg.get("qk_layernorm"):
        raise _lib.RaiB200Error(-7, "phi2 qk_layernorm is not implemented (phi2.rs:166-172)")
    s = _lib.ModelConfig()
    s.arch = ARCH_IDS[cfg["arch"]]
    s.dtype = dtype
    for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
              "max_position_embeddings"):
        setattr(s, k, int(cfg[k]))
    s.num_key_value_heads = int(cfg.get("num_key_value_heads") or cfg["num_attention_heads"])
    s.rotary_dim = rotary_dim(cfg)
    s.hidden_act = ACT_IDS[cfg["hidden_act"]]
    s.tie_word_embeddings = int(tied(cfg))
    s.max_batch, s.max_seq, s.max_tokens = int(max_batch), int(max_seq), int(max_tokens)
    s.tp_rank, s.tp_size = int(tp_rank), int(tp_size)
    # only qwen2's mask has the sliding-window term (qwen2.rs:316-327); the other families' masks are plain causal
    s.sliding_window = int(cfg.get("sliding_window") or 0) if cfg["arch"] == "qwen2" else 0
    s.reserved0 = 0
    s.rope_theta = float(cfg["rope_theta"])
    s.norm_eps = float(norm_eps(cfg))
    return s
