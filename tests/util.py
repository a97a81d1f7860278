"""Helpers shared by the tests: build the CPU oracle and the CUDA model from one seeded weight set."""
import numpy as np
import torch

import rai_cpu  # oracle/rai_cpu.py (test infrastructure)
from rai_b200 import configs, synth


def oracle_config(cfg: dict) -> "rai_cpu.Config":
    return rai_cpu.Config(
        arch=cfg["arch"], vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"],
        intermediate_size=cfg["intermediate_size"], num_hidden_layers=cfg["num_hidden_layers"],
        num_attention_heads=cfg["num_attention_heads"],
        num_key_value_heads=cfg.get("num_key_value_heads") or cfg["num_attention_heads"],
        max_position_embeddings=cfg["max_position_embeddings"], rope_theta=cfg["rope_theta"],
        norm_eps=configs.norm_eps(cfg), hidden_act=cfg["hidden_act"],
        tie_word_embeddings=configs.tied(cfg), partial_rotary_factor=cfg.get("partial_rotary_factor", 1.0),
        sliding_window=cfg.get("sliding_window", 1 << 30))


def oracle_params(cfg: dict, weights: dict) -> dict:
    p = {k: torch.from_numpy(v) for k, v in weights.items()}
    if cfg["arch"] == "qwen2" and configs.tied(cfg):
        p["lm_head.weight"] = p["model.embed_tokens.weight"]  # one matrix under both names
    return p


def build_oracle(cfg: dict, weights: dict):
    return rai_cpu.build(oracle_config(cfg), oracle_params(cfg, weights))


def logit_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| relative to the range of the reference logits."""
    got, want = got.float().cpu().reshape(-1), want.float().reshape(-1)
    rng = float(want.max() - want.min())
    return float((got - want).abs().max()) / max(rng, 1e-12)


def rel_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| / max |want| — the "relative" error used for float32 comparisons."""
    got, want = got.float().cpu().reshape(-1), want.float().reshape(-1)
    return float((got - want).abs().max()) / max(float(want.abs().max()), 1e-12)


def top2_margin(logits: torch.Tensor) -> torch.Tensor:
    v = logits.float().topk(2, dim=-1).values
    return v[..., 0] - v[..., 1]
