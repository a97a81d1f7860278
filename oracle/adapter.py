"""Builds the CPU oracle (rai_cpu.py) from a configuration dict and a name -> numpy weight map in the
checkpoint naming.  TEST INFRASTRUCTURE, like the rest of this directory: used by tests/, by
__graft_entry__.smoke() and by the cpu_baseline leg of bench.py, never by the product package."""
import torch

import rai_cpu


def _norm_eps(cfg: dict) -> float:
    return cfg["layer_norm_eps"] if cfg["arch"] == "phi2" else cfg["rms_norm_eps"]


def _tied(cfg: dict) -> bool:
    return cfg["arch"] == "gemma" or bool(cfg.get("tie_word_embeddings", False))


def oracle_config(cfg: dict) -> "rai_cpu.Config":
    return rai_cpu.Config(
        arch=cfg["arch"], vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"],
        intermediate_size=cfg["intermediate_size"], num_hidden_layers=cfg["num_hidden_layers"],
        num_attention_heads=cfg["num_attention_heads"],
        num_key_value_heads=cfg.get("num_key_value_heads") or cfg["num_attention_heads"],
        max_position_embeddings=cfg["max_position_embeddings"], rope_theta=cfg["rope_theta"],
        norm_eps=_norm_eps(cfg), hidden_act=cfg["hidden_act"], tie_word_embeddings=_tied(cfg),
        partial_rotary_factor=cfg.get("partial_rotary_factor", 1.0), sliding_window=cfg.get("sliding_window", 1 << 30))


def oracle_params(cfg: dict, weights: dict) -> dict:
    p = {k: (v if isinstance(v, torch.Tensor) else torch.from_numpy(v)) for k, v in weights.items()}
    if cfg["arch"] == "qwen2" and _tied(cfg):
        p["lm_head.weight"] = p["model.embed_tokens.weight"]  # one matrix under both names
    return p


def build_oracle(cfg: dict, weights: dict):
    return rai_cpu.build(oracle_config(cfg), oracle_params(cfg, weights))
