"""Tensor-parallel shard plan: which query / KV heads, intermediate units and vocabulary rows a rank
owns.  This is the host-side statement of what rai_b200/csrc/model.cu does when it copies a
parameter (rb_model_load_param keeps this rank's rectangle of every tensor); it exists so that the
plan can be checked on CPU ranks (gloo) against the unsharded computation.

Megatron layout: q/k/v, gate/up and lm_head are split by output rows, o_proj/down by input columns,
one allreduce after each of the latter.  When there are more ranks than KV heads, tp/kv ranks share
a KV head and split its query heads between them; a share that comes out short is padded with
zero-weight heads (their o_proj columns are zero, so the result is unchanged).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import numpy as np

from . import configs


@dataclass
class Plan:
    rank: int
    size: int
    q_heads: List[int]      # global query head of each local head, -1 = zero padding
    kv_heads: List[int]     # global KV heads held by this rank
    inter: slice            # intermediate units
    vocab: slice            # vocabulary rows


def plan(cfg: dict, rank: int, size: int) -> Plan:
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nq
    g = nq // nkv
    inter, vocab = cfg["intermediate_size"], cfg["vocab_size"]
    if inter % size or vocab % size:
        raise ValueError("intermediate_size and vocab_size must divide by the tensor-parallel size")
    if size <= nkv:
        if nkv % size:
            raise ValueError("KV heads must divide by the tensor-parallel size")
        per = nkv // size
        kv = list(range(rank * per, (rank + 1) * per))
        q = [h * g + j for h in kv for j in range(g)]
    else:
        if size % nkv:
            raise ValueError("the tensor-parallel size must be a multiple of the KV heads")
        rpk = size // nkv
        qpr = -(-g // rpk)
        kvh, sub = rank // rpk, rank % rpk
        kv = [kvh]
        q = [kvh * g + sub * qpr + j if sub * qpr + j < g else -1 for j in range(qpr)]
    il, vl = inter // size, vocab // size
    return Plan(rank, size, q, kv, slice(rank * il, (rank + 1) * il), slice(rank * vl, (rank + 1) * vl))


def shard_weights(cfg: dict, weights: Dict[str, np.ndarray], p: Plan) -> Dict[str, np.ndarray]:
    """This rank's share of a checkpoint, keeping the checkpoint's names, for the qwen2 / gemma
    layout (separate q/k/v and gate/up matrices).  Padding heads become zero rows / columns."""
    d = configs.head_dim(cfg)
    out = {}

    def rows_of_heads(w, heads):
        blocks = [w[h * d:(h + 1) * d] if h >= 0 else np.zeros((d,) + w.shape[1:], w.dtype) for h in heads]
        return np.concatenate(blocks, 0)

    def cols_of_heads(w, heads):
        blocks = [w[:, h * d:(h + 1) * d] if h >= 0 else np.zeros((w.shape[0], d), w.dtype) for h in heads]
        return np.concatenate(blocks, 1)

    for name, w in weights.items():
        if ".q_proj." in name:
            out[name] = rows_of_heads(w, p.q_heads)
        elif ".k_proj." in name or ".v_proj." in name:
            out[name] = rows_of_heads(w, p.kv_heads)
        elif ".o_proj.weight" in name:
            out[name] = cols_of_heads(w, p.q_heads)
        elif ".gate_proj." in name or ".up_proj." in name:
            out[name] = w[p.inter]
        elif ".down_proj.weight" in name:
            out[name] = w[:, p.inter]
        elif name == "lm_head.weight":
            out[name] = w[p.vocab]
        else:
            out[name] = w
    return out
