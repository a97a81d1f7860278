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


# --------------------------------------------------------------------------------------------------
# Host-side agreement and liveness of a tensor-parallel group (torch.distributed; no GPU involved)
# --------------------------------------------------------------------------------------------------
def agree_on_exchange(local_ok: bool, group=None) -> bool:
    """The decision rb_model_tp_init takes about its peer-memory exchange, stated on the host: every rank, whether
    it could map its peers' buffers or not, joins ONE sum of votes, and the exchange is used only if all voted yes.
    A rank that dropped out on its own would leave the others in a collective it never joins, and the two sides
    would go on with different protocols."""
    import torch
    import torch.distributed as dist
    vote = torch.tensor([1.0 if local_ok else 0.0])
    dist.all_reduce(vote, op=dist.ReduceOp.SUM, group=group)
    return bool(vote.item() > dist.get_world_size(group) - 0.5)


class PeerLeft(RuntimeError):
    """A member of the tensor-parallel group has announced that it leaves, or has gone silent."""


class PeerWatch:
    """Liveness of a tensor-parallel group between decode steps, through a key-value store (torch.distributed's
    TCPStore / the default store).  A decode step of a group is collective: a rank that launched it while a peer is
    gone would wait on that peer's flags until the device-side budget runs out.  So every rank posts the step it is
    about to run, a rank that leaves says so first (between steps, with none of its kernels in flight), and `check`
    is called before each launch: it raises PeerLeft instead of launching when a peer has left or has not reached
    this step within `timeout_s`."""

    def __init__(self, store, rank: int, size: int, timeout_s: float = 5.0):
        self.store, self.rank, self.size, self.timeout_s = store, rank, size, timeout_s

    def post(self, step: int) -> None:
        self.store.set(f"tp/step/{self.rank}", str(int(step)))

    def leave(self) -> None:
        self.store.set(f"tp/left/{self.rank}", "1")

    def _get(self, key: str):
        try:
            return self.store.get(key).decode() if self.store.check([key]) else None
        except Exception:
            return None

    def check(self, step: int) -> None:
        import time
        deadline = time.time() + self.timeout_s
        self.post(step)
        for r in range(self.size):
            if r == self.rank:
                continue
            while True:
                if self._get(f"tp/left/{r}") is not None:
                    raise PeerLeft(f"rank {r} left the group before step {step}")
                at = self._get(f"tp/step/{r}")
                if at is not None and int(at) >= step:
                    break
                if time.time() > deadline:
                    raise PeerLeft(f"rank {r} did not reach step {step} within {self.timeout_s} s")
                time.sleep(0.005)
