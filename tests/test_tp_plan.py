"""The tensor-parallel shard plan on CPU ranks (gloo, world size 2, and the padded 8-way layout of the
7B configuration simulated in one process): sharded partial results summed across ranks equal the
unsharded oracle."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import rai_cpu
import util
from rai_b200 import configs, synth, tp


def sharded_forward(cfg, weights, plan, ids, allreduce, allgather):
    """One qwen2-style forward where every Linear uses this rank's shard and the row-parallel outputs
    go through `allreduce` (oracle ops, rai_cpu.py, with the Megatron split of model.cu)."""
    w = {k: torch.from_numpy(v) for k, v in tp.shard_weights(cfg, weights, plan).items()}
    d = configs.head_dim(cfg)
    nq_l, nkv_l = len(plan.q_heads), len(plan.kv_heads)
    b, s = ids.shape
    sin, cos = rai_cpu.rope_tables(d, cfg["max_position_embeddings"], cfg["rope_theta"], "qwen2")
    mask = rai_cpu.additive_causal_mask(b, s, 0) if s > 1 else None
    xs = rai_cpu.embedding(w["model.embed_tokens.weight"], ids)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = rai_cpu.rms_norm(xs, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        q = rai_cpu.linear(h, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias"))
        k = rai_cpu.linear(h, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias"))
        v = rai_cpu.linear(h, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias"))
        q = q.reshape(b, s, nq_l, d).transpose(1, 2)
        k = k.reshape(b, s, nkv_l, d).transpose(1, 2)
        v = v.reshape(b, s, nkv_l, d).transpose(1, 2)
        q, k = rai_cpu.rope_full(q, k, sin, cos, 0)
        k, v = rai_cpu.repeat_kv(k, nq_l // nkv_l), rai_cpu.repeat_kv(v, nq_l // nkv_l)
        a = q.matmul(k.transpose(2, 3)) * (1.0 / d ** 0.5)
        a = rai_cpu.softmax_last(a + mask if mask is not None else a).matmul(v)
        a = a.transpose(1, 2).reshape(b, s, nq_l * d)
        xs = xs + allreduce(rai_cpu.linear(a, w[p + "self_attn.o_proj.weight"], None))
        h = rai_cpu.rms_norm(xs, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        g = rai_cpu.silu(rai_cpu.linear(h, w[p + "mlp.gate_proj.weight"], None)) * rai_cpu.linear(h, w[p + "mlp.up_proj.weight"], None)
        xs = xs + allreduce(rai_cpu.linear(g, w[p + "mlp.down_proj.weight"], None))
    xs = rai_cpu.rms_norm(xs.narrow(1, s - 1, 1), w["model.norm.weight"], cfg["rms_norm_eps"])
    return allgather(rai_cpu.linear(xs, w["lm_head.weight"], None))


def _worker(rank, world, port, cfg, weights, ids, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)

    def allreduce(t):
        t = t.contiguous()
        dist.all_reduce(t)
        return t

    def allgather(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        return torch.cat(parts, -1)

    logits = sharded_forward(cfg, weights, tp.plan(cfg, rank, world), ids, allreduce, allgather)
    if rank == 0:
        out.put(logits.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_match_the_unsharded_oracle():
    cfg = configs.get("tiny-qwen2")
    weights = synth.weights(cfg, 21)
    ids = torch.from_numpy(synth.prompt(cfg, 2, 9, 21).astype(np.int64))
    want = util.build_oracle(cfg, weights).forward(ids, 0)
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, cfg, weights, ids, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = torch.from_numpy(out.get(timeout=120))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert util.rel_error(got, want) < 2e-5


@pytest.mark.parametrize("name,size", [("tiny-qwen2-g7", 2), ("tiny-qwen2-g7", 4), ("tiny-qwen2", 2), ("tiny-qwen2", 8)])
def test_more_ranks_than_kv_heads_with_padding(name, size):
    """Ranks that share a KV head split its query heads, padded with zero heads where the split is
    uneven (7 query heads over 2 or 4 ranks).  All ranks simulated in one process."""
    cfg = configs.get(name)
    if cfg["intermediate_size"] % size or cfg["vocab_size"] % size:
        pytest.skip("sizes do not divide")
    weights = synth.weights(cfg, 22)
    ids = torch.from_numpy(synth.prompt(cfg, 1, 6, 22).astype(np.int64))
    want = util.build_oracle(cfg, weights).forward(ids, 0)
    plans = [tp.plan(cfg, r, size) for r in range(size)]
    # every real query head exactly once, every KV head on size/nkv ranks
    real = sorted(h for p in plans for h in p.q_heads if h >= 0)
    assert real == list(range(cfg["num_attention_heads"]))
    # lock-step simulation: run the ranks as coroutines that meet at each collective
    import threading
    barrier = threading.Barrier(size)
    slots, results = [None] * size, [None] * size

    def run(r):
        def allreduce(t):
            slots[r] = t
            barrier.wait()
            s = sum(slots[1:], slots[0].clone())
            barrier.wait()
            return s

        def allgather(t):
            slots[r] = t
            barrier.wait()
            g = torch.cat(list(slots), -1)
            barrier.wait()
            return g
        results[r] = sharded_forward(cfg, weights, plans[r], ids, allreduce, allgather)

    threads = [threading.Thread(target=run, args=(r,)) for r in range(size)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert util.rel_error(results[0], want) < 2e-5


def test_plan_of_the_7b_configuration_at_eight_ranks():
    cfg = configs.get("qwen2-7b")
    plans = [tp.plan(cfg, r, 8) for r in range(8)]
    assert [p.kv_heads for p in plans] == [[0], [0], [1], [1], [2], [2], [3], [3]]
    assert plans[0].q_heads == [0, 1, 2, 3] and plans[1].q_heads == [4, 5, 6, -1]
    assert plans[7].q_heads == [25, 26, 27, -1]
    assert plans[3].inter == slice(3 * 2368, 4 * 2368) and plans[3].vocab == slice(3 * 19008, 4 * 19008)
    with pytest.raises(ValueError):
        tp.plan(cfg, 0, 3)
