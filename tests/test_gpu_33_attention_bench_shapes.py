"""Decode attention at the shape the benchmark times, against the CPU oracle: 28 query heads over 4 KV heads,
head_dim 128, batch 64, a 2048-token cache that grows to 2052 (33 key tiles per sequence, one block per
(sequence, KV head)), bf16.  Both routes are checked: rb_rope_kv_append + rb_attention, and the fused
single-token step rb_rope_attention_decode (RoPE, cache append and attention in one kernel).

The oracle follows rai-models/src/llm/qwen2.rs:176-216 op for op, except that the repeated K/V heads of
repeat_kv (a pure copy, gemma.rs:191-201) are addressed through a [kv_head, group] view instead of being
materialised 7 times: at this size the copies alone would be 4 GB of float32.
"""
import ctypes
import math

import pytest
import torch

import rai_cpu
from rai_b200 import _lib

pytestmark = pytest.mark.gpu
P = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731

NQ, NKV, D, BATCH, CTX, STEPS = 28, 4, 128, 64, 2048, 4


def oracle_decode(q, k_rot, v, pos, sin, cos):
    """q [B, NQ*D] un-rotated, k_rot [B, NKV, T, D] rotated keys, v [B, NKV, T, D] -> [B, NQ*D]."""
    b = q.shape[0]
    qh = q.reshape(b, 1, NQ, D).transpose(1, 2)                      # [B, NQ, 1, D]
    qh, _ = rai_cpu.rope_full(qh, qh, sin, cos, pos)
    g = NQ // NKV
    qg = qh.reshape(b, NKV, g, D)                                     # query heads grouped by their KV head
    w = qg.matmul(k_rot.transpose(2, 3)) * (1.0 / math.sqrt(D))      # [B, NKV, G, T]; no mask at seq_len 1 (qwen2.rs:346)
    o = rai_cpu.softmax_last(w).matmul(v)                            # [B, NKV, G, D]
    return o.reshape(b, NQ * D)


@pytest.mark.parametrize("fused", [False, True])
def test_decode_attention_at_the_benchmark_shape(cuda, fused):
    g = torch.Generator().manual_seed(2048 + int(fused))
    max_seq = CTX + STEPS + 8
    cache = ctypes.c_void_p()
    _lib.call("rb_kv_cache_create", cuda.ctx, 1, NKV, D, BATCH, max_seq, _lib.BF16, ctypes.byref(cache))
    cos = torch.empty(max_seq, D // 2, dtype=torch.float32, device="cuda")
    sin = torch.empty_like(cos)
    _lib.call("rb_rope_tables", cuda.ctx, 0, D, max_seq, 1e6, P(cos), P(sin))
    s_ref, c_ref = rai_cpu.rope_tables(D, max_seq, 1e6, "qwen2")

    # ---- fill the cache: 2048 tokens per sequence through the append kernel (one query head per KV head is
    # enough for the fill; the cache layout does not depend on the number of query heads)
    k_raw = torch.randn(BATCH, CTX, NKV * D, generator=g).to(torch.bfloat16)
    v_raw = torch.randn(BATCH, CTX, NKV * D, generator=g).to(torch.bfloat16)
    fill = torch.cat([torch.zeros(BATCH, CTX, NKV * D, dtype=torch.bfloat16), k_raw, v_raw], dim=2).reshape(BATCH * CTX, 3 * NKV * D)
    fill_d = fill.cuda()
    q_fill = torch.empty(BATCH * CTX, NKV * D, dtype=torch.bfloat16, device="cuda")
    _lib.call("rb_kv_cache_set_len", cache, BATCH, CTX)
    _lib.call("rb_rope_kv_append", cuda.ctx, P(fill_d), None, 0, None, P(cos), P(sin), D, BATCH, CTX, NKV, cache, 0,
              P(q_fill), _lib.BF16)
    cuda.synchronize()
    del fill, fill_d, q_fill
    kh = k_raw.float().reshape(BATCH, CTX, NKV, D).transpose(1, 2)
    k_rot, _ = rai_cpu.rope_full(kh, kh, s_ref, c_ref, 0)
    k_rot = k_rot.to(torch.bfloat16).float()                         # the cache stores bf16
    v_all = v_raw.float().reshape(BATCH, CTX, NKV, D).transpose(1, 2).contiguous()

    ncol = (NQ + 2 * NKV) * D
    scale = 1.0 / math.sqrt(D)
    worst = 0.0
    for step in range(STEPS):
        pos = CTX + step
        qkv = torch.randn(BATCH, ncol, generator=g).to(torch.bfloat16)
        qkv_d = qkv.cuda()
        q_out = torch.empty(BATCH, NQ * D, dtype=torch.bfloat16, device="cuda")
        out = torch.empty_like(q_out)
        _lib.call("rb_kv_cache_set_len", cache, BATCH, pos + 1)
        if fused:
            _lib.call("rb_rope_attention_decode", cuda.ctx, P(qkv_d), None, 0, None, P(cos), P(sin), D, BATCH, NQ, cache, 0,
                      scale, P(q_out), P(out), _lib.BF16)
        else:
            _lib.call("rb_rope_kv_append", cuda.ctx, P(qkv_d), None, 0, None, P(cos), P(sin), D, BATCH, 1, NQ, cache, 0,
                      P(q_out), _lib.BF16)
            _lib.call("rb_attention", cuda.ctx, P(q_out), cache, 0, BATCH, 1, NQ, scale, P(out), _lib.BF16)
        cuda.synchronize()
        f = qkv.float()
        k_new = f[:, NQ * D:(NQ + NKV) * D].reshape(BATCH, 1, NKV, D).transpose(1, 2)
        k_new, _ = rai_cpu.rope_full(k_new, k_new, s_ref, c_ref, pos)
        k_rot = torch.cat([k_rot, k_new.to(torch.bfloat16).float()], dim=2)
        v_all = torch.cat([v_all, f[:, (NQ + NKV) * D:].reshape(BATCH, 1, NKV, D).transpose(1, 2)], dim=2)
        ref = oracle_decode(f[:, : NQ * D], k_rot, v_all, pos, s_ref, c_ref)
        got = out.cpu().float()
        err = float((got - ref).abs().max()) / max(1.0, float(ref.abs().max()))
        worst = max(worst, err)
        assert err <= 2.5e-2, f"step {step}: attention output differs from the oracle by {err:.2e}"
    # KV-cache indexing stays bit-exact at this size: the last appended V row of the last sequence and KV head
    k_host = torch.empty(1, D, dtype=torch.bfloat16)
    v_host = torch.empty(1, D, dtype=torch.bfloat16)
    _lib.call("rb_kv_cache_read", cache, 0, BATCH - 1, NKV - 1, CTX + STEPS - 1, 1, P(k_host), P(v_host))
    assert torch.equal(v_host.float()[0], v_all[BATCH - 1, NKV - 1, -1])
    _lib.call("rb_kv_cache_destroy", cache)
    print(f"decode attention at batch {BATCH}, context {CTX}: worst error {worst:.2e} ({'fused' if fused else 'separate'})")
