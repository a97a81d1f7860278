"""RoPE + paged KV append + attention against the CPU oracle, prefill and decode, every head size."""
import ctypes
import math

import pytest
import torch

import rai_cpu
from rai_b200 import _lib

pytestmark = pytest.mark.gpu
P = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


class Cache:
    def __init__(self, cuda, layers, kvh, d, max_batch, max_seq, dtype):
        self.h = ctypes.c_void_p()
        _lib.call("rb_kv_cache_create", cuda.ctx, layers, kvh, d, max_batch, max_seq, DT[dtype], ctypes.byref(self.h))
        self.d, self.dtype = d, dtype

    def set_len(self, batch, n):
        _lib.call("rb_kv_cache_set_len", self.h, batch, n)

    def read(self, layer, seq, kvh, t0, n):
        k = torch.empty(n, self.d, dtype=self.dtype)
        v = torch.empty(n, self.d, dtype=self.dtype)
        _lib.call("rb_kv_cache_read", self.h, layer, seq, kvh, t0, n, P(k), P(v))
        return k, v

    def close(self):
        _lib.call("rb_kv_cache_destroy", self.h)


def oracle_attention(q, k, v, offset, nq, nkv, d, rot, sin, cos):
    """q [B,S,nq*d], k/v [B,T,nkv*d] un-rotated (T = offset + S) -> attention output [B,S,nq*d] and
    the rotated keys, through the reference's op sequence."""
    b, s, _ = q.shape
    t = k.shape[1]
    qh = q.reshape(b, s, nq, d).transpose(1, 2)
    kh = k.reshape(b, t, nkv, d).transpose(1, 2)
    vh = v.reshape(b, t, nkv, d).transpose(1, 2)
    if rot == d:
        qh, _ = rai_cpu.rope_full(qh, qh, sin, cos, offset)
        kh, _ = rai_cpu.rope_full(kh, kh, sin, cos, 0)
    else:
        qh = rai_cpu.rope_partial(qh, sin, cos, rot, offset)
        kh = rai_cpu.rope_partial(kh, sin, cos, rot, 0)
    kr, vr = rai_cpu.repeat_kv(kh, nq // nkv), rai_cpu.repeat_kv(vh, nq // nkv)
    w = qh.matmul(kr.transpose(2, 3)) * (1.0 / math.sqrt(d))
    if s > 1:
        w = w + rai_cpu.additive_causal_mask(b, s, offset)
    o = rai_cpu.softmax_last(w).matmul(vr)
    return o.transpose(1, 2).reshape(b, s, nq * d), kh


CASES = [  # (nq, nkv, d, rot, batch, prompt, decode steps)
    (4, 2, 64, 64, 2, 70, 3),
    (2, 2, 80, 32, 2, 33, 2),      # phi2: partial rotary, head_dim 80
    (2, 2, 96, 96, 1, 129, 2),     # phi3 head size
    (7, 1, 128, 128, 3, 200, 3),   # 7 query heads per KV head (the 7B grouping)
    (8, 1, 256, 256, 2, 65, 2),    # gemma: MQA, head_dim 256
    (4, 4, 128, 128, 1, 1, 4),     # one-token prompt
    (14, 2, 64, 64, 2, 640, 2),    # long enough for several KV splits at decode
    (1, 1, 64, 64, 2, 40, 6),      # one query head on one KV head (an 8-way shard of a small model)
    (1, 1, 64, 64, 2, 64, 6),
    (1, 1, 64, 64, 2, 100, 6),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("nq,nkv,d,rot,batch,prompt,steps", CASES)
def test_rope_append_attention_matches_oracle(cuda, dtype, nq, nkv, d, rot, batch, prompt, steps):
    g = torch.Generator().manual_seed(nq * 100 + d)
    max_seq = prompt + steps + 5
    cache = Cache(cuda, 2, nkv, d, batch, max_seq, dtype)
    layer = 1
    ncol = (nq + 2 * nkv) * d
    recipe, name = (1, "phi2") if rot != d else (0, "qwen2")
    cos = torch.empty(max_seq + 64, rot // 2, dtype=torch.float32, device="cuda")
    sin = torch.empty_like(cos)
    _lib.call("rb_rope_tables", cuda.ctx, recipe, rot, max_seq + 64, 1e4, P(cos), P(sin))
    s_ref, c_ref = rai_cpu.rope_tables(rot, max_seq + 64, 1e4, name)
    tol = 2.5e-2 if dtype == torch.bfloat16 else 3e-5
    k_all = torch.empty(batch, 0, nkv * d)
    v_all = torch.empty(batch, 0, nkv * d)
    pos = 0
    for step in range(steps + 1):
        s_new = prompt if step == 0 else 1
        qkv = (torch.randn(batch * s_new, ncol, generator=g)).to(dtype)
        qkv_d = qkv.cuda()
        q_out = torch.empty(batch * s_new, nq * d, dtype=dtype, device="cuda")
        out = torch.empty_like(q_out)
        cache.set_len(batch, pos + s_new)
        _lib.call("rb_rope_kv_append", cuda.ctx, P(qkv_d), None, 0, None, P(cos), P(sin), rot, batch, s_new, nq,
                  cache.h, layer, P(q_out), DT[dtype])
        _lib.call("rb_attention", cuda.ctx, P(q_out), cache.h, layer, batch, s_new, nq, 1.0 / math.sqrt(d), P(out),
                  DT[dtype])
        cuda.synchronize()
        f = qkv.float().reshape(batch, s_new, ncol)
        k_all = torch.cat([k_all, f[:, :, nq * d:(nq + nkv) * d]], 1)
        v_all = torch.cat([v_all, f[:, :, (nq + nkv) * d:]], 1)
        ref, k_rot = oracle_attention(f[:, :, : nq * d], k_all, v_all, pos, nq, nkv, d, rot, s_ref, c_ref)
        got = out.cpu().float().reshape(batch, s_new, nq * d)
        assert float((got - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max())), f"step {step}"
        pos += s_new
    # KV-cache indexing: V rows are stored untouched (bit for bit), K rows are the rotated keys
    for b in range(batch):
        for h in range(nkv):
            kc, vc = cache.read(layer, b, h, 0, pos)
            assert torch.equal(vc.float(), v_all[b, :, h * d:(h + 1) * d].to(dtype).float())
            assert float((kc.float() - k_rot[b, h]).abs().max()) <= tol * float(k_rot.abs().max())
    # the other layer of the cache was never written
    kc, vc = cache.read(0, 0, 0, 0, pos)
    assert float(kc.float().abs().max()) == 0.0 and float(vc.float().abs().max()) == 0.0
    cache.close()


def test_rope_append_from_partials_and_bias(cuda):
    """The split-K form: qkv arrives as float32 partial slabs plus a bias."""
    g = torch.Generator().manual_seed(5)
    nq, nkv, d, batch = 4, 2, 64, 3
    ncol = (nq + 2 * nkv) * d
    cache = Cache(cuda, 1, nkv, d, batch, 64, torch.bfloat16)
    cos = torch.empty(64, d // 2, dtype=torch.float32, device="cuda")
    sin = torch.empty_like(cos)
    _lib.call("rb_rope_tables", cuda.ctx, 0, d, 64, 1e6, P(cos), P(sin))
    acc = torch.randn(3, batch, ncol, generator=g).cuda()
    bias = torch.randn(ncol, generator=g).to(torch.bfloat16).cuda()
    total = (acc.sum(0) + bias.float()).to(torch.bfloat16)
    qa = torch.empty(batch, nq * d, dtype=torch.bfloat16, device="cuda")
    qb = torch.empty_like(qa)
    cache.set_len(batch, 1)
    _lib.call("rb_rope_kv_append", cuda.ctx, None, P(acc), 3, P(bias), P(cos), P(sin), d, batch, 1, nq, cache.h, 0,
              P(qa), _lib.BF16)
    cuda.synchronize()
    _, va = cache.read(0, 1, 1, 0, 1)
    _lib.call("rb_rope_kv_append", cuda.ctx, P(total), None, 0, None, P(cos), P(sin), d, batch, 1, nq, cache.h, 0,
              P(qb), _lib.BF16)
    cuda.synchronize()
    _, vb = cache.read(0, 1, 1, 0, 1)
    # position 0 rotates by nothing, so both routes store the rounded sum itself
    assert torch.equal(qa, total[:, : nq * d]) and torch.equal(qb, qa) and torch.equal(va, vb)
    cache.close()


def test_append_beyond_capacity_is_rejected(cuda):
    cache = Cache(cuda, 1, 1, 64, 1, 64, torch.bfloat16)
    with pytest.raises(_lib.RaiB200Error):
        cache.set_len(1, 65)
    with pytest.raises(_lib.RaiB200Error):
        cache.set_len(2, 1)
    cache.close()
