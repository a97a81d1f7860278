"""rb_attention_decode_static: the decode-attention entry point for callers that may not allocate.

Some users of this library cannot let it call cudaMalloc: a host runtime that owns every byte of
device memory through its own pool, or a serving loop where an allocation's device-wide
synchronisation is not acceptable.  rb_attention grows its split-KV scratch on demand; the static
variant keeps that scratch in a fixed array inside the library.  This test calls the new entry point
through the C ABI twice in a row and checks both results against rb_attention on the same inputs
(the two run the same kernels, so they must agree exactly; this is a bit-identity check between two entry points -
rb_attention itself is held to the CPU oracle by test_gpu_30_attention.py - and it does cross two merge paths, the merge
kernel here against the last-arriving block there), and checks that an over-size shape is refused with a clear message.  It lives in the last-collected file so that a run which stops at the
first failure has already run everything else."""
import ctypes
import math

import pytest
import torch

from rai_b200 import _lib

pytestmark = pytest.mark.gpu
P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731


def make_cache(cuda, layers, kvh, d, batch, max_seq):
    h = ctypes.c_void_p()
    _lib.call("rb_kv_cache_create", cuda.ctx, layers, kvh, d, batch, max_seq, _lib.BF16, ctypes.byref(h))
    return h


def fill(cuda, cache, batch, n_tokens, nq, nkv, d, seed):
    """Appends n_tokens random tokens per sequence (as one prefill), returns nothing."""
    g = torch.Generator().manual_seed(seed)
    cos = torch.empty(n_tokens + 8, d // 2, dtype=torch.float32, device="cuda")
    sin = torch.empty_like(cos)
    _lib.call("rb_rope_tables", cuda.ctx, 0, d, n_tokens + 8, 1e4, P(cos), P(sin))
    qkv = torch.randn(batch * n_tokens, (nq + 2 * nkv) * d, generator=g).to(torch.bfloat16).cuda()
    q = torch.empty(batch * n_tokens, nq * d, dtype=torch.bfloat16, device="cuda")
    _lib.call("rb_kv_cache_set_len", cache, batch, n_tokens)
    _lib.call("rb_rope_kv_append", cuda.ctx, P(qkv), None, 0, None, P(cos), P(sin), d, batch, n_tokens, nq, cache, 0,
              P(q), _lib.BF16)
    cuda.synchronize()


@pytest.mark.parametrize("nq,nkv,d,batch,ctx_len", [(4, 2, 128, 2, 700), (8, 1, 64, 3, 330), (28, 4, 128, 64, 200)])
def test_static_scratch_attention_matches_rb_attention_twice(cuda, nq, nkv, d, batch, ctx_len):
    cache = make_cache(cuda, 1, nkv, d, batch, ctx_len + 8)
    fill(cuda, cache, batch, ctx_len, nq, nkv, d, seed=nq + d)
    g = torch.Generator().manual_seed(7)
    scale = 1.0 / math.sqrt(d)
    for call in range(2):  # two calls in a row share the built-in array
        q = torch.randn(batch, nq * d, generator=g).to(torch.bfloat16).cuda()
        want = torch.empty_like(q)
        got = torch.full_like(q, float("nan"))
        _lib.call("rb_attention", cuda.ctx, P(q), cache, 0, batch, 1, nq, scale, P(want), _lib.BF16)
        _lib.call("rb_attention_decode_static", cuda.ctx, P(q), cache, 0, batch, nq, scale, P(got))
        cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want), f"call {call}: max diff {(got.float() - want.float()).abs().max()}"
    _lib.call("rb_kv_cache_destroy", cache)


def test_static_scratch_attention_refuses_shapes_beyond_its_array(cuda):
    # 9 sequences x 64 heads x 4 splits x (256 + 2) floats = 594,432 > 512 Ki floats
    # (36 (sequence, KV head) pairs on 148 SMs, one resident block each at this head size: the library splits the keys 4 ways)
    nq, nkv, d, batch, ctx_len = 64, 4, 256, 9, 4200
    cache = make_cache(cuda, 1, nkv, d, batch, ctx_len + 8)
    _lib.call("rb_kv_cache_set_len", cache, batch, ctx_len)
    q = torch.zeros(batch, nq * d, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(q)
    with pytest.raises(_lib.RaiB200Error) as e:
        _lib.call("rb_attention_decode_static", cuda.ctx, P(q), cache, 0, batch, nq, 0.1, P(out))
    assert e.value.code == -1 and "scratch floats" in str(e.value)
    _lib.call("rb_kv_cache_destroy", cache)
