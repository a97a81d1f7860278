"""The single-token step as one kernel (rb_rope_attention_decode) against the two separate calls it replaces
(rb_rope_kv_append then rb_attention): attention output and the appended K/V rows must be identical bit for
bit, for every input form (bf16 rows, float32 split-K partials, bias), group size, page boundary and KV split.

This is a bit-identity check between two entry points of the same library, not a parity check: the separate path is
held to the CPU oracle by test_gpu_30_attention.py, the fused path by the model tests (every decode step they run goes
through it) and, at the benchmark's shape, by test_gpu_33_attention_bench_shapes.py."""
import ctypes
import math

import pytest
import torch

from rai_b200 import _lib
from test_gpu_30_attention import Cache, P

pytestmark = pytest.mark.gpu
BF = torch.bfloat16

CASES = [  # (nq, nkv, d, rot, batch, tokens already cached, form)
    (4, 2, 64, 64, 2, 0, "rows"),          # the very first token
    (4, 2, 64, 64, 2, 62, "rows"),         # new token is the last slot of a page
    (4, 2, 64, 64, 2, 63, "partials"),     # ... the first slot of the next page
    (4, 2, 64, 32, 3, 64, "partials+bias"),  # partial rotary
    (7, 1, 128, 128, 3, 200, "partials+bias"),
    (28, 4, 128, 128, 4, 300, "partials+bias"),   # the 7B grouping
    (8, 1, 256, 256, 2, 65, "rows"),       # gemma: MQA, head_dim 256
    (16, 1, 128, 128, 2, 130, "rows+partials"),   # a full 16-row query tile
    (14, 2, 64, 64, 2, 1500, "partials"),  # several KV splits: only the last one appends
    (1, 1, 64, 64, 2, 1000, "rows"),       # one head per KV head, split
    (4, 4, 128, 64, 1, 1023, "partials+bias"),
    (2, 2, 80, 32, 2, 33, "rows"),            # phi2: head_dim 80, partial rotary, padded-row loads
    (4, 4, 80, 32, 3, 200, "partials+bias"),
    (2, 2, 96, 96, 1, 129, "partials"),       # phi3 head size
    (8, 8, 96, 96, 2, 700, "rows+partials"),  # several KV splits on the padded-row path
]


@pytest.mark.parametrize("nq,nkv,d,rot,batch,cached,form", CASES)
def test_fused_step_equals_separate_calls(cuda, nq, nkv, d, rot, batch, cached, form):
    g = torch.Generator().manual_seed(nq * 1000 + d + cached)
    max_seq = cached + 8
    ncol = (nq + 2 * nkv) * d
    scale = 1.0 / math.sqrt(d)
    cos = torch.empty(max_seq + 64, rot // 2, dtype=torch.float32, device="cuda")
    sin = torch.empty_like(cos)
    _lib.call("rb_rope_tables", cuda.ctx, 1 if rot != d else 0, rot, max_seq + 64, 1e4, P(cos), P(sin))
    caches = [Cache(cuda, 2, nkv, d, batch, max_seq, BF) for _ in range(2)]
    layer = 1
    if cached:
        prior = torch.randn(batch * cached, ncol, generator=g).to(BF).cuda()
        q_tmp = torch.empty(batch * cached, nq * d, dtype=BF, device="cuda")
        for c in caches:
            c.set_len(batch, cached)
            _lib.call("rb_rope_kv_append", cuda.ctx, P(prior), None, 0, None, P(cos), P(sin), rot, batch, cached, nq, c.h,
                      layer, P(q_tmp), _lib.BF16)
    outs, rows = [], []
    for step in range(3):                                   # three steps in a row: each sees the previous one's append
        n_acc = 3 if "partials" in form else 0
        qkv = torch.randn(batch, ncol, generator=g).to(BF).cuda() if "rows" in form else None
        acc = torch.randn(n_acc, batch, ncol, generator=g).cuda() if n_acc else None
        bias = torch.randn(ncol, generator=g).to(BF).cuda() if "bias" in form else None
        pos = cached + step
        got = []
        for fused, c in zip((False, True), caches):
            c.set_len(batch, pos + 1)
            q_s = torch.zeros(batch, nq * d, dtype=BF, device="cuda")
            out = torch.empty(batch, nq * d, dtype=BF, device="cuda")
            if fused:
                _lib.call("rb_rope_attention_decode", cuda.ctx, P(qkv), P(acc), n_acc, P(bias), P(cos), P(sin), rot, batch, nq,
                          c.h, layer, scale, P(q_s), P(out), _lib.BF16)
            else:
                _lib.call("rb_rope_kv_append", cuda.ctx, P(qkv), P(acc), n_acc, P(bias), P(cos), P(sin), rot, batch, 1, nq,
                          c.h, layer, P(q_s), _lib.BF16)
                _lib.call("rb_attention", cuda.ctx, P(q_s), c.h, layer, batch, 1, nq, scale, P(out), _lib.BF16)
            cuda.synchronize()
            got.append(out.cpu())
        assert torch.isfinite(got[0].float()).all()
        assert torch.equal(got[0], got[1]), f"step {step}: outputs differ by {float((got[0].float() - got[1].float()).abs().max()):.3e}"
    for b in range(batch):
        for h in range(nkv):
            t0 = max(0, cached - 2)
            ka, va = caches[0].read(layer, b, h, t0, cached + 3 - t0)
            kb, vb = caches[1].read(layer, b, h, t0, cached + 3 - t0)
            assert torch.equal(ka, kb) and torch.equal(va, vb), f"cache rows of sequence {b}, KV head {h} differ"
    status = (ctypes.c_uint32 * 4)()
    _lib.call("rb_status_word", cuda.ctx, status)
    assert status[0] == 0
    for c in caches:
        c.close()
