"""The sliding-window term of qwen2's mask (rai-models/src/llm/qwen2.rs:316-327: key j is hidden from query i when
j + sliding_window < i) against the CPU oracle: at the attention call with a cache-level window, and through a
whole qwen2 model whose configured window is shorter than its context (prefill, chunked prefill and decode)."""
import ctypes
import math

import numpy as np
import pytest
import torch

import rai_cpu
import util
from rai_b200 import _lib, configs, synth
from rai_b200.models import Model

pytestmark = pytest.mark.gpu
P = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("window", [0, 5, 63, 64, 100])
def test_attention_honours_the_window(cuda, dtype, window):
    nq, nkv, d, batch, prompt, steps = 4, 2, 64, 2, 150, 3
    g = torch.Generator().manual_seed(window + 7)
    cache = ctypes.c_void_p()
    _lib.call("rb_kv_cache_create", cuda.ctx, 1, nkv, d, batch, 256, DT[dtype], ctypes.byref(cache))
    _lib.call("rb_kv_cache_set_window", cache, window)
    tol = 2.5e-2 if dtype == torch.bfloat16 else 3e-5
    k_all = torch.empty(batch, nkv, 0, d)
    v_all = torch.empty(batch, nkv, 0, d)
    pos = 0
    for step in range(steps + 1):
        s_new = prompt if step == 0 else 1
        q = torch.randn(batch, s_new, nq * d, generator=g).to(dtype)
        kv = torch.randn(batch, s_new, 2 * nkv * d, generator=g).to(dtype)
        # no rotation (rot = 0): the test is about the mask
        qkv_d = torch.cat([q, kv], dim=2).reshape(batch * s_new, -1).cuda()
        q_out = torch.empty(batch * s_new, nq * d, dtype=dtype, device="cuda")
        out = torch.empty_like(q_out)
        dummy = torch.zeros(256, 1, dtype=torch.float32, device="cuda")
        _lib.call("rb_kv_cache_set_len", cache, batch, pos + s_new)
        _lib.call("rb_rope_kv_append", cuda.ctx, P(qkv_d), None, 0, None, P(dummy), P(dummy), 0, batch, s_new, nq, cache, 0,
                  P(q_out), DT[dtype])
        _lib.call("rb_attention", cuda.ctx, P(q_out), cache, 0, batch, s_new, nq, 1.0 / math.sqrt(d), P(out), DT[dtype])
        cuda.synchronize()
        f = kv.float()
        k_all = torch.cat([k_all, f[:, :, : nkv * d].reshape(batch, s_new, nkv, d).transpose(1, 2)], 2)
        v_all = torch.cat([v_all, f[:, :, nkv * d:].reshape(batch, s_new, nkv, d).transpose(1, 2)], 2)
        qh = q.float().reshape(batch, s_new, nq, d).transpose(1, 2)
        w = qh.matmul(rai_cpu.repeat_kv(k_all, nq // nkv).transpose(2, 3)) * (1.0 / math.sqrt(d))
        # the reference adds the mask for every seq_len > 1 and none at seq_len 1 (qwen2.rs:346); with a window shorter
        # than the context the decode step needs the window term too, which is what the mask rule states
        w = w + rai_cpu.additive_causal_mask(batch, s_new, pos, window)
        ref = rai_cpu.softmax_last(w).matmul(rai_cpu.repeat_kv(v_all, nq // nkv)).transpose(1, 2).reshape(batch, s_new, nq * d)
        got = out.cpu().float().reshape(batch, s_new, nq * d)
        assert float((got - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max())), f"window {window} step {step}"
        pos += s_new
    _lib.call("rb_kv_cache_destroy", cache)


@pytest.mark.parametrize("dtype,tol", [(_lib.F32, 1e-4), (_lib.BF16, 2e-2)])
def test_qwen2_model_with_a_short_window(cuda, dtype, tol):
    cfg = configs.get("tiny-qwen2")
    cfg["sliding_window"] = 24           # shorter than the 70-token prompt
    w = synth.weights(cfg, 5)
    ids = synth.prompt(cfg, 2, 70, 5)
    steps = 4
    # the oracle feeds the prompt in one piece, so its mask carries the window; the GPU side is fed the same prompt
    want, ref = rai_cpu.greedy_generate(util.build_oracle(cfg, w), torch.from_numpy(ids.astype(np.int64)), 1, True)
    m = Model(cfg, dtype, cuda, 2, 128)
    m.update_params(w)
    logits = m.forward(ids, 0).reshape(2, -1)
    err = util.logit_error(logits, ref[0]) if dtype == _lib.BF16 else util.rel_error(logits, ref[0])
    assert err <= tol, f"prefill with a 24-token window: error {err:.2e}"
    # without the window the logits must differ visibly: the test would otherwise prove nothing
    cfg2 = dict(cfg, sliding_window=4096)
    m2 = Model(cfg2, dtype, cuda, 2, 128)
    m2.update_params(w)
    other = m2.forward(ids, 0).reshape(2, -1)
    assert util.logit_error(other, ref[0]) > 10 * tol
    m.close()
    m2.close()
