"""The give-up path of the bounded device-side waits, exercised without faulting or hanging anything: kernels whose
wait can never be satisfied run with a 2 ms budget, must return, must name themselves in the status word, must leave
their outputs alone, and the context must work normally afterwards.  Also the robustness fixes around shared
per-context state: the split-KV scratch may grow under a captured decode graph, and the tensor-map cache may be
emptied between two look-ups of one launch."""
import ctypes
import math
import time

import numpy as np
import pytest
import torch

from rai_b200 import _lib, configs, synth
from rai_b200.models import Model

pytestmark = pytest.mark.gpu
P = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731


def small_linear_is_right(cuda, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(8, 256, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(384, 256, generator=g) * 0.05).to(torch.bfloat16).cuda()
    out = torch.empty(8, 384, dtype=torch.bfloat16, device="cuda")
    _lib.call("rb_linear", cuda.ctx, P(x), P(w), None, None, P(out), 8, 384, 256, _lib.ACT_NONE, _lib.BF16)
    _lib.call("rb_sync", cuda.ctx)
    ref = x.cpu().float() @ w.cpu().float().t()
    return float((out.cpu().float() - ref).abs().max()) <= 8e-3 * float(ref.abs().max())


@pytest.mark.parametrize("which,what", [(0, "an mbarrier nobody arrives on"),
                                        (1, "a tensor-parallel peer that never raises its flag"),
                                        (2, "a tensor-parallel peer whose words never show the exchange number"),
                                        (3, "a row's owner that never sends the finished row")])
def test_a_wait_that_cannot_be_satisfied_gives_up_and_reports(cuda, which, what):
    t0 = time.time()
    _lib.call("rb_selftest_wait_gives_up", cuda.ctx, which, 2000)     # 2 ms budget; raises if anything is off
    assert time.time() - t0 < 5.0, f"waiting on {what} took far longer than its budget"
    # the status word is clear again and ordinary work runs
    _lib.call("rb_sync", cuda.ctx)
    assert small_linear_is_right(cuda, which)


def test_wait_budget_setter_validates(cuda):
    with pytest.raises(_lib.RaiB200Error):
        _lib.call("rb_set_wait_budget_us", cuda.ctx, 0)
    with pytest.raises(_lib.RaiB200Error):
        _lib.call("rb_set_wait_budget_us", cuda.ctx, 10**9)
    _lib.call("rb_set_wait_budget_us", cuda.ctx, 500000)
    assert small_linear_is_right(cuda, 3)
    _lib.call("rb_set_wait_budget_us", cuda.ctx, 1000000)


def test_scratch_growth_does_not_break_a_captured_decode_step(cuda):
    """Model A decodes with its captured step; an unrelated attention call on the same context then needs more
    split-KV scratch than anything before it; model A's next steps must be exactly what they are without the
    interruption (and those are checked against the oracle by the model tests)."""
    cfg = configs.get("tiny-qwen2-g7")
    w = synth.weights(cfg, 21)
    prompt = synth.prompt(cfg, 2, 200, 21)      # long enough for the decode attention to split its keys
    steps = 8
    m = Model(cfg, _lib.BF16, cuda, 2, 256)
    m.update_params(w)
    whole = np.asarray(m.generate(prompt, steps))             # uninterrupted: prefill + 7 decode steps
    first = np.asarray(m.generate(prompt, 4))                 # prefill + 3 decode steps: the captured step replays
    assert bool(_lib.lib().rb_model_decode_graph_active(m._m))
    # a much larger decode attention on the same context: more split-KV scratch than the model reserved
    nq, nkv, d, batch, ctx_len = 32, 2, 128, 64, 1500
    cache = ctypes.c_void_p()
    _lib.call("rb_kv_cache_create", cuda.ctx, 1, nkv, d, batch, ctx_len + 8, _lib.BF16, ctypes.byref(cache))
    _lib.call("rb_kv_cache_set_len", cache, batch, ctx_len)
    q = torch.randn(batch, nq * d, dtype=torch.float32).to(torch.bfloat16).cuda()
    out = torch.empty_like(q)
    _lib.call("rb_attention", cuda.ctx, P(q), cache, 0, batch, 1, nq, 1.0 / math.sqrt(d), P(out), _lib.BF16)
    _lib.call("rb_sync", cuda.ctx)
    _lib.call("rb_kv_cache_destroy", cache)
    # model A goes on where it was: its cache holds the prompt and the first three generated tokens
    last = torch.from_numpy(first[:, -1].astype(np.int32)).cuda()
    rest = m.decode_loop(last, prompt.shape[1] + 3, steps - 4)
    cuda.synchronize()
    _lib.call("rb_sync", cuda.ctx)
    got = np.concatenate([first, rest.cpu().numpy().T.astype(np.int64)], axis=1)
    assert (got == whole).all(), "the generation changed after another call grew the context's scratch"
    m.close()


def test_tensor_map_cache_survives_many_distinct_operands(cuda):
    """More distinct operand addresses than the tensor-map cache holds: the cache is emptied along the way (possibly
    between the look-ups of one launch), and every result must still be right."""
    g = torch.Generator().manual_seed(11)
    m_, n_, k_ = 4, 128, 64
    w = (torch.randn(n_, k_, generator=g) * 0.05).to(torch.bfloat16).cuda()
    n_calls = 4300
    pool = torch.randn(n_calls * 8 + m_ * k_, generator=g).to(torch.bfloat16).cuda()   # operand i starts 16 bytes after operand i-1
    out = torch.empty(m_, n_, dtype=torch.bfloat16, device="cuda")
    wf = w.cpu().float()
    pool_f = pool.cpu().float()
    for i in range(n_calls):
        x = pool[i * 8: i * 8 + m_ * k_]
        _lib.call("rb_linear", cuda.ctx, P(x), P(w), None, None, P(out), m_, n_, k_, _lib.ACT_NONE, _lib.BF16)
        if i % 97 == 0 or i >= n_calls - 3:
            _lib.call("rb_sync", cuda.ctx)
            ref = pool_f[i * 8: i * 8 + m_ * k_].reshape(m_, k_) @ wf.t()
            assert float((out.cpu().float() - ref).abs().max()) <= 8e-3 * float(ref.abs().max()) + 1e-6, f"call {i}"
    _lib.call("rb_sync", cuda.ctx)
