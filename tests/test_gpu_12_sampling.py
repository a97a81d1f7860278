"""The sampling of the examples' generation loops on the device (examples/qwen2/src/main.rs:32-53,84-96):
repeat penalty over the context window as a set, float32 total-order argmax with the last index among
equals, and the end-of-sequence rule.  Integer results: bit-exact against the CPU oracle."""
import ctypes

import numpy as np
import pytest
import torch

import rai_cpu
import util
from rai_b200 import _lib, configs, synth
from rai_b200.models import Model

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _sample(cuda, logits, penalty, context, counts, eos=-1, finished=None):
    dev = f"cuda:{cuda.id}"
    rows, cols = logits.shape
    x = logits.to(dev).contiguous()
    out = torch.empty((rows,), dtype=torch.int32, device=dev)
    ctx_d = torch.from_numpy(context.astype(np.int32)).to(dev).contiguous() if context is not None else None
    cnt_d = torch.from_numpy(counts.astype(np.int32)).to(dev).contiguous() if counts is not None else None
    cuda.use_torch_stream()
    _lib.call("rb_sample_greedy", cuda.ctx, _ptr(x), _lib.BF16 if x.dtype == torch.bfloat16 else _lib.F32, rows, cols,
              float(penalty), _ptr(ctx_d), 0 if context is None else context.shape[1], _ptr(cnt_d), int(eos), _ptr(finished),
              _ptr(out))
    cuda.synchronize()
    return out.cpu().numpy()


def _oracle(logits, penalty, context, counts):
    want = []
    for r in range(logits.shape[0]):
        row = logits[r].float()
        if penalty >= 1.0 and context is not None:
            valid = min(int(counts[r]), context.shape[1])
            row = rai_cpu.apply_repeat_penalty(row, penalty, context[r, :valid])
        want.append(rai_cpu.sample_argmax(row))
    return np.asarray(want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols,stride", [(1, 512, 64), (7, 1000, 5), (64, 152064, 64), (3, 32064, 256), (130, 4099, 17)])
def test_penalised_argmax_is_bit_exact(cuda, dtype, rows, cols, stride):
    g = np.random.default_rng(rows * 1000 + cols + stride)
    x = torch.from_numpy(g.standard_normal((rows, cols)).astype(np.float32)).to(dtype)
    context = g.integers(0, cols, size=(rows, stride))
    counts = g.integers(0, 3 * stride, size=(rows,))
    counts[0] = 0 if rows > 1 else stride                      # an empty window; full when it is the only row
    for r in range(rows):
        top = torch.topk(x[r].float(), 6).indices.numpy()
        context[r, : min(3, stride)] = top[: min(3, stride)]      # the leaders are penalised, so the winner changes
        if stride >= 5:
            context[r, 3] = context[r, 0]                         # a repeated id must be penalised once, not twice
            context[r, 4] = int(torch.argmin(x[r].float()))       # a negative logit is multiplied
    if rows >= 3:
        x[1, cols - 1] = x[1].float().max() + 1                   # unpenalised maximum at the very end
        x[2, 5] = x[2, 700] = x[2].float().max() + 2              # two equal maxima: the last index wins
        context[2, :] = 1
    for penalty in (1.10, 1.0, 3.5, 0.5):
        got = _sample(cuda, x, penalty, context, counts)
        assert np.array_equal(got, _oracle(x, penalty, context, counts)), f"penalty {penalty}"
    # no window at all is plain argmax
    assert np.array_equal(_sample(cuda, x, 1.1, None, None), _oracle(x, 0.0, None, None))


def test_total_order_special_values(cuda):
    x = torch.zeros((4, 64), dtype=torch.float32)
    x[0, :] = -0.0
    x[0, 10] = 0.0                                                # +0.0 beats -0.0 under total_cmp
    x[1, :] = -float("inf")
    x[1, 3] = -3.0e38
    x[2, :] = -1.0
    x[2, 7] = float("inf")
    x[2, 9] = float("inf")
    x[3, :] = 5.0                                                 # all equal: the last index
    context = np.array([[10], [3], [9], [63]])
    counts = np.ones((4,), dtype=np.int32)
    for penalty in (0.0, 1.1):
        got = _sample(cuda, x, penalty, context, counts)
        assert np.array_equal(got, _oracle(x, penalty, context, counts)), f"penalty {penalty}: {got}"


def test_end_of_sequence_rule(cuda):
    dev = f"cuda:{cuda.id}"
    x = torch.zeros((3, 100), dtype=torch.float32)
    x[0, 42] = 1.0
    x[1, 7] = 1.0
    x[2, 42] = 1.0
    finished = torch.zeros((3,), dtype=torch.uint8, device=dev)
    assert list(_sample(cuda, x, 0.0, None, None, eos=42, finished=finished)) == [42, 7, 42]
    assert list(finished.cpu().numpy()) == [1, 0, 1]
    y = torch.zeros((3, 100), dtype=torch.float32)
    y[:, 9] = 1.0
    assert list(_sample(cuda, y, 0.0, None, None, eos=42, finished=finished)) == [42, 9, 42]   # finished rows stay finished
    assert list(finished.cpu().numpy()) == [1, 0, 1]


@pytest.mark.parametrize("name,dtype", [("tiny-qwen2", _lib.F32), ("tiny-qwen2", _lib.BF16), ("tiny-phi2", _lib.F32),
                                        ("tiny-qwen2-g7", _lib.BF16)])
@pytest.mark.parametrize("last_n", [64, 6])
def test_generation_loop_with_penalty_and_eos(cuda, name, dtype, last_n):
    """generate_step + the captured decode loop with the examples' sampling against the oracle's loop: the
    window (prompt and generated tokens, wrapping when it is shorter than the sequence), the penalty and the
    stop rule all have to agree for the token streams to be identical."""
    cfg = configs.get(name)
    w = synth.weights(cfg, 5)
    batch, prompt_len, steps, penalty = 3, 20, 40, 1.10
    ids = synth.prompt(cfg, batch, prompt_len, 6)
    oracle = util.build_oracle(cfg, w)
    free = rai_cpu.generate_with_penalty(oracle, torch.from_numpy(ids.astype(np.int64)), steps, penalty, last_n)
    eos = int(free[0, 12])                                        # a token the first sequence does produce
    want, ref = rai_cpu.generate_with_penalty(oracle, torch.from_numpy(ids.astype(np.int64)), steps, penalty, last_n, eos, True)
    assert bool((want[0] == eos).any())
    plain = rai_cpu.greedy_generate(oracle, torch.from_numpy(ids.astype(np.int64)), steps)
    assert not torch.equal(plain, want), "the case must be one where the sampling rule changes the tokens"
    m = Model(cfg, dtype, cuda, 4, 128, batch * prompt_len)
    m.update_params(w)
    m.set_sampling(penalty, last_n, eos)
    for attempt in range(2):                                      # the second run re-uses the history buffers
        got = m.generate(ids, steps)
        for b in range(batch):
            hist = [int(t) for t in ids[b]]
            for t in range(steps):
                if got[b, t] != int(want[b, t]):
                    # only excusable at a near-tie of the PENALISED reference logits
                    row = rai_cpu.apply_repeat_penalty(ref[t, b], penalty, hist[max(0, len(hist) - last_n):])
                    margin, rng = float(util.top2_margin(row)), float(row.max() - row.min())
                    tol = (1e-4 if dtype == _lib.F32 else 2e-2) * rng
                    assert margin < tol, f"{name} run {attempt} seq {b} step {t}: got {got[b, t]} want {int(want[b, t])}, margin {margin / rng:.1e}"
                    break
                hist.append(int(want[b, t]))
        fin = m.finished(batch)
        if np.array_equal(got, want.numpy()):
            assert list(fin) == [bool((want[b] == eos).any()) for b in range(batch)]
    m.set_sampling(0.0, 0, -1)                                    # back to plain argmax: the benchmark's "greedy"
    assert np.array_equal(m.generate(ids, 8), plain[:, :8].numpy()) or dtype == _lib.BF16
    m.close()
