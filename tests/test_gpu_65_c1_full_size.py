"""The reference's own CPU-runnable case at FULL size: the qwen2-0.5b architecture (24 layers, hidden 896,
14 query / 2 KV heads of 64, vocabulary 151936, tied embeddings), batch 1, a 128-token prompt, then greedy
decode steps with the KV cache (examples/qwen2/src/main.rs:60-100).  float32 on the GPU must match the CPU
oracle to 1e-4 relative; bf16 must stay within 2e-2 of the logit range with the greedy tokens identical
(teacher-forced, so one near-tie cannot change every later step)."""
import numpy as np
import pytest
import torch

import rai_cpu
import util
from rai_b200 import _lib, configs, synth
from rai_b200.models import Model

pytestmark = pytest.mark.gpu

PROMPT, STEPS = 128, 32


@pytest.fixture(scope="module")
def c1():
    cfg = configs.get("qwen2-0.5b")
    cfg["max_position_embeddings"] = 512
    w = synth.weights(cfg, 1234)
    ids = synth.prompt(cfg, 1, PROMPT, 1235)
    want, ref = rai_cpu.greedy_generate(util.build_oracle(cfg, w), torch.from_numpy(ids.astype(np.int64)), STEPS, True)
    return cfg, w, ids, want, ref


def _teacher_forced(m, ids, want):
    cur, pos = ids, 0
    for t in range(STEPS):
        yield t, m.forward(cur, pos).reshape(1, -1)
        pos += cur.shape[1]
        cur = want[:, t:t + 1].numpy()


def test_c1_float32_logits_and_tokens(cuda, c1):
    cfg, w, ids, want, ref = c1
    m = Model(cfg, _lib.F32, cuda, 1, 256, PROMPT)
    m.update_params(w)
    for t, logits in _teacher_forced(m, ids, want):
        err = util.rel_error(logits, ref[t])
        assert err <= 1e-4, f"step {t}: float32 logits differ by {err:.2e} relative"
        got = int(logits.float().cpu().argmax(-1)[0])
        if got != int(want[0, t]):
            margin = float(util.top2_margin(ref[t, 0])) / float(ref[t, 0].abs().max())
            assert margin < 1e-4, f"step {t}: token differs at relative margin {margin:.1e}"
    m.close()


def test_c1_bf16_logits_and_first_32_tokens(cuda, c1):
    cfg, w, ids, want, ref = c1
    m = Model(cfg, _lib.BF16, cuda, 1, 256, PROMPT)
    m.update_params(w)
    for t, logits in _teacher_forced(m, ids, want):
        err = util.logit_error(logits, ref[t])
        assert err <= 2e-2, f"step {t}: bf16 logits error {err:.2e} of the logit range"
        got = int(logits.float().cpu().argmax(-1)[0])
        if got != int(want[0, t]):   # only excusable at a genuine near-tie of the reference
            rng = float(ref[t, 0].max() - ref[t, 0].min())
            margin = float(util.top2_margin(ref[t, 0]))
            assert margin < 2e-2 * rng, f"step {t}: token differs at margin {margin / rng:.1e} of the range"
    m.close()


def test_c1_bf16_free_running_generation_matches_until_a_near_tie(cuda, c1):
    """The library's own decode loop (on-device argmax, CUDA-graph steps), not teacher-forced: its tokens
    must equal the oracle's up to the first step whose reference top-2 margin is inside the bf16 tolerance."""
    cfg, w, ids, want, ref = c1
    m = Model(cfg, _lib.BF16, cuda, 1, 256, PROMPT)
    m.update_params(w)
    tok_in = torch.from_numpy(ids.astype(np.int32)).pin_memory()
    first = torch.empty((1,), dtype=torch.int32).pin_memory()
    m.generate_step(tok_in, 0, first)                     # prefill + on-device argmax
    rest = m.decode_loop(first.to(f"cuda:{cuda.id}"), PROMPT, STEPS - 1)
    cuda.synchronize()
    got = np.concatenate([first.numpy().reshape(1, 1), rest.cpu().numpy().reshape(STEPS - 1, 1).T], axis=1)
    for t in range(STEPS):
        if int(got[0, t]) == int(want[0, t]):
            continue
        rng = float(ref[t, 0].max() - ref[t, 0].min())
        margin = float(util.top2_margin(ref[t, 0]))
        assert margin < 2e-2 * rng, f"step {t}: free-running token differs at margin {margin / rng:.1e} of the range"
        break
    m.close()
