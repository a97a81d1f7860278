"""The benchmark configurations at their full widths (hidden size, heads, head size, intermediate size,
vocabulary) with the depth cut to two layers, so that the float32 CPU oracle finishes in seconds: bf16 on
the GPU against the oracle on the same bf16-rounded weights, prefill and teacher-forced decode steps.

Sizes: short prompts at small batches first; then each configuration at its OWN batch and context - phi2 8 x 512 and
phi3-mini 4 x 2048 by really prefilling, gemma-2b 32 x 1024 and qwen2-7b 64 x 2048 (the shape the benchmark times)
from an injected cache, because a float32 CPU prefill of 131 072 tokens at 7B width takes minutes
(oracle/parity_kit.py)."""
import numpy as np
import pytest
import torch

import rai_cpu
import util
from rai_b200 import _lib, configs, synth
from rai_b200.models import Model

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,batch,prompt", [("phi2", 3, 70), ("phi3-mini", 2, 130), ("gemma-2b", 4, 65), ("qwen2-7b", 2, 100),
                                               ("phi2", 8, 512), ("phi3-mini", 4, 2048)])
def test_full_width_two_layer_model_matches_oracle(cuda, name, batch, prompt):
    cfg = configs.get(name)
    cfg["num_hidden_layers"] = 2
    cfg["max_position_embeddings"] = max(512, prompt + 16)
    torch.set_num_threads(max(1, (torch.get_num_threads())))
    w = synth.weights(cfg, 77)
    ids = synth.prompt(cfg, batch, prompt, 77)
    steps = 4
    want, ref = rai_cpu.greedy_generate(util.build_oracle(cfg, w), torch.from_numpy(ids.astype(np.int64)), steps, True)
    m = Model(cfg, _lib.BF16, cuda, batch, max(256, prompt + 16), batch * prompt)
    m.update_params(w)
    del w
    cur, pos = ids, 0
    for t in range(steps):
        logits = m.forward(cur, pos).reshape(batch, -1)
        err = util.logit_error(logits, ref[t])
        assert err <= 2e-2, f"{name} step {t}: logits error {err:.2e} of the logit range"
        got = logits.float().cpu().argmax(-1)
        for b in range(batch):
            if int(got[b]) != int(want[b, t]):   # only excusable at a genuine near-tie of the reference
                margin = float(util.top2_margin(ref[t, b]))
                rng = float(ref[t, b].max() - ref[t, b].min())
                assert margin < 2e-2 * rng, f"{name} step {t} seq {b}: token differs at margin {margin / rng:.1e}"
        pos += cur.shape[1]
        cur = want[:, t:t + 1].numpy()
    m.close()


@pytest.mark.parametrize("name,batch,ctx", [("gemma-2b", 32, 1024), ("qwen2-7b", 64, 2048)])
def test_decode_at_the_configurations_own_batch_and_context(cuda, name, batch, ctx):
    """Four decode steps of the two-layer full-width model at the benchmark's batch and context (for qwen2-7b: batch
    64 over a 2048-token cache, the captured single-token step with its 33-tile attention walk), from an injected
    cache, against the oracle."""
    import parity_kit
    cfg = configs.get(name)
    cfg["num_hidden_layers"] = 2
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], ctx + 16)
    params = parity_kit.rounded_params(cfg, 60)
    m = Model(cfg, _lib.BF16, cuda, batch, ctx + 16, batch)
    for k, v in params.items():
        m.update_param(k, v)
    m.finalize()
    r = parity_kit.decode_parity(cfg, params, m, batch, ctx, 4, 61)
    m.close()
    print(f"{name} batch {batch} context {ctx}: {r}")
    assert r["max_logit_err_of_range"] <= 2e-2, r
    assert r["of_which_not_near_ties"] == 0, r
