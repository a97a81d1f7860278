"""The benchmark configurations at their full widths (hidden size, heads, head size, intermediate size,
vocabulary) with the depth cut to two layers, so that the float32 CPU oracle finishes in seconds: bf16 on
the GPU against the oracle on the same bf16-rounded weights, prefill and teacher-forced decode steps."""
import numpy as np
import pytest
import torch

import rai_cpu
import util
from rai_b200 import _lib, configs, synth
from rai_b200.models import Model

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,batch,prompt", [("phi2", 3, 70), ("phi3-mini", 2, 130), ("gemma-2b", 4, 65), ("qwen2-7b", 2, 100)])
def test_full_width_two_layer_model_matches_oracle(cuda, name, batch, prompt):
    cfg = configs.get(name)
    cfg["num_hidden_layers"] = 2
    cfg["max_position_embeddings"] = 512
    torch.set_num_threads(max(1, (torch.get_num_threads())))
    w = synth.weights(cfg, 77)
    ids = synth.prompt(cfg, batch, prompt, 77)
    steps = 4
    want, ref = rai_cpu.greedy_generate(util.build_oracle(cfg, w), torch.from_numpy(ids.astype(np.int64)), steps, True)
    m = Model(cfg, _lib.BF16, cuda, batch, 256, batch * prompt)
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
