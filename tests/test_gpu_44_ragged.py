"""Batches whose sequences have different lengths (right-padded prompts, then every sequence decoding at its own
position) against the CPU oracle run on each sequence alone: the pads must influence nothing."""
import numpy as np
import pytest
import torch

import rai_cpu
import util
from rai_b200 import _lib, configs, synth
from rai_b200.models import Model

pytestmark = pytest.mark.gpu
LENS = [5, 70, 12, 64]          # one shorter than a cache page, one longer, one exactly a page
STEPS = 10


def _prompts(cfg, seed):
    g = np.random.default_rng(seed)
    return [g.integers(0, cfg["vocab_size"], size=(n,)).astype(np.int32) for n in LENS]


def _tol(dtype, rng):
    return (1e-4 if dtype == _lib.F32 else 2e-2) * rng


@pytest.mark.parametrize("name,dtype", [("tiny-qwen2", _lib.F32), ("tiny-qwen2", _lib.BF16), ("tiny-phi2", _lib.BF16),
                                        ("tiny-phi3", _lib.BF16), ("tiny-gemma", _lib.BF16), ("tiny-qwen2-g7", _lib.BF16)])
def test_ragged_prefill_logits_match_each_sequence_alone(cuda, name, dtype):
    cfg = configs.get(name)
    w = synth.weights(cfg, 31)
    prompts = _prompts(cfg, 32)
    oracle = util.build_oracle(cfg, w)
    m = Model(cfg, dtype, cuda, len(LENS), 128, len(LENS) * max(LENS))
    m.update_params(w)
    ids = np.full((len(LENS), max(LENS)), 7, dtype=np.int32)       # pad token 7: any valid id
    for i, p in enumerate(prompts):
        ids[i, : len(p)] = p
    got = m.forward_ragged(ids, LENS).float().cpu()
    for b, p in enumerate(prompts):
        oracle.clear_kv_cache()
        want = oracle.forward(torch.from_numpy(p.astype(np.int64)).reshape(1, -1), 0).reshape(-1)
        if dtype == _lib.F32:
            assert util.rel_error(got[b], want) <= 1e-4, f"{name} sequence {b}"
        else:
            assert util.logit_error(got[b], want) <= 2e-2, f"{name} sequence {b}"
    # different pad tokens, same logits bit for bit: the pads are really invisible
    ids2 = ids.copy()
    for i, n in enumerate(LENS):
        ids2[i, n:] = 3
    m.clear_kv_cache()
    again = m.forward_ragged(ids2, LENS).float().cpu()
    assert torch.equal(got, again)
    m.close()


@pytest.mark.parametrize("name,dtype", [("tiny-qwen2", _lib.F32), ("tiny-qwen2", _lib.BF16), ("tiny-phi2", _lib.BF16),
                                        ("tiny-qwen2-g7", _lib.BF16)])
@pytest.mark.parametrize("penalty", [0.0, 1.10])
def test_ragged_generation_matches_each_sequence_alone(cuda, name, dtype, penalty):
    """Prompt call + captured decode loop with every sequence at its own length, with and without the examples'
    repeat penalty (whose window must hold the valid tokens only, never the pads)."""
    cfg = configs.get(name)
    w = synth.weights(cfg, 33)
    prompts = _prompts(cfg, 34)
    oracle = util.build_oracle(cfg, w)
    m = Model(cfg, dtype, cuda, len(LENS), 128, len(LENS) * max(LENS))
    m.update_params(w)
    m.set_sampling(penalty, 64, -1)
    got = m.generate_ragged(prompts, STEPS)
    for b, p in enumerate(prompts):
        pt = torch.from_numpy(p.astype(np.int64)).reshape(1, -1)
        want, ref = rai_cpu.generate_with_penalty(oracle, pt, STEPS, penalty, 64, -1, True)
        hist = [int(t) for t in p]
        for t in range(STEPS):
            if got[b, t] != int(want[0, t]):
                row = ref[t, 0]
                if penalty >= 1.0:
                    row = rai_cpu.apply_repeat_penalty(row, penalty, hist[max(0, len(hist) - 64):])
                margin, rng = float(util.top2_margin(row)), float(row.max() - row.min())
                assert margin < _tol(dtype, rng), (f"{name} sequence {b} step {t}: got {got[b, t]} want {int(want[0, t])}, "
                                                   f"margin {margin / rng:.1e} of the range")
                break
            hist.append(int(want[0, t]))
    m.close()


def test_ragged_argument_checks(cuda):
    cfg = configs.get("tiny-qwen2")
    m = Model(cfg, _lib.BF16, cuda, 2, 64, 64)
    m.update_params(synth.weights(cfg, 35))
    ids = np.zeros((2, 8), dtype=np.int32)
    with pytest.raises(_lib.RaiB200Error, match="valid tokens"):
        m.forward_ragged(ids, [0, 8])
    with pytest.raises(_lib.RaiB200Error, match="valid tokens"):
        m.forward_ragged(ids, [9, 8])
    m.close()
