"""The CPU oracle against the committed golden vectors and against its own invariants."""
import glob
import math
import os

import numpy as np
import pytest
import torch

import rai_cpu
import util
from rai_b200 import configs, synth

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_reproduces_golden(path):
    g = np.load(path)
    name = os.path.basename(path)[:-4]
    cfg = configs.get(name)
    model = util.build_oracle(cfg, synth.weights(cfg, int(g["seed"])))
    steps = g["tokens"].shape[1]
    toks, logits = rai_cpu.greedy_generate(model, torch.from_numpy(g["prompt"].astype(np.int64)), steps, True)
    assert np.array_equal(toks.numpy(), g["tokens"])
    assert util.rel_error(logits, torch.from_numpy(g["logits"])) < 1e-5


@pytest.mark.parametrize("name", sorted(configs.TINY))
def test_cached_decode_equals_full_recompute(name):
    """Growing the KV cache one token at a time gives the logits of a from-scratch pass over the
    whole sequence (the property the reference's cat-based cache relies on)."""
    cfg = configs.get(name)
    w = synth.weights(cfg, 99)
    ids = torch.from_numpy(synth.prompt(cfg, 2, 9, 99).astype(np.int64))
    m = util.build_oracle(cfg, w)
    m.forward(ids[:, :6], 0)
    for t in range(6, 9):
        step = m.forward(ids[:, t:t + 1], t).reshape(2, -1)
    full = util.build_oracle(cfg, w).forward(ids, 0).reshape(2, -1)
    assert util.rel_error(step, full) < 2e-5


def test_gqa_equals_mha_with_repeated_kv_weights():
    """A GQA model equals the MHA model whose k/v projections repeat each KV head n_rep times
    (this is what repeat_kv, gemma.rs:191-201, computes)."""
    cfg = configs.get("tiny-qwen2")
    w = synth.weights(cfg, 7)
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], configs.head_dim(cfg)
    rep = nq // nkv
    mha_cfg = dict(cfg, num_key_value_heads=nq)
    w2 = dict(w)
    for i in range(cfg["num_hidden_layers"]):
        for n in ("k_proj", "v_proj"):
            for suffix in ("weight", "bias"):
                key = f"model.layers.{i}.self_attn.{n}.{suffix}"
                x = w[key].reshape(nkv, d, -1)
                w2[key] = np.repeat(x, rep, axis=0).reshape((nq * d,) + w[key].shape[1:])
    ids = torch.from_numpy(synth.prompt(cfg, 2, 7, 3).astype(np.int64))
    a = util.build_oracle(cfg, w).forward(ids, 0)
    b = util.build_oracle(mha_cfg, w2).forward(ids, 0)
    assert util.rel_error(a, b) < 1e-5


def test_module_formulas():
    torch.manual_seed(0)
    x = torch.randn(3, 5, 64)
    w, b = torch.randn(64), torch.randn(64)
    # rms_norm.rs:18-22 is the usual RMSNorm
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert torch.allclose(rai_cpu.rms_norm(x, w, 1e-6), ref, atol=1e-5)
    assert torch.allclose(rai_cpu.gemma_rms_norm(x, w, 1e-6), ref / w * (1 + w), atol=1e-4)
    assert torch.allclose(rai_cpu.layer_norm(x, w, b, 1e-5), torch.nn.functional.layer_norm(x, (64,), w, b, 1e-5), atol=1e-5)
    assert torch.allclose(rai_cpu.silu(x), torch.nn.functional.silu(x), atol=1e-6)
    assert torch.allclose(rai_cpu.new_gelu(x), torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-6)
    assert torch.allclose(rai_cpu.gelu(x), torch.nn.functional.gelu(x), atol=1e-6)
    assert torch.allclose(rai_cpu.softmax_last(x), torch.softmax(x, -1), atol=1e-6)


def test_rope_is_a_rotation_and_position_zero_is_identity():
    sin, cos = rai_cpu.rope_tables(64, 32, 1e6, "qwen2")
    q = torch.randn(1, 2, 5, 64)
    q0, _ = rai_cpu.rope_full(q[:, :, :1], q[:, :, :1], sin, cos, 0)
    assert torch.equal(q0, q[:, :, :1])
    q5, _ = rai_cpu.rope_full(q, q, sin, cos, 3)
    assert torch.allclose(q5.norm(dim=-1), q.norm(dim=-1), atol=1e-4)
    # partial rotary leaves the pass-through lanes untouched (phi2.rs:66-77)
    sin2, cos2 = rai_cpu.rope_tables(32, 32, 1e4, "phi2")
    x = torch.randn(1, 2, 4, 80)
    y = rai_cpu.rope_partial(x, sin2, cos2, 32, 5)
    assert torch.equal(y[..., 32:], x[..., 32:])


def test_sample_argmax_takes_the_last_of_equal_maxima():
    # examples/qwen2/src/main.rs:32-40: Iterator::max_by returns the last maximum
    assert rai_cpu.sample_argmax(torch.tensor([1.0, 5.0, 2.0, 5.0, 0.0])) == 3
    assert rai_cpu.sample_argmax(torch.tensor([-1.0, -1.0])) == 1


def test_repeat_penalty():
    out = rai_cpu.apply_repeat_penalty(torch.tensor([2.0, -2.0, 3.0]), 1.1, [0, 1, 1])
    assert math.isclose(float(out[0]), 2.0 / 1.1, rel_tol=1e-6)
    assert math.isclose(float(out[1]), -2.2, rel_tol=1e-6) and float(out[2]) == 3.0


def test_mask_matches_reference_loops():
    # qwen2.rs:316-327 written as the nested loop it is
    tgt, off, win = 5, 3, 2
    m = rai_cpu.additive_causal_mask(1, tgt, off, win)[0, 0]
    for i in range(tgt):
        for j in range(tgt):
            want = float("-inf") if (i < j or j + win < i) else 0.0
            assert float(m[i, off + j]) == want
    assert torch.all(m[:, :off] == 0)


def test_sampling_rules_of_the_examples():
    """examples/qwen2/src/main.rs:32-53 worked by hand: the penalty divides non-negative logits and multiplies
    negative ones, once per distinct token id; argmax is the last index of the maximum under total_cmp."""
    x = torch.tensor([1.0, -1.0, 2.0, 0.0])
    got = rai_cpu.apply_repeat_penalty(x, 2.0, [0, 1, 1, 3])
    assert got.tolist() == [0.5, -2.0, 2.0, 0.0]
    assert rai_cpu.sample_argmax(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 2
    assert rai_cpu.sample_argmax(torch.tensor([0.0, -0.0, -0.0])) == 0          # +0.0 > -0.0 under the total order
    assert rai_cpu.sample_argmax(torch.tensor([-0.0, 0.0, 0.0])) == 2
    assert rai_cpu.sample_argmax(torch.tensor([float("-inf"), float("-inf")])) == 1
    p = np.float32(1.10)
    y = rai_cpu.apply_repeat_penalty(torch.tensor([3.3, -3.3]), 1.10, [0, 1])
    assert y[0].item() == np.float32(np.float32(3.3) / p) and y[1].item() == np.float32(np.float32(-3.3) * p)


@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-qwen2-tied", "tiny-qwen2-g7", "tiny-phi2", "tiny-phi3", "tiny-gemma"])
def test_c_restatement_agrees_with_the_torch_restatement(name):
    """Two restatements of the reference written independently (plain C loops, torch ops) must produce the same
    logits on prefill and on cached decode steps, and the same greedy tokens."""
    import rai_ref
    cfg = configs.get(name)
    w = synth.weights(cfg, 21)
    ids = synth.prompt(cfg, 2, 19, 22)
    want_tok, want = rai_cpu.greedy_generate(util.build_oracle(cfg, w), torch.from_numpy(ids.astype(np.int64)), 4, True)
    m = rai_ref.RefModel(cfg, w, batch_cap=2)
    cur, pos = ids, 0
    for t in range(4):
        got = torch.from_numpy(m.forward(cur, pos))
        assert util.rel_error(got, want[t]) <= 2e-5, f"{name} step {t}"
        assert got.argmax(-1).tolist() == want_tok[:, t].tolist()
        pos += cur.shape[1]
        cur = want_tok[:, t:t + 1].numpy()
    m.close()
