"""End-to-end parity of the four decoders with the CPU oracle: golden logits, greedy tokens, and the
size-independent properties (cached decode == recompute, batch invariance, API routes agree)."""
import glob
import os

import numpy as np
import pytest
import torch

import rai_cpu
import util
from rai_b200 import _lib, configs, synth
from rai_b200.models import Model

pytestmark = pytest.mark.gpu
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
F32_TOL = 1e-4      # float32 logits: relative
BF16_TOL = 2e-2     # bf16 logits: max-abs relative to the logit range


def build(cuda, cfg, weights, dtype, max_batch=4, max_seq=128, max_tokens=None):
    m = Model(cfg, dtype, cuda, max_batch, max_seq, max_tokens)
    m.update_params(weights)
    return m


def assert_tokens_match(got, want, logits_ref, what):
    """Greedy tokens must be identical; a mismatch is only tolerated at a genuine near-tie of the
    reference (top-1/top-2 margin below the logit tolerance), after which the sequences diverge."""
    got, want = np.asarray(got), np.asarray(want)
    for b in range(want.shape[0]):
        for t in range(want.shape[1]):
            if got[b, t] != want[b, t]:
                margin = float(util.top2_margin(logits_ref[t, b]))
                rng = float(logits_ref[t, b].max() - logits_ref[t, b].min())
                assert margin < BF16_TOL * rng, (f"{what}: sequence {b} step {t}: got {got[b, t]} want {want[b, t]}, "
                                                 f"reference margin {margin:.3g} of range {rng:.3g}")
                break


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_f32_matches_golden(cuda, path):
    g = np.load(path)
    cfg = configs.get(os.path.basename(path)[:-4])
    m = build(cuda, cfg, synth.weights(cfg, int(g["seed"])), _lib.F32)
    toks, logits = m.greedy_generate(g["prompt"], g["tokens"].shape[1], collect_logits=True)
    assert util.rel_error(logits, torch.from_numpy(g["logits"])) <= F32_TOL
    assert np.array_equal(toks.numpy(), g["tokens"])
    m.close()


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_bf16_matches_golden(cuda, path):
    g = np.load(path)
    cfg = configs.get(os.path.basename(path)[:-4])
    m = build(cuda, cfg, synth.weights(cfg, int(g["seed"])), _lib.BF16)
    ref = torch.from_numpy(g["logits"])
    # teacher-forced: feed the reference's tokens so that every step's logits are comparable
    m.clear_kv_cache()
    b = g["prompt"].shape[0]
    ids, pos = g["prompt"], 0
    for t in range(g["tokens"].shape[1]):
        logits = m.forward(ids, pos).reshape(b, -1)
        assert util.logit_error(logits, ref[t]) <= BF16_TOL, f"step {t}"
        pos += ids.shape[1]
        ids = g["tokens"][:, t:t + 1]
    toks = m.greedy_generate(g["prompt"], g["tokens"].shape[1])
    assert_tokens_match(toks.numpy(), g["tokens"], ref, "bf16 greedy")
    m.close()


@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-qwen2-g7", "tiny-phi2", "tiny-phi3", "tiny-gemma"])
def test_first_32_greedy_tokens_identical(cuda, name):
    cfg = configs.get(name)
    w = synth.weights(cfg, 17)
    prompt = synth.prompt(cfg, 2, 20, 17)
    want, ref_logits = rai_cpu.greedy_generate(util.build_oracle(cfg, w), torch.from_numpy(prompt.astype(np.int64)), 32, True)
    m = build(cuda, cfg, w, _lib.BF16)
    got = m.greedy_generate(prompt, 32)
    assert_tokens_match(got.numpy(), want.numpy(), ref_logits, name)
    m32 = build(cuda, cfg, w, _lib.F32)
    assert np.array_equal(m32.greedy_generate(prompt, 32).numpy(), want.numpy())
    m.close(); m32.close()


@pytest.mark.parametrize("dtype", [_lib.F32, _lib.BF16])
@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-phi2", "tiny-gemma"])
def test_cached_decode_equals_recompute_and_chunked_prefill(cuda, dtype, name):
    cfg = configs.get(name)
    m = build(cuda, cfg, synth.weights(cfg, 5), dtype, max_batch=2, max_seq=128)
    ids = synth.prompt(cfg, 2, 70, 5)
    full = m.forward(ids, 0).reshape(2, -1).float().cpu()
    m.clear_kv_cache()
    m.forward(ids[:, :64], 0)
    for t in range(64, 70):
        step = m.forward(ids[:, t:t + 1], t).reshape(2, -1).float().cpu()
    tol = 1e-4 if dtype == _lib.F32 else BF16_TOL
    assert util.logit_error(step, full) <= tol
    if cfg["arch"] != "phi2":  # phi2's mask has no offset form (phi2.rs:104-109)
        m.clear_kv_cache()
        m.forward(ids[:, :37], 0)
        chunk = m.forward(ids[:, 37:], 37).reshape(2, -1).float().cpu()   # prefill with seqlen_offset > 0
        assert util.logit_error(chunk, full) <= tol
    m.close()


def test_batch_rows_are_independent(cuda):
    cfg = configs.get("tiny-qwen2-g7")
    m = build(cuda, cfg, synth.weights(cfg, 8), _lib.BF16, max_batch=4, max_seq=64)
    ids = synth.prompt(cfg, 4, 30, 8)
    all4 = m.forward(ids, 0).reshape(4, -1).float().cpu()
    m.clear_kv_cache()
    one = m.forward(ids[2:3], 0).reshape(1, -1).float().cpu()
    assert util.logit_error(one, all4[2:3]) <= BF16_TOL
    m.close()


def test_generate_step_and_decode_loop_agree_with_forward(cuda):
    cfg = configs.get("tiny-qwen2")
    m = build(cuda, cfg, synth.weights(cfg, 3), _lib.BF16, max_batch=2, max_seq=64)
    prompt = synth.prompt(cfg, 2, 10, 3)
    want = m.greedy_generate(prompt, 6).numpy()
    # host route: pinned tokens in, token ids out
    m.clear_kv_cache()
    tin = torch.from_numpy(prompt.astype(np.int32)).pin_memory()
    tout = torch.empty(2, dtype=torch.int32).pin_memory()
    got, pos = [], 0
    for _ in range(6):
        m.generate_step(tin, pos, tout)
        pos += tin.shape[1]
        got.append(tout.clone())
        tin = tout.clone().reshape(2, 1).pin_memory()
    assert np.array_equal(torch.stack(got, 1).numpy(), want)
    # device loop: first token from the prefill, the rest without leaving the GPU
    m.clear_kv_cache()
    m.generate_step(torch.from_numpy(prompt.astype(np.int32)).pin_memory(), 0, tout)
    rest = m.decode_loop(tout.cuda(), 10, 5)
    cuda.synchronize()
    assert np.array_equal(rest.cpu().numpy().T, want[:, 1:])
    m.close()


def test_forward_rejects_wrong_offset_and_overflow(cuda):
    cfg = configs.get("tiny-qwen2")
    m = build(cuda, cfg, synth.weights(cfg, 3), _lib.BF16, max_batch=2, max_seq=64)
    ids = synth.prompt(cfg, 2, 10, 3)
    with pytest.raises(_lib.RaiB200Error):
        m.forward(ids, 5)                       # cache is empty: offset must be 0
    with pytest.raises(_lib.RaiB200Error):
        m.forward(synth.prompt(cfg, 3, 4, 3), 0)  # batch beyond capacity
    m.forward(ids, 0)
    with pytest.raises(_lib.RaiB200Error):
        m.forward(synth.prompt(cfg, 2, 60, 3), 10)  # cache overflow
    m.close()


def test_missing_and_misshapen_parameters(cuda):
    cfg = configs.get("tiny-phi3")
    w = synth.weights(cfg, 1)
    m = Model(cfg, _lib.BF16, cuda, 1, 64)
    with pytest.raises(_lib.RaiB200Error) as e:
        m.update_param("model.layers.0.self_attn.q_proj.weight", w["model.norm.weight"])
    assert e.value.code == -8
    with pytest.raises(_lib.RaiB200Error) as e:
        m.update_param("model.norm.weight", w["model.embed_tokens.weight"])
    assert e.value.code == -2
    w.pop("model.layers.1.mlp.down_proj.weight")
    with pytest.raises(_lib.RaiB200Error) as e:
        m.update_params(w)
    assert e.value.code == -8 and "down_proj" in str(e.value)
    assert sorted(m.param_names()) == sorted(n for n, _, _ in synth.param_shapes(cfg))
    m.close()


def test_qwen2_half_billion_config_against_oracle(cuda):
    """The first benchmark configuration at full size: Qwen2-0.5B architecture, batch 1, 128-token
    prompt, bf16 on the GPU against the float32 oracle on the same bf16-rounded weights."""
    cfg = configs.get("qwen2-0.5b")
    cfg["max_position_embeddings"] = 512
    w = synth.weights(cfg, 1234)
    prompt = synth.prompt(cfg, 1, 128, 1234)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    want, ref_logits = rai_cpu.greedy_generate(util.build_oracle(cfg, w), torch.from_numpy(prompt.astype(np.int64)), 32, True)
    m = build(cuda, cfg, w, _lib.BF16, max_batch=1, max_seq=256, max_tokens=128)
    m.clear_kv_cache()
    ids, pos = prompt, 0
    for t in range(32):
        logits = m.forward(ids, pos).reshape(1, -1)
        assert util.logit_error(logits, ref_logits[t]) <= BF16_TOL, f"step {t}"
        pos += ids.shape[1]
        ids = want[:, t:t + 1].numpy()
    got = m.greedy_generate(prompt, 32)
    assert_tokens_match(got.numpy(), want.numpy(), ref_logits, "qwen2-0.5b")
    m.close()
