"""The Tensor / nn mirror of rai-core and rai-nn on `Cuda`: an UNFUSED qwen2 decoder layer written with
Tensor methods exactly as rai-models/src/llm/qwen2.rs does, evaluated through the primitive rules, against
the CPU oracle and against the fused decoder driver."""
import math

import numpy as np
import pytest
import torch

import rai_cpu
import util
from rai_b200 import _lib, configs, nn, synth
from rai_b200.models import Model
from rai_b200.tensor import Tensor, eval_rule, register

pytestmark = pytest.mark.gpu


def T(arr, cuda, dtype=_lib.F32):
    return Tensor.from_array(arr, arr.shape, cuda, dtype)


def rotate_half(x):  # qwen2.rs:33-38
    last = x.size(-1)
    return Tensor.cat([x.narrow(-1, last // 2, last - last // 2).neg(), x.narrow(-1, 0, last // 2)], -1)


def unfused_qwen2_forward(cfg, w, ids, cuda):
    """Model::fwd of qwen2.rs:338-359 with the GQA form of gemma.rs:191-201, from primitives only."""
    H, nq, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d, eps = H // nq, cfg["rms_norm_eps"]
    b, s = ids.shape
    P = {k: T(v, cuda) for k, v in w.items()}
    sin, cos = rai_cpu.rope_tables(d, cfg["max_position_embeddings"], cfg["rope_theta"], "qwen2")
    cos_t, sin_t = T(cos.numpy()[:s], cuda).unsqueeze(0).unsqueeze(0), T(sin.numpy()[:s], cuda).unsqueeze(0).unsqueeze(0)
    mask = T(rai_cpu.additive_causal_mask(b, s, 0).contiguous().numpy(), cuda)
    lin = lambda n, x: nn.Linear(P[n + ".weight"], P.get(n + ".bias")).fwd(x)  # noqa: E731
    xs = nn.Embedding(P["model.embed_tokens.weight"]).fwd(Tensor.from_array(ids, ids.shape, cuda, _lib.U32))
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = nn.RmsNorm(P[p + "input_layernorm.weight"], eps).fwd(xs)
        q = lin(p + "self_attn.q_proj", h).reshape([b, s, nq, d]).transpose(1, 2)
        k = lin(p + "self_attn.k_proj", h).reshape([b, s, nkv, d]).transpose(1, 2)
        v = lin(p + "self_attn.v_proj", h).reshape([b, s, nkv, d]).transpose(1, 2)
        q = q * cos_t + rotate_half(q) * sin_t
        k = k * cos_t + rotate_half(k) * sin_t
        rep = nq // nkv
        k = k.unsqueeze(2).broadcast_to([b, nkv, rep, s, d]).reshape([b, nq, s, d])
        v = v.unsqueeze(2).broadcast_to([b, nkv, rep, s, d]).reshape([b, nq, s, d])
        a = (q.matmul(k.transpose(2, 3)) * (1.0 / math.sqrt(d)) + mask).softmax(-1).matmul(v)
        a = a.transpose(1, 2).reshape([b, s, H])
        xs = lin(p + "self_attn.o_proj", a) + xs
        h = nn.RmsNorm(P[p + "post_attention_layernorm.weight"], eps).fwd(xs)
        g = nn.Activation(cfg["hidden_act"]).fwd(lin(p + "mlp.gate_proj", h)) * lin(p + "mlp.up_proj", h)
        xs = xs + lin(p + "mlp.down_proj", g)
    xs = nn.RmsNorm(P["model.norm.weight"], eps).fwd(xs.narrow(1, s - 1, 1))
    return lin("lm_head", xs)


def test_unfused_graph_matches_oracle_and_fused_driver(cuda):
    cfg = configs.get("tiny-qwen2")
    w = synth.weights(cfg, 41)
    ids = synth.prompt(cfg, 2, 10, 41)
    want = util.build_oracle(cfg, w).forward(torch.from_numpy(ids.astype(np.int64)), 0)
    got = unfused_qwen2_forward(cfg, w, ids, cuda).as_vec()
    assert util.rel_error(torch.from_numpy(got), want) <= 1e-4
    m = Model(cfg, _lib.F32, cuda, 2, 64)
    m.update_params(w)
    fused = m.forward(ids, 0).float().cpu()
    assert util.rel_error(fused, torch.from_numpy(got)) <= 1e-4
    m.close()


def test_tensor_views_and_shape_algebra(cuda):
    x = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 4)
    t = T(x, cuda)
    assert np.array_equal(t.transpose(0, 2).as_vec(), x.transpose(2, 1, 0))
    assert np.array_equal(t.permute([2, 0, 1]).as_vec(), x.transpose(2, 0, 1))          # ops/permute.rs
    assert np.array_equal(t.permute([-1, 0, 1]).narrow(0, 1, 2).as_vec(), x.transpose(2, 0, 1)[1:3])
    with pytest.raises(_lib.RaiB200Error):
        t.permute([0, 0, 1])
    assert np.array_equal(t.narrow(-1, 1, 2).as_vec(), x[..., 1:3])
    assert np.array_equal(t.narrow(1, 2, 1).squeeze(1).as_vec(), x[:, 2])
    assert np.array_equal(t.unsqueeze(0).broadcast_to([5, 2, 3, 4]).as_vec(), np.broadcast_to(x, (5, 2, 3, 4)))
    assert np.array_equal(t.reshape([6, 4]).t().as_vec(), x.reshape(6, 4).T)
    assert np.array_equal(t.flatten(1).as_vec(), x.reshape(2, 12))
    assert np.array_equal(Tensor.cat([t, t.narrow(1, 0, 1)], 1).as_vec(), np.concatenate([x, x[:, :1]], 1))
    assert np.allclose(t.sum(1).as_vec(), x.sum(1)) and np.allclose(t.max(0, True).as_vec(), x.max(0, keepdims=True))
    assert np.allclose(t.softmax(1).as_vec(), torch.softmax(torch.from_numpy(x), 1).numpy(), atol=1e-6)
    assert np.allclose(t.mean(-1).as_vec(), x.mean(-1)) and np.allclose(t.var(-1).as_vec(), x.var(-1), rtol=1e-5)
    assert np.array_equal(t.argmax(-1).as_vec(), x.argmax(-1))
    # dims resolve like rai-core/tests/shape.rs: negative indices count from the end, out of range is an error
    assert t.size(-1) == 4 and t.size(-3) == 2
    with pytest.raises(_lib.RaiB200Error):
        t.size(3)
    with pytest.raises(_lib.RaiB200Error):
        t.reshape([5, 5])          # OpError::IncompatibleShape
    with pytest.raises(_lib.RaiB200Error):
        t.broadcast_to([2, 3, 5])


def test_scalar_ops_activations_where_gather(cuda):
    g = np.random.default_rng(0)
    x = g.standard_normal((4, 33)).astype(np.float32)
    t, xt = T(x, cuda), torch.from_numpy(x)
    assert np.allclose(((t * 2.0 + 1.0) / 4.0 - 0.5).as_vec(), (x * 2 + 1) / 4 - 0.5, atol=1e-6)
    assert np.allclose(t.silu().as_vec(), rai_cpu.silu(xt).numpy(), atol=1e-6)
    assert np.allclose(t.new_gelu().as_vec(), rai_cpu.new_gelu(xt).numpy(), atol=1e-6)
    assert np.allclose(t.gelu().as_vec(), rai_cpu.gelu(xt).numpy(), atol=1e-6)
    assert np.allclose(t.relu().as_vec(), np.maximum(x, 0))
    cond = (x > 0).astype(np.uint8)
    c = Tensor.from_array(cond, cond.shape, cuda, _lib.U8)
    assert np.array_equal(c.where_cond(t, t.neg()).as_vec(), np.abs(x))   # phi2.rs:111-117 style masking
    idx = g.integers(0, 33, (4, 5))
    gi = Tensor.from_array(idx, idx.shape, cuda, _lib.U32)
    assert np.array_equal(t.gather(-1, gi).as_vec(), np.take_along_axis(x, idx, -1))
    bf = t.to_dtype(_lib.BF16)
    assert np.array_equal(bf.to_dtype(_lib.F32).as_vec(), xt.to(torch.bfloat16).float().numpy())
    assert np.array_equal(Tensor.arange(2, 9, cuda).as_vec(), np.arange(2, 9))


def test_dispatch_registry_reports_missing_rules_and_can_be_overridden(cuda):
    with pytest.raises(_lib.RaiB200Error) as e:
        eval_rule(cuda, "Random")          # Error::Unimplemented{op, device} (eval.rs:40-43)
    assert e.value.code == -7
    calls = []
    old = eval_rule(cuda, "Negative")
    register(type(cuda), "Negative", lambda x, s: (calls.append(1), old(x, s))[1])   # dispatch::register overwrites
    try:
        T(np.ones((2, 2), np.float32), cuda).neg()
        assert calls == [1]
    finally:
        register(type(cuda), "Negative", old)
