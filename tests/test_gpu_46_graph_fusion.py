"""The lazy graph and its pre-eval rewrite pass (rai_b200/graph.py): a qwen2-style block written with the rai-nn mirror
on lazy tensors evaluates to the same values as the eager mirror, and after `optimize` the RmsNorm, Linear and
silu(gate) * up sub-graphs run as single fused entry points (fewer nodes, fewer launches, same values)."""
import numpy as np
import pytest
import torch

from rai_b200 import _lib, nn
from rai_b200.graph import LazyTensor, evaluate, optimize, topological
from rai_b200.tensor import Tensor

pytestmark = pytest.mark.gpu


def T(a, cuda, dtype=_lib.F32):
    a = np.asarray(a, dtype=np.float32)
    return Tensor.from_array(a, a.shape, cuda, dtype)


def block(x, w, make_linear):
    """post-attention half of a qwen2 decoder layer: h = x + down(silu(gate(n)) * up(n)), n = rms_norm(x)  (qwen2.rs:100-104,264-265)."""
    n = nn.RmsNorm(w["ln"], 1e-6).fwd(x)
    gate, up, down = make_linear(w["gate"]), make_linear(w["up"]), make_linear(w["down"], w["down_b"])
    return x + down.fwd(gate.fwd(n).silu() * up.fwd(n))


@pytest.mark.parametrize("dtype,tol", [(_lib.F32, 2e-5), (_lib.BF16, 3e-2)])
def test_fused_graph_matches_eager_and_launches_less(cuda, dtype, tol):
    g = np.random.default_rng(3)
    B, S, H, I = 2, 5, 128, 256
    host = {"x": g.standard_normal((B, S, H)), "ln": 1.0 + 0.1 * g.standard_normal(H), "gate": 0.05 * g.standard_normal((I, H)),
            "up": 0.05 * g.standard_normal((I, H)), "down": 0.05 * g.standard_normal((H, I)), "down_b": 0.1 * g.standard_normal(H)}
    dev = {k: T(v, cuda, dtype) for k, v in host.items()}
    # eager mirror: every primitive runs as it is met
    eager = block(dev["x"], dev, lambda w_, b_=None: nn.Linear(w_, b_)).as_vec()
    # the same module code on lazy tensors builds a graph
    lz = {k: LazyTensor.constant(v) for k, v in dev.items()}
    out = block(lz["x"], lz, lambda w_, b_=None: nn.Linear(w_, b_))
    n_plain = len([n for n in topological([out]) if n.op != "Const"])
    l0 = cuda.launch_count()
    plain = evaluate([out])[0].as_vec()
    plain_launches = cuda.launch_count() - l0
    np.testing.assert_allclose(plain, eager, rtol=tol, atol=tol)
    # rewritten graph
    out2 = block(lz["x"], lz, lambda w_, b_=None: nn.Linear(w_, b_))
    fused_out = optimize([out2])[0]
    stats = dict(optimize.last_stats)
    assert stats["rms_norm"] == 1 and stats["gated_linear"] == 1 and stats["linear"] == 1, stats
    n_fused = len([n for n in topological([fused_out]) if n.op != "Const"])
    l0 = cuda.launch_count()
    fused = evaluate([fused_out])[0].as_vec()
    fused_launches = cuda.launch_count() - l0
    scale = max(1.0, float(np.abs(eager).max()))
    assert float(np.abs(fused - eager).max()) <= tol * scale
    assert n_fused <= 4 and n_fused < n_plain // 4, (n_fused, n_plain)
    assert fused_launches < plain_launches, (fused_launches, plain_launches)
    print(f"nodes {n_plain} -> {n_fused}, launches {plain_launches} -> {fused_launches}")


def test_constants_are_shared_like_the_reference_optimize(cuda):
    """x * 2.0-as-a-tensor twice: the two Full nodes collapse into one (rai-core/src/transforms/optimize.rs:41-87)."""
    x = LazyTensor.constant(T(np.arange(6).reshape(2, 3), cuda))
    two_a, two_b = LazyTensor.full(2.0, [2, 3], _lib.F32, cuda), LazyTensor.full(2.0, [2, 3], _lib.F32, cuda)
    y = (x * two_a) * two_b + LazyTensor.full(1.0, [2, 3], _lib.F32, cuda)
    opt = optimize([y])[0]
    assert optimize.last_stats["constants_shared"] == 1
    fulls = [n for n in topological([opt]) if n.op == "Full"]
    assert len(fulls) == 2
    np.testing.assert_allclose(evaluate([opt])[0].as_vec(), np.arange(6).reshape(2, 3) * 4.0 + 1.0)


def test_patterns_that_do_not_match_are_left_alone(cuda):
    x = LazyTensor.constant(T(np.ones((3, 8)), cuda))
    w = LazyTensor.constant(T(np.ones((4, 8)), cuda))
    y = x.matmul(w.t()).exp()            # a Linear, then something else
    z = (x * 0.5).square().sum(-1, True)  # the inside of an RmsNorm without the rest
    outs = optimize([y, z])
    assert optimize.last_stats["linear"] == 1 and optimize.last_stats["rms_norm"] == 0
    a, b = evaluate(outs)
    np.testing.assert_allclose(a.as_vec(), np.exp(np.full((3, 4), 8.0)), rtol=1e-5)
    np.testing.assert_allclose(b.as_vec(), np.full((3, 1), 2.0), rtol=1e-6)
