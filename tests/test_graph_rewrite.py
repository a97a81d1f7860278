"""The pre-eval rewrite pass of the lazy graph (rai_b200/graph.py: optimize) is host logic: it can be checked without
a GPU by building graphs over leaves that carry no data.  The module code of the rai-nn mirror (RmsNorm, Linear, silu)
written on such leaves must come out of `optimize` as the three fused nodes, shared constants must be shared, the
input graph must be left as it was, and near-misses of the patterns must be left alone.  (What the fused nodes compute
is checked on the GPU by test_gpu_46_graph_fusion.py.)"""
from rai_b200 import _lib, nn
from rai_b200.graph import LazyTensor, Node, optimize, topological


def leaf(shape, dtype=_lib.BF16):
    return LazyTensor(Node("Const", (), [], shape, dtype, None))


def ops(outputs):
    return [n.op for n in topological(outputs)]


def mlp_block(x, w):
    """post-attention half of a qwen2 decoder layer (qwen2.rs:100-104,264-265)."""
    n = nn.RmsNorm(w["ln"], 1e-6).fwd(x)
    gate, up, down = nn.Linear(w["gate"]), nn.Linear(w["up"]), nn.Linear(w["down"], w["down_b"])
    return x + down.fwd(gate.fwd(n).silu() * up.fwd(n))


def weights(H=64, I=128):
    return {"ln": leaf([H]), "gate": leaf([I, H]), "up": leaf([I, H]), "down": leaf([H, I]), "down_b": leaf([H])}


def test_the_three_patterns_are_found_and_the_input_graph_is_untouched():
    x, w = leaf([2, 5, 64]), weights()
    out = mlp_block(x, w)
    before = ops([out])
    fused = optimize([out])
    assert ops([out]) == before, "optimize must not modify the graph it was given"
    after = ops(fused)
    assert optimize.last_stats["rms_norm"] == 1 and optimize.last_stats["gated_linear"] == 1 and optimize.last_stats["linear"] == 1
    for name in ("FusedRmsNorm", "FusedGatedLinear", "FusedLinear"):
        assert after.count(name) == 1, (name, after)
    for gone in ("MatMul", "Rsqrt", "Exp", "Transpose", "Broadcast"):
        assert gone not in after, f"{gone} should have been absorbed: {after}"
    assert len(after) < len(before)
    assert fused[0].shape == out.shape and fused[0].dtype == out.dtype
    # the down projection keeps its bias as a third input, the gated node takes (x, W_gate, W_up)
    by_op = {n.op: n for n in topological(fused)}
    assert len(by_op["FusedLinear"].inputs) == 3 and len(by_op["FusedGatedLinear"].inputs) == 3
    assert by_op["FusedGatedLinear"].inputs[0] is by_op["FusedRmsNorm"]


def test_equal_constants_are_shared():
    x = leaf([4, 8], _lib.F32)
    a = x.relu() + x.relu()                     # two Full(0.0) leaves of the same shape and dtype
    n_full = ops([a]).count("Full")
    assert n_full == 2
    b = optimize([a])
    assert ops(b).count("Full") == 1 and optimize.last_stats["constants_shared"] == 1


def test_near_misses_are_left_alone():
    H = 64
    x, other, w = leaf([3, H]), leaf([3, H]), leaf([H])
    # the statistics come from a different tensor than the one that is scaled: not an RmsNorm
    r = ((other * (1.0 / H ** 0.5)).square().sum(-1, True) + 1e-6).rsqrt()
    y = (w * x) * r
    assert "FusedRmsNorm" not in ops(optimize([y]))
    # a matmul with an untransposed weight is not a Linear
    z = x.matmul(leaf([H, 16]))
    assert "FusedLinear" not in ops(optimize([z])) and "MatMul" in ops(optimize([z]))
    # silu(gate(x)) * up(x2) with different inputs must stay two Linears and a product
    x2 = leaf([3, H])
    g, u = nn.Linear(leaf([32, H])), nn.Linear(leaf([32, H]))
    t = optimize([g.fwd(x).silu() * u.fwd(x2)])
    assert ops(t).count("FusedLinear") == 2 and "FusedGatedLinear" not in ops(t)
