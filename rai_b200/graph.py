"""A lazy graph over the `Cuda` rules, with a rewrite pass that runs BEFORE evaluation.

rai builds a graph of `Tensor` nodes — device, dtype, shape, op, inputs (rai-core/src/tensor.rs:28-60) — and `eval`
walks it in topological order, looking one rule up per node (rai-core/src/eval.rs:31-51, dispatch.rs:207-212).  Its
only graph rewrite is constant sharing (rai-core/src/transforms/optimize.rs:41-87).  This module is the same thing on
the host side of this library, plus the rewrite that matters on a GPU: sub-graphs that rai-nn composes from a dozen
primitives are recognised and replaced by ONE fused entry point of the C ABI,

    RmsNorm::fwd  (rai-nn/src/rms_norm.rs:18-22, 9 nodes here)        ->  rb_norm
    Linear::fwd   (rai-nn/src/linear.rs:59-69: broadcast, t, matmul, add)  ->  rb_linear
    silu(gate(x)) * up(x)  (rai-models/src/llm/qwen2.rs:100-103)      ->  rb_gated_linear

`LazyTensor` quacks like `rai_b200.tensor.Tensor` for the methods the rai-nn mirror (rai_b200/nn.py) uses, so the same
module code builds either eager results or a graph.  `evaluate` is eval.rs's loop; `optimize` returns rewritten outputs.
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _lib
from .tensor import Tensor, eval_rule


class Node:
    """One graph node: the op's registry name, its non-tensor parameters, its inputs, and (once evaluated) its data."""
    __slots__ = ("op", "params", "inputs", "shape", "dtype", "device", "data")

    def __init__(self, op: str, params: tuple, inputs: List["Node"], shape: Sequence[int], dtype: int, device,
                 data: Optional[Tensor] = None):
        self.op, self.params, self.inputs = op, params, inputs
        self.shape, self.dtype, self.device, self.data = list(shape), dtype, device, data


def _rdim(dim: int, rank: int) -> int:
    return dim + rank if dim < 0 else dim


class LazyTensor:
    """Builds nodes; nothing runs until `evaluate`."""

    def __init__(self, node: Node):
        self.node = node

    # ---- leaves
    @staticmethod
    def constant(t: Tensor) -> "LazyTensor":
        return LazyTensor(Node("Const", (), [], t.shape, t.dtype, t.device, t))

    @staticmethod
    def full(value: float, shape, dtype: int, device) -> "LazyTensor":
        return LazyTensor(Node("Full", (float(value),), [], shape, dtype, device))

    # ---- what modules ask of a tensor
    @property
    def shape(self): return self.node.shape
    @property
    def dtype(self): return self.node.dtype
    @property
    def device(self): return self.node.device
    def size(self, dim: int) -> int: return self.node.shape[_rdim(dim, len(self.node.shape))]

    def _new(self, op, params, inputs, shape, dtype=None) -> "LazyTensor":
        return LazyTensor(Node(op, tuple(params), [i.node for i in inputs], shape, self.dtype if dtype is None else dtype, self.device))

    def _un(self, op: str, scalar: float = 0.0) -> "LazyTensor":
        return self._new(op, (float(scalar),), [self], self.shape)

    def _bin(self, op: str, other) -> "LazyTensor":
        if not isinstance(other, LazyTensor):
            table = {"Add": ("AddScalar", float(other)), "Sub": ("AddScalar", -float(other)), "Mul": ("MulScalar", float(other)),
                     "Div": ("MulScalar", 1.0 / float(other)) if op == "Div" and other != 0 else None}
            if table.get(op):
                return self._un(*table[op])
            other = LazyTensor.full(float(other), [], self.dtype, self.device)
        shape = list(np.broadcast_shapes(tuple(self.shape), tuple(other.shape)))
        return self._new(op, (), [self, other], shape)

    def __add__(self, o): return self._bin("Add", o)
    def __radd__(self, o): return self._bin("Add", o)
    def __sub__(self, o): return self._bin("Sub", o)
    def __mul__(self, o): return self._bin("Mul", o)
    def __rmul__(self, o): return self._bin("Mul", o)
    def __truediv__(self, o): return self._bin("Div", o)
    def maximum(self, o): return self._bin("Maximum", o)
    def neg(self): return self._un("Negative")
    def exp(self): return self._un("Exp")
    def sqrt(self): return self._un("Sqrt")
    def rsqrt(self): return self._un("Rsqrt")
    def square(self): return self._un("Square")
    def tanh(self): return self._un("Tanh")
    def erf(self): return self._un("Erf")
    def powf(self, e: float): return self._un("Powf", e)
    def silu(self): return self / (self.neg().exp() + 1.0)          # hlops/activations.rs:20-23, as Tensor.silu
    def relu(self): return self.maximum(LazyTensor.full(0.0, [], self.dtype, self.device))

    def _reduce(self, op, dim, keep_dim):
        d = _rdim(dim, len(self.shape))
        shape = [1 if i == d else n for i, n in enumerate(self.shape)] if keep_dim else [n for i, n in enumerate(self.shape) if i != d]
        return self._new(op, (d, bool(keep_dim)), [self], shape)

    def sum(self, dim: int = -1, keep_dim: bool = False): return self._reduce("ReduceSum", dim, keep_dim)
    def max(self, dim: int = -1, keep_dim: bool = False): return self._reduce("ReduceMax", dim, keep_dim)
    def mean(self, dim: int = -1, keep_dim: bool = False): return self.sum(dim, keep_dim) / float(self.size(dim))

    def var(self, dim: int = -1, keep_dim: bool = False):
        m = self.mean(dim, True)
        return (self - m).square().sum(dim, keep_dim) / float(self.size(dim))

    def softmax(self, dim: int = -1): return self._new("Softmax", (_rdim(dim, len(self.shape)),), [self], self.shape)

    def matmul(self, other: "LazyTensor"):
        batch = list(np.broadcast_shapes(tuple(self.shape[:-2]), tuple(other.shape[:-2])))
        return self._new("MatMul", (), [self, other], batch + [self.shape[-2], other.shape[-1]])

    def transpose(self, d0: int, d1: int):
        r = len(self.shape)
        a, b = _rdim(d0, r), _rdim(d1, r)
        shape = list(self.shape)
        shape[a], shape[b] = shape[b], shape[a]
        return self._new("Transpose", (a, b), [self], shape)

    def t(self): return self.transpose(-1, -2)
    def broadcast_to(self, shape): return self._new("Broadcast", (tuple(shape),), [self], list(shape))

    def reshape(self, shape):
        shape = list(shape)
        if -1 in shape:
            known = int(np.prod([s for s in shape if s != -1])) or 1
            shape[shape.index(-1)] = int(np.prod(self.shape)) // known
        return self._new("Reshape", (tuple(shape),), [self], shape)

    def flatten(self, start: int = 0): return self.reshape(list(self.shape[:start]) + [-1])
    def unsqueeze(self, dim: int):
        d = _rdim(dim, len(self.shape) + 1)
        return self.reshape(self.shape[:d] + [1] + self.shape[d:])

    def narrow(self, dim: int, start: int, length: int):
        d = _rdim(dim, len(self.shape))
        shape = list(self.shape)
        shape[d] = length
        return self._new("Narrow", (d, start, length), [self], shape)

    def index_select(self, dim: int, index: "LazyTensor"):
        d = _rdim(dim, len(self.shape))
        return self._new("IndexSelect", (d,), [self, index], self.shape[:d] + [int(np.prod(index.shape))] + self.shape[d + 1:])

    def to_dtype(self, dtype: int): return self if dtype == self.dtype else self._new("ToDType", (dtype,), [self], self.shape, dtype)


# --------------------------------------------------------------------------------------------------
# eval (rai-core/src/eval.rs:31-51): topological order, one rule per node
# --------------------------------------------------------------------------------------------------
def topological(outputs: Sequence[LazyTensor]) -> List[Node]:
    order, seen = [], set()

    def visit(n: Node):
        if id(n) in seen:
            return
        seen.add(id(n))
        for i in n.inputs:
            visit(i)
        order.append(n)
    for o in outputs:
        visit(o.node)
    return order


def _run(n: Node) -> Tensor:
    x = [i.data for i in n.inputs]
    op, p = n.op, n.params
    if op == "Full":
        return Tensor.full(p[0], n.shape, n.dtype, n.device)
    if op in ("Add", "Sub", "Mul", "Div", "Maximum", "Minimum"):
        return eval_rule(n.device, op)(x[0], x[1])
    if op in ("ReduceSum", "ReduceMax", "ReduceMin"):
        return eval_rule(n.device, op)(x[0], p[0], p[1])
    if op == "Softmax":
        return eval_rule(n.device, op)(x[0], p[0])
    if op == "MatMul":
        return eval_rule(n.device, op)(x[0], x[1])
    if op == "Transpose":
        return x[0].transpose(p[0], p[1])
    if op == "Broadcast":
        return x[0].broadcast_to(list(p[0]))
    if op == "Reshape":
        return x[0].reshape(list(p[0]))
    if op == "Narrow":
        return x[0].narrow(*p)
    if op == "IndexSelect":
        return eval_rule(n.device, op)(x[0], p[0], x[1])
    if op == "ToDType":
        return eval_rule(n.device, op)(x[0], p[0])
    if op in _FUSED:
        return _FUSED[op](n, x)
    return eval_rule(n.device, op)(x[0], p[0])        # the unary family: (tensor, scalar)


def evaluate(outputs: Sequence[LazyTensor]) -> List[Tensor]:
    """Evaluates every node the outputs depend on, inputs first, and returns the outputs' data."""
    for n in topological(outputs):
        if n.data is None:
            n.data = _run(n)
    return [o.node.data for o in outputs]


# --------------------------------------------------------------------------------------------------
# fused nodes: one C-ABI call each
# --------------------------------------------------------------------------------------------------
def _rows(t: Tensor):
    d = t.contiguous()
    return d, int(np.prod(d.shape[:-1])) if len(d.shape) > 1 else 1


def _fused_rms_norm(n: Node, x: List[Tensor]) -> Tensor:
    h, w = x
    hd, rows = _rows(h)
    out = Tensor._alloc(hd.shape, hd.dtype, hd.device)
    _lib.call("rb_norm", hd.device.ctx, _lib.NORM_RMS, hd.ptr(), None, None, 0, None, w.contiguous().ptr(), None, float(n.params[0]),
              rows, hd.shape[-1], out.ptr(), None, hd.dtype)
    return out


def _fused_linear(n: Node, x: List[Tensor]) -> Tensor:
    h, w = x[0], x[1]
    b = x[2] if len(x) > 2 else None
    hd, rows = _rows(h)
    wd = w.contiguous()
    out = Tensor._alloc(hd.shape[:-1] + [wd.shape[0]], hd.dtype, hd.device)
    _lib.call("rb_linear", hd.device.ctx, hd.ptr(), wd.ptr(), b.contiguous().ptr() if b is not None else None, None, out.ptr(), rows,
              wd.shape[0], wd.shape[1], _lib.ACT_NONE, hd.dtype)
    return out


def _fused_gated_linear(n: Node, x: List[Tensor]) -> Tensor:
    h, wg, wu = x
    hd, rows = _rows(h)
    g, u = wg.contiguous(), wu.contiguous()
    out = Tensor._alloc(hd.shape[:-1] + [g.shape[0]], hd.dtype, hd.device)
    _lib.call("rb_gated_linear", hd.device.ctx, hd.ptr(), g.ptr(), u.ptr(), out.ptr(), rows, g.shape[0], g.shape[1], _lib.ACT_SILU,
              hd.dtype)
    return out


_FUSED = {"FusedRmsNorm": _fused_rms_norm, "FusedLinear": _fused_linear, "FusedGatedLinear": _fused_gated_linear}


# --------------------------------------------------------------------------------------------------
# the rewrite pass
# --------------------------------------------------------------------------------------------------
def _is(n: Node, op: str, n_in: Optional[int] = None) -> bool:
    return n.op == op and (n_in is None or len(n.inputs) == n_in)


def _match_linear(n: Node):
    """MatMul(x, Transpose(-1,-2)(W or Broadcast(W))) [+ bias]  ->  (x, W, bias)  (linear.rs:59-69)."""
    bias = None
    if _is(n, "Add", 2) and _is(n.inputs[0], "MatMul", 2) and len(n.inputs[1].shape) == 1:
        n, bias = n.inputs[0], n.inputs[1]
    if not _is(n, "MatMul", 2):
        return None
    x, wt = n.inputs
    if not _is(wt, "Transpose", 1):
        return None
    r = len(wt.shape)
    if tuple(sorted(wt.params)) != (r - 2, r - 1):
        return None
    w = wt.inputs[0]
    if _is(w, "Broadcast", 1):
        w = w.inputs[0]
    if len(w.shape) != 2 or (bias is not None and bias.shape[0] != w.shape[0]):
        return None
    return x, w, bias


def _match_rms_norm(n: Node):
    """Mul(Mul(w, x), Rsqrt(AddScalar(ReduceSum(Square(MulScalar(x, 1/sqrt(H))), last, keep), eps)))  (rms_norm.rs:18-22)."""
    if not _is(n, "Mul", 2):
        return None
    wx, r = n.inputs
    if not (_is(wx, "Mul", 2) and _is(r, "Rsqrt", 1)):
        return None
    w, x = wx.inputs
    if len(w.shape) != 1:
        w, x = x, w
    if len(w.shape) != 1:
        return None
    a = r.inputs[0]
    if not _is(a, "AddScalar", 1):
        return None
    eps = a.params[0]
    s = a.inputs[0]
    if not (_is(s, "ReduceSum", 1) and s.params == (len(x.shape) - 1, True)):
        return None
    sq = s.inputs[0]
    if not (_is(sq, "Square", 1) and _is(sq.inputs[0], "MulScalar", 1)):
        return None
    ms = sq.inputs[0]
    if ms.inputs[0] is not x or abs(ms.params[0] - 1.0 / math.sqrt(x.shape[-1])) > 1e-9 or w.shape[0] != x.shape[-1]:
        return None
    return x, w, eps


def _match_silu(n: Node):
    """Div(g, AddScalar(Exp(Negative(g)), 1))  ->  g."""
    if not _is(n, "Div", 2):
        return None
    g, d = n.inputs
    if _is(d, "AddScalar", 1) and d.params[0] == 1.0 and _is(d.inputs[0], "Exp", 1) and _is(d.inputs[0].inputs[0], "Negative", 1) \
            and d.inputs[0].inputs[0].inputs[0] is g:
        return g
    return None


def optimize(outputs: Sequence[LazyTensor]) -> List[LazyTensor]:
    """Returns outputs over a rewritten graph: shared constants (what rai's `optimize` does, optimize.rs:41-87) and the
    three fusions named at the top.  The input graph is left as it was."""
    consts: Dict[tuple, Node] = {}
    done: Dict[int, Node] = {}
    stats = {"constants_shared": 0, "rms_norm": 0, "linear": 0, "gated_linear": 0}

    def rewrite(n: Node) -> Node:
        if id(n) in done:
            return done[id(n)]
        out = None
        if n.op == "Full":
            key = (n.params, tuple(n.shape), n.dtype)
            if key in consts:
                stats["constants_shared"] += 1
            out = consts.setdefault(key, n)
        elif n.op == "Const":
            out = n
        if out is None:
            m = _match_rms_norm(n)
            if m and n.dtype in (_lib.BF16, _lib.F32):
                x, w, eps = m
                out = Node("FusedRmsNorm", (eps,), [rewrite(x), rewrite(w)], n.shape, n.dtype, n.device)
                stats["rms_norm"] += 1
        if out is None and _is(n, "Mul", 2):
            for a, b in (n.inputs, n.inputs[::-1]):
                g = _match_silu(a)
                lg, lu = (_match_linear(g) if g is not None else None), _match_linear(b)
                if lg and lu and lg[0] is lu[0] and lg[2] is None and lu[2] is None and lg[1].shape == lu[1].shape:
                    out = Node("FusedGatedLinear", (), [rewrite(lg[0]), rewrite(lg[1]), rewrite(lu[1])], n.shape, n.dtype, n.device)
                    stats["gated_linear"] += 1
                    break
        if out is None:
            m = _match_linear(n)
            if m and n.dtype in (_lib.BF16, _lib.F32):
                x, w, b = m
                out = Node("FusedLinear", (), [rewrite(x), rewrite(w)] + ([rewrite(b)] if b is not None else []), n.shape, n.dtype,
                           n.device)
                stats["linear"] += 1
        if out is None:
            out = Node(n.op, n.params, [rewrite(i) for i in n.inputs], n.shape, n.dtype, n.device, n.data)
        done[id(n)] = out
        return out

    outs = [LazyTensor(rewrite(o.node)) for o in outputs]
    optimize.last_stats = stats
    return outs


optimize.last_stats = {}
