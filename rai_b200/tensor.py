"""`Tensor` on `Cuda`: the host-side mirror of rai-core's tensor / primitive-dispatch surface
(rai-core/src/tensor.rs, ops/*.rs, dispatch.rs) over the primitive entry points of the C ABI.

Every op looks its rule up in a registry keyed by (device type, op name) — the Python statement of
`EVAL_DISPATCHER` (rai-core/src/dispatch.rs:159-212) — and the rules registered here for `Cuda`
call `rb_unary`, `rb_binary`, `rb_matmul`, … .  Evaluation is eager (the reference is lazy and
evaluates on `as_vec`; the values are the same).  Views (transpose, narrow, broadcast, reshape of a
dense tensor) share storage like candle's layouts do; an op that needs dense input makes it dense
with `rb_copy_strided`, which is what candle's `contiguous()` does (candle.rs:417-440,980-988).

torch is used for device memory only.  This layer is the correctness net for arbitrary graphs; the
decoder driver uses the fused kernels instead.
"""
from __future__ import annotations

import ctypes
import math
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from . import shape as _shape
from .device import Cuda

_TORCH = {_lib.F32: torch.float32, _lib.BF16: torch.bfloat16, _lib.U32: torch.int32, _lib.U8: torch.uint8}
_TAG = {v: k for k, v in _TORCH.items()}
_ESIZE = {_lib.F32: 4, _lib.BF16: 2, _lib.U32: 4, _lib.U8: 1}

# ------------------------------------------------------------------------------ dispatch registry
_RULES: Dict[Tuple[type, str], Callable] = {}


def register(device_type: type, op: str, rule: Callable) -> None:
    """dispatch::register (rai-core/src/dispatch.rs:181-204): inserts or overwrites the rule."""
    _RULES[(device_type, op)] = rule


def eval_rule(device, op: str) -> Callable:
    """dispatch::eval_rule (dispatch.rs:207-212); a missing rule is Error::Unimplemented (eval.rs:40-43)."""
    rule = _RULES.get((type(device), op))
    if rule is None:
        raise _lib.RaiB200Error(-7, f"op {op!r} has no rule for device {device!r}")
    return rule


def _i64(xs: Sequence[int]):
    return (ctypes.c_int64 * max(1, len(xs)))(*[int(x) for x in xs])


def _dense_strides(shape: Sequence[int]) -> List[int]:
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= s
    return list(reversed(st))


def _resolve_dim(dim: int, rank: int) -> int:
    """Negative dims count from the end (rai-core/src/dim.rs:7-104)."""
    try:
        return _shape.dim([0] * rank, dim)
    except IndexError:
        raise _lib.RaiB200Error(-2, f"dim {dim} out of range for rank {rank}")


class Tensor:
    """A strided view over device storage: (storage, shape, strides in elements, offset)."""

    def __init__(self, storage: torch.Tensor, shape, strides, offset, dtype: int, device: Cuda):
        self.storage, self.shape, self.strides, self.offset = storage, list(shape), list(strides), int(offset)
        self.dtype, self.device = dtype, device

    # ---- construction / readback -------------------------------------------------------------
    @staticmethod
    def _alloc(shape, dtype: int, device: Cuda) -> "Tensor":
        n = int(np.prod(shape)) if len(shape) else 1
        st = torch.empty(max(n, 1), dtype=_TORCH[dtype], device=f"cuda:{device.id}")
        return Tensor(st, shape, _dense_strides(shape), 0, dtype, device)

    @staticmethod
    def from_array(data, shape, device: Cuda, dtype: Optional[int] = None) -> "Tensor":
        """ops::FromArray + ToDevice (candle.rs:241-273,776-790)."""
        a = np.asarray(data)
        if dtype is None:
            dtype = _lib.U32 if a.dtype.kind in "iu" and a.dtype.itemsize >= 4 else _lib.U8 if a.dtype.kind in "iub" else _lib.F32
        t = torch.from_numpy(np.ascontiguousarray(a.astype({_lib.F32: np.float32, _lib.U32: np.int32, _lib.U8: np.uint8,
                                                            _lib.BF16: np.float32}[dtype]))).reshape(-1)
        out = Tensor._alloc(list(shape), dtype, device)
        out.storage[: t.numel()].copy_(t.to(_TORCH[dtype]))
        return out

    @staticmethod
    def full(value: float, shape, dtype: int, device: Cuda) -> "Tensor":
        return eval_rule(device, "Full")(device, float(value), list(shape), dtype)

    @staticmethod
    def arange(start, stop, device: Cuda, dtype: int = _lib.U32, step=1) -> "Tensor":
        return eval_rule(device, "Arange")(device, float(start), float(stop), float(step), dtype)

    def numel(self) -> int:
        return int(np.prod(self.shape)) if self.shape else 1

    def is_dense(self) -> bool:
        return self.strides == _dense_strides(self.shape)

    def ptr(self) -> ctypes.c_void_p:
        return ctypes.c_void_p(self.storage.data_ptr() + self.offset * _ESIZE[self.dtype])

    def as_vec(self) -> np.ndarray:
        """TensorLike::as_vec (tensor.rs:198-201): dense float32 / integer numpy copy."""
        d = self.contiguous()
        self.device.synchronize()
        flat = d.storage[d.offset: d.offset + d.numel()]
        flat = flat.float() if d.dtype in (_lib.BF16, _lib.F32) else flat
        return flat.cpu().numpy().reshape(d.shape)

    def size(self, dim: int) -> int:
        return self.shape[_resolve_dim(dim, len(self.shape))]

    # ---- views ---------------------------------------------------------------------------------
    def _view(self, shape, strides, offset) -> "Tensor":
        return Tensor(self.storage, shape, strides, offset, self.dtype, self.device)

    def transpose(self, d0: int, d1: int) -> "Tensor":   # ops/transpose.rs:53-61
        r = len(self.shape)
        d0, d1 = _resolve_dim(d0, r), _resolve_dim(d1, r)
        sh, st = list(self.shape), list(self.strides)
        sh[d0], sh[d1], st[d0], st[d1] = sh[d1], sh[d0], st[d1], st[d0]
        return self._view(sh, st, self.offset)

    def t(self) -> "Tensor":
        return self.transpose(-1, -2)

    def permute(self, dims) -> "Tensor":   # ops/permute.rs:51-60: output dimension i is input dimension dims[i]
        r = len(self.shape)
        dims = [_resolve_dim(int(d), r) for d in dims]
        if sorted(dims) != list(range(r)):
            raise _lib.RaiB200Error(-2, f"permute{tuple(dims)} is not a permutation of the {r} dimensions of {self.shape}")
        return self._view([self.shape[d] for d in dims], [self.strides[d] for d in dims], self.offset)

    def narrow(self, dim: int, start: int, length: int) -> "Tensor":   # ops/narrow.rs:82-90
        d = _resolve_dim(dim, len(self.shape))
        if start < 0 or start + length > self.shape[d]:
            raise _lib.RaiB200Error(-2, f"narrow({dim}, {start}, {length}) exceeds {self.shape}")
        sh = list(self.shape)
        sh[d] = length
        return self._view(sh, self.strides, self.offset + start * self.strides[d])

    def broadcast_to(self, shape) -> "Tensor":   # ops/broadcast.rs:58-95, shape.rs:88-127
        shape = list(shape)
        pad = len(shape) - len(self.shape)
        if pad < 0:
            raise _lib.RaiB200Error(-2, f"cannot broadcast {self.shape} to {shape}")
        sh, st = [1] * pad + self.shape, [0] * pad + self.strides
        out = []
        for have, want, s in zip(sh, shape, st):
            if have == want:
                out.append(s)
            elif have == 1:
                out.append(0)
            else:
                raise _lib.RaiB200Error(-2, f"cannot broadcast {self.shape} to {shape}")
        return self._view(shape, out, self.offset)

    def unsqueeze(self, dim: int) -> "Tensor":
        d = dim + len(self.shape) + 1 if dim < 0 else dim
        return self._view(self.shape[:d] + [1] + self.shape[d:], self.strides[:d] + [0] + self.strides[d:], self.offset)

    def squeeze(self, dim: int) -> "Tensor":
        d = _resolve_dim(dim, len(self.shape))
        if self.shape[d] != 1:
            return self
        return self._view(self.shape[:d] + self.shape[d + 1:], self.strides[:d] + self.strides[d + 1:], self.offset)

    def reshape(self, shape) -> "Tensor":   # ops/reshape.rs:50-78: copies when the source is not dense
        shape = list(shape)
        if -1 in shape:
            known = int(np.prod([s for s in shape if s != -1]))
            shape[shape.index(-1)] = self.numel() // max(known, 1)
        if int(np.prod(shape)) != self.numel():
            raise _lib.RaiB200Error(-2, f"cannot reshape {self.shape} to {shape}")   # OpError::IncompatibleShape
        d = self.contiguous()
        return d._view(shape, _dense_strides(shape), d.offset)

    def flatten(self, start: int = 0) -> "Tensor":
        s = _resolve_dim(start, len(self.shape))
        return self.reshape(self.shape[:s] + [int(np.prod(self.shape[s:]))])

    def contiguous(self) -> "Tensor":   # ops/to_contiguous.rs:32-38
        return self if self.is_dense() else eval_rule(self.device, "ToContiguous")(self)

    # ---- ops: each goes through the registry ---------------------------------------------------
    def _un(self, op: str, scalar: float = 0.0) -> "Tensor":
        return eval_rule(self.device, op)(self, scalar)

    def _bin(self, op: str, other) -> "Tensor":
        if not isinstance(other, Tensor):
            # rai materialises a full-shape constant for `tensor op scalar` (ops/mod.rs:266-290); here the
            # scalar is a kernel argument
            if op == "Add":
                return self._un("AddScalar", float(other))
            if op == "Sub":
                return self._un("AddScalar", -float(other))
            if op == "Mul":
                return self._un("MulScalar", float(other))
            if op == "Div":
                return self._un("MulScalar", 1.0 / float(other))
            other = Tensor.full(float(other), [], self.dtype, self.device)
        return eval_rule(self.device, op)(self, other)

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
    def sin(self): return self._un("Sin")
    def cos(self): return self._un("Cos")
    def powf(self, e: float): return self._un("Powf", e)

    # hlops/activations.rs:5-32 written as the reference composes them
    def silu(self): return self / (self.neg().exp() + 1.0)
    def gelu(self): return self * 0.5 * ((self / math.sqrt(2.0)).erf() + 1.0)
    def new_gelu(self): return 0.5 * self * (((self + 0.044715 * self.powf(3.0)) * math.sqrt(2.0 / math.pi)).tanh() + 1.0)
    def relu(self): return self.maximum(Tensor.full(0.0, [], self.dtype, self.device))

    def to_dtype(self, dtype: int) -> "Tensor":
        return self if dtype == self.dtype else eval_rule(self.device, "ToDType")(self, dtype)

    def matmul(self, other: "Tensor") -> "Tensor":
        return eval_rule(self.device, "MatMul")(self, other)

    def softmax(self, dim: int = -1) -> "Tensor":
        return eval_rule(self.device, "Softmax")(self, dim)

    def sum(self, dim: int = -1, keep_dim: bool = False) -> "Tensor":
        return eval_rule(self.device, "ReduceSum")(self, dim, keep_dim)

    def max(self, dim: int = -1, keep_dim: bool = False) -> "Tensor":
        return eval_rule(self.device, "ReduceMax")(self, dim, keep_dim)

    def mean(self, dim: int = -1, keep_dim: bool = False) -> "Tensor":   # hlops/mean.rs:4-7
        return self.sum(dim, keep_dim) / float(self.size(dim))

    def var(self, dim: int = -1, keep_dim: bool = False) -> "Tensor":    # hlops/var.rs:33-38 (ddof 0)
        m = self.mean(dim, True)
        return (self - m).square().sum(dim, keep_dim) / float(self.size(dim))

    # the rest of the rule set (dispatch.rs:41-157): what graphs beyond the decoders use
    def minimum(self, o): return self._bin("Minimum", o)
    def log(self): return self._un("Log")
    def log2(self): return self._un("Log2")
    def log10(self): return self._un("Log10")
    def abs(self): return self._un("Abs")
    def sign(self): return self._un("Sign")
    def eq(self, o): return eval_rule(self.device, "Equal")(self, o)
    def ne(self, o): return eval_rule(self.device, "NotEqual")(self, o)
    def gt(self, o): return eval_rule(self.device, "Greater")(self, o)
    def ge(self, o): return eval_rule(self.device, "GreaterEqual")(self, o)
    def lt(self, o): return eval_rule(self.device, "Less")(self, o)
    def le(self, o): return eval_rule(self.device, "LessEqual")(self, o)

    def min(self, dim=-1, keep_dim: bool = False) -> "Tensor":
        return eval_rule(self.device, "ReduceMin")(self, dim, keep_dim)

    def log_softmax(self, dim: int = -1) -> "Tensor":
        return eval_rule(self.device, "LogSoftmax")(self, dim)

    def argmin(self, dim: int = -1) -> "Tensor":
        return eval_rule(self.device, "ArgMin")(self, dim)

    def scatter_add(self, dim: int, index: "Tensor", source: "Tensor") -> "Tensor":   # ops/scatter_add.rs
        return eval_rule(self.device, "ScatterAdd")(self, source, index, dim)

    def index_add(self, dim: int, index: "Tensor", source: "Tensor") -> "Tensor":     # ops/index_add.rs
        return eval_rule(self.device, "IndexAdd")(self, source, index, dim)

    def conv2d(self, w: "Tensor", padding=(0, 0), stride=(1, 1), dilation=(1, 1)) -> "Tensor":   # ops/conv2d.rs
        return eval_rule(self.device, "Conv2d")(self, w, padding, stride, dilation)

    def conv1d(self, w: "Tensor", padding=0, stride=1, dilation=1) -> "Tensor":                    # ops/conv1d.rs
        y = self.unsqueeze(2).conv2d(w.unsqueeze(2), (0, padding), (1, stride), (1, dilation))
        return y.squeeze(2)

    def conv_transpose2d(self, w: "Tensor", padding=(0, 0), out_padding=(0, 0), stride=(1, 1), dilation=(1, 1)) -> "Tensor":
        return eval_rule(self.device, "ConvTranspose2d")(self, w, padding, out_padding, stride, dilation)

    def conv_transpose1d(self, w: "Tensor", padding=0, out_padding=0, stride=1, dilation=1) -> "Tensor":
        y = self.unsqueeze(2).conv_transpose2d(w.unsqueeze(2), (0, padding), (0, out_padding), (1, stride), (1, dilation))
        return y.squeeze(2)

    def max_pool2d(self, kernel, stride=None, padding=(0, 0), dilation=(1, 1)) -> "Tensor":   # ops/max_pool2d.rs
        return eval_rule(self.device, "MaxPool2d")(self, kernel, stride or kernel, padding, dilation)

    def avg_pool2d(self, kernel, stride=None, padding=(0, 0)) -> "Tensor":                    # ops/avg_pool2d.rs
        return eval_rule(self.device, "AvgPool2d")(self, kernel, stride or kernel, padding)

    def max_pool1d(self, kernel, stride=None, padding=0, dilation=1) -> "Tensor":
        return self.unsqueeze(2).max_pool2d((1, kernel), (1, stride or kernel), (0, padding), (1, dilation)).squeeze(2)

    def avg_pool1d(self, kernel, stride=None, padding=0) -> "Tensor":
        return self.unsqueeze(2).avg_pool2d((1, kernel), (1, stride or kernel), (0, padding)).squeeze(2)

    def upsample_nearest2d(self, size) -> "Tensor":                                            # ops/upsample_nearest2d.rs
        return eval_rule(self.device, "UpsampleNearest2d")(self, size)

    def upsample_nearest1d(self, size: int) -> "Tensor":
        return self.unsqueeze(2).upsample_nearest2d((1, size)).squeeze(2)

    def index_select(self, dim: int, index: "Tensor") -> "Tensor":
        return eval_rule(self.device, "IndexSelect")(self, dim, index)

    def gather(self, dim: int, index: "Tensor") -> "Tensor":
        return eval_rule(self.device, "Gather")(self, dim, index)

    def where_cond(self, on_true: "Tensor", on_false: "Tensor") -> "Tensor":
        """self is the u8 condition (ops/where.rs:37-45)."""
        return eval_rule(self.device, "Where")(on_true, on_false, self)

    def argmax(self, dim: int = -1) -> "Tensor":
        return eval_rule(self.device, "ArgMax")(self, dim)

    @staticmethod
    def cat(tensors: Sequence["Tensor"], dim: int) -> "Tensor":
        return eval_rule(tensors[0].device, "Concatenate")(list(tensors), dim)


# ------------------------------------------------------------------------------ rules for Cuda
def _strided_copy(x: Tensor, out: Tensor, out_strides, out_offset) -> None:
    _lib.call("rb_copy_strided", x.device.ctx, ctypes.c_void_p(x.storage.data_ptr()), _i64(x.strides), x.offset,
              ctypes.c_void_p(out.storage.data_ptr()), _i64(out_strides), out_offset, len(x.shape), _i64(x.shape),
              _ESIZE[x.dtype])


def _to_contiguous(x: Tensor) -> Tensor:
    if len(x.shape) > 6:
        raise _lib.RaiB200Error(-7, "copies of more than 6 dimensions")
    out = Tensor._alloc(x.shape, x.dtype, x.device)
    if x.numel():
        _strided_copy(x, out, out.strides, 0)
    return out


_UNARY = {"Negative": _lib.UN_NEG, "Exp": _lib.UN_EXP, "Sqrt": _lib.UN_SQRT, "Rsqrt": _lib.UN_RSQRT, "Square": _lib.UN_SQUARE,
          "Tanh": _lib.UN_TANH, "Erf": _lib.UN_ERF, "Sin": _lib.UN_SIN, "Cos": _lib.UN_COS, "Powf": _lib.UN_POWF,
          "AddScalar": _lib.UN_ADD_SCALAR, "MulScalar": _lib.UN_MUL_SCALAR, "Log": _lib.UN_LOG, "Abs": _lib.UN_ABS,
          "Sign": _lib.UN_SIGN, "Log2": _lib.UN_LOG2, "Log10": _lib.UN_LOG10}
_BINARY = {"Add": _lib.BIN_ADD, "Sub": _lib.BIN_SUB, "Mul": _lib.BIN_MUL, "Div": _lib.BIN_DIV, "Maximum": _lib.BIN_MAXIMUM,
           "Minimum": _lib.BIN_MINIMUM}
_COMPARE = {"Equal": _lib.CMP_EQ, "NotEqual": _lib.CMP_NE, "Greater": _lib.CMP_GT, "GreaterEqual": _lib.CMP_GE,
            "Less": _lib.CMP_LT, "LessEqual": _lib.CMP_LE}


def _unary_rule(code):
    def rule(x: Tensor, scalar: float) -> Tensor:
        d = x.contiguous()
        out = Tensor._alloc(d.shape, d.dtype, d.device)
        _lib.call("rb_unary", d.device.ctx, code, d.ptr(), out.ptr(), d.numel(), float(scalar), d.dtype)
        return out
    return rule


def _binary_rule(code):
    def rule(a: Tensor, b: Tensor) -> Tensor:
        # broadcast_binary_op! (ops/mod.rs:299-340): both sides are broadcast to the common shape first
        ra, rb_ = len(a.shape), len(b.shape)
        r = max(ra, rb_)
        sa, sb = [1] * (r - ra) + a.shape, [1] * (r - rb_) + b.shape
        shape = []
        for x, y in zip(sa, sb):
            if x != y and 1 not in (x, y):
                raise _lib.RaiB200Error(-2, f"cannot broadcast {a.shape} with {b.shape}")
            shape.append(max(x, y))
        a, b = a.broadcast_to(shape), b.broadcast_to(shape)
        if len(shape) > 4:  # the kernel takes up to 4 dims: make the operands dense and flatten
            a, b = a.contiguous().reshape([-1]), b.contiguous().reshape([-1])
        out = Tensor._alloc(shape, a.dtype, a.device)
        _lib.call("rb_binary", a.device.ctx, code, a.ptr(), _i64(a.strides), b.ptr(), _i64(b.strides), out.ptr(),
                  len(a.shape), _i64(a.shape), a.dtype)
        return out
    return rule


def _matmul(a: Tensor, b: Tensor) -> Tensor:
    """ops/matmul.rs:34-70 + candle.rs:401-443: batched, batch dims broadcast (shape.rs:130-160)."""
    if len(a.shape) < 2 or len(b.shape) < 2:
        raise _lib.RaiB200Error(-7, "matmul of rank-1 operands")
    m, k = a.shape[-2], a.shape[-1]
    k2, n = b.shape[-2], b.shape[-1]
    if k != k2:
        raise _lib.RaiB200Error(-2, f"matmul of {a.shape} and {b.shape}")
    try:
        batch_shape = _shape.broadcast_matmul(a.shape, b.shape)[0][:-2]   # shape.rs:129-160
    except ValueError as e:
        raise _lib.RaiB200Error(-2, str(e))
    batch = int(np.prod(batch_shape)) if batch_shape else 1
    # Linear's `weight.broadcast_left(batch).t()` (linear.rs:59-69): B is a broadcast, transposed [n, k] matrix
    b_is_linear = b.strides[-1] == k and b.strides[-2] == 1 and all(s == 0 for s in b.strides[:-2])
    ad = a.broadcast_to(batch_shape + [m, k]).contiguous()
    out = Tensor._alloc(batch_shape + [m, n], a.dtype, a.device)
    if b_is_linear:
        _lib.call("rb_matmul", a.device.ctx, ad.ptr(), b.ptr(), out.ptr(), batch, m, n, k, m * k, 0, 1, a.dtype)
    else:
        bd = b.broadcast_to(batch_shape + [k, n]).contiguous()
        _lib.call("rb_matmul", a.device.ctx, ad.ptr(), bd.ptr(), out.ptr(), batch, m, n, k, m * k, k * n, 0, a.dtype)
    return out


def _rows_last(x: Tensor, dim: int) -> Tuple[Tensor, bool, int]:
    """x with `dim` moved to the end (the other dims keep their order), dense."""
    d = _resolve_dim(dim, len(x.shape))
    moved = d != len(x.shape) - 1
    if moved:
        order = [i for i in range(len(x.shape)) if i != d] + [d]
        x = x._view([x.shape[i] for i in order], [x.strides[i] for i in order], x.offset)
    return x.contiguous(), moved, d


def _softmax(x: Tensor, dim: int) -> Tensor:
    xs, moved, d = _rows_last(x, dim)
    out = Tensor._alloc(xs.shape, xs.dtype, xs.device)
    cols = xs.shape[-1]
    _lib.call("rb_softmax_rows", xs.device.ctx, xs.ptr(), out.ptr(), xs.numel() // cols, cols, xs.dtype)
    if moved:  # put the softmax dim back where it was
        r = len(out.shape)
        order = list(range(d)) + [r - 1] + list(range(d, r - 1))
        out = out._view([out.shape[i] for i in order], [out.strides[i] for i in order], out.offset)
    return out


def _reduce_rule(code):
    def rule(x: Tensor, dim, keep_dim: bool) -> Tensor:
        if not isinstance(dim, int):
            # ReduceSum{dims, keep_dim} over any set of dims (ops/reduce_sum.rs:63-76): the reduced dims are moved to
            # the end and flattened into one, then it is a row reduction
            r = len(x.shape)
            dims = sorted({_resolve_dim(d, r) for d in dim})
            kept = [i for i in range(r) if i not in dims]
            order = kept + dims
            moved_x = x._view([x.shape[i] for i in order], [x.strides[i] for i in order], x.offset).contiguous()
            cols = int(np.prod([x.shape[i] for i in dims])) if dims else 1
            flat = moved_x.reshape([x.shape[i] for i in kept] + [cols])
            out = rule(flat, -1, False)
            if keep_dim:
                out = out.reshape([1 if i in dims else x.shape[i] for i in range(r)])
            return out
        xs, moved, d = _rows_last(x, dim)
        cols = xs.shape[-1]
        out = Tensor._alloc(xs.shape[:-1], xs.dtype, xs.device)
        _lib.call("rb_reduce_rows", xs.device.ctx, code, xs.ptr(), out.ptr(), xs.numel() // cols, cols, xs.dtype)
        return out.unsqueeze(d) if keep_dim else out
    return rule


def _index_select(x: Tensor, dim: int, index: Tensor) -> Tensor:
    d = _resolve_dim(dim, len(x.shape))
    xd, idx = x.contiguous(), index.contiguous()
    outer, inner = int(np.prod(xd.shape[:d])) if d else 1, int(np.prod(xd.shape[d + 1:])) if d + 1 < len(xd.shape) else 1
    out = Tensor._alloc(xd.shape[:d] + [idx.numel()] + xd.shape[d + 1:], xd.dtype, xd.device)
    _lib.call("rb_index_select", xd.device.ctx, xd.ptr(), outer, xd.shape[d], inner, idx.ptr(), idx.numel(), out.ptr(),
              _ESIZE[xd.dtype])
    return out


def _gather(x: Tensor, dim: int, index: Tensor) -> Tensor:
    d = _resolve_dim(dim, len(x.shape))
    if d != len(x.shape) - 1:   # move the gathered dim last on both operands, gather, move it back
        last = len(x.shape) - 1
        return _gather(x.transpose(d, last), -1, index.transpose(d, last)).transpose(d, last)
    xd, idx = x.contiguous(), index.contiguous()
    out = Tensor._alloc(idx.shape, xd.dtype, xd.device)
    _lib.call("rb_gather_last", xd.device.ctx, xd.ptr(), xd.numel() // xd.shape[-1], xd.shape[-1], idx.ptr(), idx.shape[-1],
              out.ptr(), _ESIZE[xd.dtype])
    return out


def _where(on_true: Tensor, on_false: Tensor, cond: Tensor) -> Tensor:
    shape = list(np.broadcast_shapes(tuple(on_true.shape), tuple(on_false.shape), tuple(cond.shape)))
    a, b, c = (t.broadcast_to(shape).contiguous() for t in (on_true, on_false, cond))
    out = Tensor._alloc(shape, a.dtype, a.device)
    _lib.call("rb_where", a.device.ctx, c.ptr(), a.ptr(), b.ptr(), out.ptr(), out.numel(), a.dtype)
    return out


def _argmax(x: Tensor, dim: int) -> Tensor:
    xs, _, _ = _rows_last(x, dim)
    out = Tensor._alloc(xs.shape[:-1], _lib.U32, xs.device)
    _lib.call("rb_argmax_rows", xs.device.ctx, xs.ptr(), xs.dtype, xs.numel() // xs.shape[-1], xs.shape[-1], out.ptr())
    return out


def _concatenate(ts: List[Tensor], dim: int) -> Tensor:
    d = _resolve_dim(dim, len(ts[0].shape))
    shape = list(ts[0].shape)
    shape[d] = sum(t.shape[d] for t in ts)
    out = Tensor._alloc(shape, ts[0].dtype, ts[0].device)
    at = 0
    for t in ts:   # each input is written at its offset of the output (candle's Tensor::cat, candle.rs:880-889)
        if t.numel():
            _strided_copy(t, out, out.strides, at * out.strides[d])
        at += t.shape[d]
    return out


def _to_dtype(x: Tensor, dtype: int) -> Tensor:
    d = x.contiguous()
    out = Tensor._alloc(d.shape, dtype, d.device)
    _lib.call("rb_cast", d.device.ctx, d.ptr(), d.dtype, out.ptr(), dtype, d.numel())
    return out


def _full(device: Cuda, value: float, shape, dtype: int) -> Tensor:
    out = Tensor._alloc(shape, dtype, device)
    _lib.call("rb_fill", device.ctx, out.ptr(), out.numel(), value, dtype)
    return out


def _arange(device: Cuda, start: float, stop: float, step: float, dtype: int) -> Tensor:
    n = max(0, int(math.ceil((stop - start) / step)))
    out = Tensor._alloc([n], dtype, device)
    _lib.call("rb_arange", device.ctx, out.ptr(), n, start, step, dtype)
    return out


def _compare_rule(code):
    def rule(a: Tensor, b) -> Tensor:
        if not isinstance(b, Tensor):
            b = Tensor.full(float(b), [], a.dtype, a.device)
        shape = list(np.broadcast_shapes(tuple(a.shape), tuple(b.shape)))
        a, b = a.broadcast_to(shape), b.broadcast_to(shape)
        if len(shape) > 4:
            a, b = a.contiguous().reshape([-1]), b.contiguous().reshape([-1])
        out = Tensor._alloc(shape, _lib.U8, a.device)
        _lib.call("rb_compare", a.device.ctx, code, a.ptr(), _i64(a.strides), b.ptr(), _i64(b.strides), out.ptr(), len(a.shape),
                  _i64(a.shape), a.dtype)
        return out
    return rule


def _log_softmax(x: Tensor, dim: int) -> Tensor:
    xs, moved, d = _rows_last(x, dim)
    out = Tensor._alloc(xs.shape, xs.dtype, xs.device)
    cols = xs.shape[-1]
    _lib.call("rb_log_softmax_rows", xs.device.ctx, xs.ptr(), out.ptr(), xs.numel() // cols, cols, xs.dtype)
    if moved:
        r = len(out.shape)
        order = list(range(d)) + [r - 1] + list(range(d, r - 1))
        out = out._view([out.shape[i] for i in order], [out.strides[i] for i in order], out.offset)
    return out


def _argmin(x: Tensor, dim: int) -> Tensor:
    xs, _, _ = _rows_last(x, dim)
    out = Tensor._alloc(xs.shape[:-1], _lib.U32, xs.device)
    _lib.call("rb_argmin_rows", xs.device.ctx, xs.ptr(), xs.dtype, xs.numel() // xs.shape[-1], xs.shape[-1], out.ptr())
    return out


def _scatter_rule(index_is_1d: bool):
    def rule(x: Tensor, source: Tensor, index: Tensor, dim: int) -> Tensor:
        """Inputs in the reference's order: x, source/updates, index (candle.rs:853-855, 993-995)."""
        d = _resolve_dim(dim, len(x.shape))
        xd, sd, idx = x.contiguous(), source.contiguous(), index.contiguous()
        outer = int(np.prod(xd.shape[:d])) if d else 1
        inner = int(np.prod(xd.shape[d + 1:])) if d + 1 < len(xd.shape) else 1
        out = Tensor._alloc(xd.shape, xd.dtype, xd.device)
        _lib.call("rb_scatter_add", xd.device.ctx, xd.ptr(), sd.ptr(), idx.ptr(), out.ptr(), outer, xd.shape[d], sd.shape[d],
                  inner, int(index_is_1d), xd.dtype)
        return out
    return rule


def _i32(xs: Sequence[int]):
    return (ctypes.c_int32 * max(1, len(xs)))(*[int(v) for v in xs])


def _conv2d(x: Tensor, w: Tensor, padding, stride, dilation) -> Tensor:
    xd, wd = x.contiguous(), w.contiguous()
    shape = (ctypes.c_int32 * 4)()
    args = (xd.device.ctx, xd.ptr(), _i32(xd.shape), wd.ptr(), _i32(wd.shape), _i32(padding), _i32(stride), _i32(dilation))
    _lib.call("rb_conv2d", *args, None, shape, xd.dtype)            # shape query
    out = Tensor._alloc(list(shape), xd.dtype, xd.device)
    _lib.call("rb_conv2d", *args, out.ptr(), shape, xd.dtype)
    return out


def _conv_transpose2d(x: Tensor, w: Tensor, padding, out_padding, stride, dilation) -> Tensor:
    xd, wd = x.contiguous(), w.contiguous()
    shape = (ctypes.c_int32 * 4)()
    args = (xd.device.ctx, xd.ptr(), _i32(xd.shape), wd.ptr(), _i32(wd.shape), _i32(padding), _i32(out_padding), _i32(stride),
            _i32(dilation))
    _lib.call("rb_conv_transpose2d", *args, None, shape, xd.dtype)
    out = Tensor._alloc(list(shape), xd.dtype, xd.device)
    _lib.call("rb_conv_transpose2d", *args, out.ptr(), shape, xd.dtype)
    return out


def _pool_rule(is_max: bool):
    def rule(x: Tensor, kernel, stride, padding, dilation=(1, 1)) -> Tensor:
        xd = x.contiguous()
        shape = (ctypes.c_int32 * 4)()
        args = (xd.device.ctx, int(is_max), xd.ptr(), _i32(xd.shape), _i32(kernel), _i32(stride), _i32(padding), _i32(dilation))
        _lib.call("rb_pool2d", *args, None, shape, xd.dtype)
        out = Tensor._alloc(list(shape), xd.dtype, xd.device)
        _lib.call("rb_pool2d", *args, out.ptr(), shape, xd.dtype)
        return out
    return rule


def _upsample_nearest2d(x: Tensor, size) -> Tensor:
    xd = x.contiguous()
    out = Tensor._alloc(xd.shape[:2] + [int(size[0]), int(size[1])], xd.dtype, xd.device)
    _lib.call("rb_upsample_nearest2d", xd.device.ctx, xd.ptr(), _i32(xd.shape), int(size[0]), int(size[1]), out.ptr(), xd.dtype)
    return out


def register_all() -> None:
    """The `register_backend!` list (rai-core/src/dispatch.rs:41-157) for the ops the decoders reach."""
    for name, code in _UNARY.items():
        register(Cuda, name, _unary_rule(code))
    for name, code in _BINARY.items():
        register(Cuda, name, _binary_rule(code))
    register(Cuda, "MatMul", _matmul)
    register(Cuda, "Softmax", _softmax)
    register(Cuda, "ReduceSum", _reduce_rule(_lib.RED_SUM))
    register(Cuda, "ReduceMax", _reduce_rule(_lib.RED_MAX))
    register(Cuda, "ReduceMin", _reduce_rule(_lib.RED_MIN))
    register(Cuda, "IndexSelect", _index_select)
    register(Cuda, "Gather", _gather)
    register(Cuda, "Where", _where)
    register(Cuda, "ArgMax", _argmax)
    register(Cuda, "Concatenate", _concatenate)
    register(Cuda, "ToContiguous", _to_contiguous)
    register(Cuda, "ToDType", _to_dtype)
    register(Cuda, "Full", _full)
    register(Cuda, "Arange", _arange)
    for name, code in _COMPARE.items():
        register(Cuda, name, _compare_rule(code))
    register(Cuda, "LogSoftmax", _log_softmax)
    register(Cuda, "ArgMin", _argmin)
    register(Cuda, "ScatterAdd", _scatter_rule(False))
    register(Cuda, "IndexAdd", _scatter_rule(True))
    register(Cuda, "Conv2d", _conv2d)
    register(Cuda, "ConvTranspose2d", _conv_transpose2d)
    register(Cuda, "MaxPool2d", _pool_rule(True))
    register(Cuda, "AvgPool2d", _pool_rule(False))
    register(Cuda, "UpsampleNearest2d", _upsample_nearest2d)


register_all()
