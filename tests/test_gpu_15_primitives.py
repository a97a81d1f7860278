"""The primitive set (the Eval rules of rai-core/src/backend/candle.rs the decoders' unfused graphs
reach) against the CPU oracle's torch restatement of the same ops."""
import ctypes

import pytest
import torch

import rai_cpu
from rai_b200 import _lib

pytestmark = pytest.mark.gpu
P = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}
I64 = lambda xs: (ctypes.c_int64 * len(xs))(*xs)  # noqa: E731


def close(got, want, dtype):
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    want = want.float()
    assert float((got.cpu().float() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))


UNARY = [
    (_lib.UN_NEG, lambda x, s: x.neg(), False), (_lib.UN_EXP, lambda x, s: x.exp(), False),
    (_lib.UN_SQRT, lambda x, s: x.sqrt(), True), (_lib.UN_RSQRT, lambda x, s: rai_cpu.rsqrt(x), True),
    (_lib.UN_SQUARE, lambda x, s: x.square(), False), (_lib.UN_TANH, lambda x, s: x.tanh(), False),
    (_lib.UN_ERF, lambda x, s: x.erf(), False), (_lib.UN_SIN, lambda x, s: x.sin(), False),
    (_lib.UN_COS, lambda x, s: x.cos(), False), (_lib.UN_POWF, lambda x, s: x.pow(s), True),
    (_lib.UN_SILU, lambda x, s: rai_cpu.silu(x), False), (_lib.UN_GELU_TANH, lambda x, s: rai_cpu.new_gelu(x), False),
    (_lib.UN_GELU_ERF, lambda x, s: rai_cpu.gelu(x), False), (_lib.UN_RELU, lambda x, s: rai_cpu.relu(x), False),
    (_lib.UN_LOG, lambda x, s: x.log(), True), (_lib.UN_ABS, lambda x, s: x.abs(), False),
    (_lib.UN_RECIP, lambda x, s: x.reciprocal(), True), (_lib.UN_ADD_SCALAR, lambda x, s: x + s, False),
    (_lib.UN_MUL_SCALAR, lambda x, s: x * s, False),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("op,ref,positive", UNARY, ids=[str(u[0]) for u in UNARY])
def test_unary(cuda, dtype, op, ref, positive):
    g = torch.Generator().manual_seed(op)
    x = torch.randn(1000, generator=g)
    if positive:
        x = x.abs() + 0.5
    xd = x.to(dtype).cuda()
    out = torch.empty_like(xd)
    _lib.call("rb_unary", cuda.ctx, op, P(xd), P(out), xd.numel(), 3.0, DT[dtype])
    cuda.synchronize()
    close(out, ref(xd.cpu().float(), 3.0), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_binary_with_broadcast(cuda, dtype):
    g = torch.Generator().manual_seed(1)
    a = torch.randn(2, 3, 5, 7, generator=g).to(dtype).cuda()
    b = (torch.randn(3, 1, 7, generator=g).abs() + 0.5).to(dtype).cuda()   # broadcast over dims 0 and 2
    out = torch.empty_like(a)
    refs = {_lib.BIN_ADD: torch.add, _lib.BIN_SUB: torch.sub, _lib.BIN_MUL: torch.mul, _lib.BIN_DIV: torch.div,
            _lib.BIN_MAXIMUM: torch.maximum, _lib.BIN_MINIMUM: torch.minimum}
    for op, ref in refs.items():
        _lib.call("rb_binary", cuda.ctx, op, P(a), None, P(b), I64([0, 7, 0, 1]), P(out), 4, I64([2, 3, 5, 7]), DT[dtype])
        cuda.synchronize()
        close(out, ref(a.cpu().float(), b.cpu().float()), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1, 1), (5, 33), (16, 2048), (3, 5000)])
def test_softmax_and_reductions(cuda, dtype, rows, cols):
    g = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=g).to(dtype).cuda()
    out = torch.empty_like(x)
    _lib.call("rb_softmax_rows", cuda.ctx, P(x), P(out), rows, cols, DT[dtype])
    cuda.synchronize()
    close(out, rai_cpu.softmax_last(x.cpu().float()), dtype)
    red = torch.empty(rows, dtype=dtype, device="cuda")
    xf = x.cpu().float()
    for op, want in ((_lib.RED_SUM, xf.sum(-1)), (_lib.RED_MAX, xf.max(-1).values), (_lib.RED_MIN, xf.min(-1).values)):
        _lib.call("rb_reduce_rows", cuda.ctx, op, P(x), P(red), rows, cols, DT[dtype])
        cuda.synchronize()
        tol = 2e-5 if dtype == torch.float32 else 1e-2
        assert float((red.cpu().float() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))


def test_copy_strided_transpose_narrow_concat(cuda):
    x = torch.arange(2 * 3 * 4 * 5, dtype=torch.float32).reshape(2, 3, 4, 5).cuda()
    # transpose(1, 2) made contiguous (qwen2.rs:180-182 followed by a reshape)
    out = torch.empty(2, 4, 3, 5, dtype=torch.float32, device="cuda")
    _lib.call("rb_copy_strided", cuda.ctx, P(x), I64([60, 5, 20, 1]), 0, P(out), None, 0, 4, I64([2, 4, 3, 5]), 4)
    cuda.synchronize()
    assert torch.equal(out, x.transpose(1, 2).contiguous())
    # narrow(-1, 1, 3)
    out = torch.empty(2, 3, 4, 3, dtype=torch.float32, device="cuda")
    _lib.call("rb_copy_strided", cuda.ctx, P(x), I64([60, 20, 5, 1]), 1, P(out), None, 0, 4, I64([2, 3, 4, 3]), 4)
    cuda.synchronize()
    assert torch.equal(out, x.narrow(-1, 1, 3).contiguous())
    # cat([a, b], dim=1): each input written at its offset of the output
    a = torch.randn(2, 3, 4).to(torch.bfloat16).cuda()
    b = torch.randn(2, 2, 4).to(torch.bfloat16).cuda()
    out = torch.empty(2, 5, 4, dtype=torch.bfloat16, device="cuda")
    _lib.call("rb_copy_strided", cuda.ctx, P(a), None, 0, P(out), I64([20, 4, 1]), 0, 3, I64([2, 3, 4]), 2)
    _lib.call("rb_copy_strided", cuda.ctx, P(b), None, 0, P(out), I64([20, 4, 1]), 12, 3, I64([2, 2, 4]), 2)
    cuda.synchronize()
    assert torch.equal(out, torch.cat([a, b], 1))


def test_cast_fill_arange(cuda):
    x = torch.randn(777).cuda()
    out = torch.empty(777, dtype=torch.bfloat16, device="cuda")
    _lib.call("rb_cast", cuda.ctx, P(x), _lib.F32, P(out), _lib.BF16, 777)
    cuda.synchronize()
    assert torch.equal(out, x.to(torch.bfloat16))
    back = torch.empty(777, dtype=torch.float32, device="cuda")
    _lib.call("rb_cast", cuda.ctx, P(out), _lib.BF16, P(back), _lib.F32, 777)
    u8 = torch.tensor([0, 1, 200], dtype=torch.uint8).cuda()
    f = torch.empty(3, dtype=torch.float32, device="cuda")
    _lib.call("rb_cast", cuda.ctx, P(u8), _lib.U8, P(f), _lib.F32, 3)
    cuda.synchronize()
    assert torch.equal(back, out.float()) and f.tolist() == [0.0, 1.0, 200.0]
    full = torch.empty(100, dtype=torch.float32, device="cuda")
    _lib.call("rb_fill", cuda.ctx, P(full), 100, -2.5, _lib.F32)
    ar = torch.empty(100, dtype=torch.int32, device="cuda")
    _lib.call("rb_arange", cuda.ctx, P(ar), 100, 3.0, 2.0, _lib.U32)
    cuda.synchronize()
    assert torch.all(full == -2.5) and ar.tolist() == list(range(3, 203, 2))


def test_index_select_gather_where_are_bit_exact(cuda):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(3, 10, 6, generator=g).to(torch.bfloat16).cuda()
    idx = torch.tensor([9, 0, 0, 4], dtype=torch.int32).cuda()
    out = torch.empty(3, 4, 6, dtype=torch.bfloat16, device="cuda")
    _lib.call("rb_index_select", cuda.ctx, P(x), 3, 10, 6, P(idx), 4, P(out), 2)
    cuda.synchronize()
    assert torch.equal(out, x.index_select(1, idx.long()))
    y = torch.randn(5, 8, generator=g).cuda()
    gi = torch.randint(0, 8, (5, 3), generator=g).to(torch.int32).cuda()
    go = torch.empty(5, 3, dtype=torch.float32, device="cuda")
    _lib.call("rb_gather_last", cuda.ctx, P(y), 5, 8, P(gi), 3, P(go), 4)
    cond = (torch.rand(40, generator=g) > 0.5).to(torch.uint8).cuda()
    a, b = torch.randn(40, generator=g).cuda(), torch.randn(40, generator=g).cuda()
    wo = torch.empty(40, dtype=torch.float32, device="cuda")
    _lib.call("rb_where", cuda.ctx, P(cond), P(a), P(b), P(wo), 40, _lib.F32)
    cuda.synchronize()
    assert torch.equal(go, y.gather(1, gi.long()))
    assert torch.equal(wo, torch.where(cond.bool(), a, b))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_matmul_forms(cuda, dtype):
    g = torch.Generator().manual_seed(3)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    # q @ k^T style: batched, row-major B ([k, n])
    a = torch.randn(6, 17, 32, generator=g).to(dtype).cuda()
    b = torch.randn(6, 32, 24, generator=g).to(dtype).cuda()
    c = torch.empty(6, 17, 24, dtype=dtype, device="cuda")
    _lib.call("rb_matmul", cuda.ctx, P(a), P(b), P(c), 6, 17, 24, 32, 17 * 32, 32 * 24, 0, DT[dtype])
    cuda.synchronize()
    want = a.cpu().float() @ b.cpu().float()
    assert float((c.cpu().float() - want).abs().max()) <= tol * float(want.abs().max())
    # Linear style: the weight [n, k] broadcast over the batch (rai-nn/src/linear.rs:59-69)
    w = torch.randn(24, 32, generator=g).to(dtype).cuda()
    _lib.call("rb_matmul", cuda.ctx, P(a), P(w), P(c), 6, 17, 24, 32, 17 * 32, 0, 1, DT[dtype])
    cuda.synchronize()
    want = a.cpu().float() @ w.cpu().float().t()
    assert float((c.cpu().float() - want).abs().max()) <= tol * float(want.abs().max())
