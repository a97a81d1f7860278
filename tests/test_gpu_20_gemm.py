"""Parity of the Linear kernels (tcgen05 bf16 GEMM and the plain fp32 GEMM) with the CPU oracle."""
import ctypes

import pytest
import torch

import rai_cpu
from rai_b200 import _lib

pytestmark = pytest.mark.gpu
P = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}
ACTS = {_lib.ACT_NONE: lambda v: v, _lib.ACT_SILU: rai_cpu.silu, _lib.ACT_GELU_TANH: rai_cpu.new_gelu,
        _lib.ACT_GELU_ERF: rai_cpu.gelu}


def make(m, n, k, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).to(dtype).cuda()
    w = (torch.randn(n, k, generator=g) * 0.05).to(dtype).cuda()
    w2 = (torch.randn(n, k, generator=g) * 0.05).to(dtype).cuda()
    b = torch.randn(n, generator=g).to(dtype).cuda()
    r = torch.randn(m, n, generator=g).to(dtype).cuda()
    return x, w, w2, b, r


def tol(dtype, ref):
    # bf16: one rounding of the output (2^-9 relative) plus accumulation-order noise
    return (8e-3 if dtype == torch.bfloat16 else 2e-5) * float(ref.abs().max()) + 1e-6


# (m, n, k): decode-sized (swapped operands), the tile edges, prefill-sized (normal operands), ragged
SHAPES = [(2, 192, 256), (2, 256, 64), (2, 256, 40), (2, 64, 256), (80, 256, 40), (2, 40, 256),  # 8-way shard shapes
          (1, 256, 128), (8, 384, 320), (64, 1152, 896), (64, 128, 64), (16, 136, 72), (100, 520, 256),
          (128, 512, 512), (200, 264, 192), (257, 512, 256), (300, 1000, 328), (1024, 768, 512), (640, 2048, 1024)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_linear_matches_oracle(cuda, dtype, m, n, k):
    x, w, _, b, r = make(m, n, k, dtype, m * 7 + n)
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    _lib.call("rb_linear", cuda.ctx, P(x), P(w), None, None, P(out), m, n, k, _lib.ACT_NONE, DT[dtype])
    cuda.synchronize()
    ref = rai_cpu.linear(x.cpu().float(), w.cpu().float(), None)
    assert float((out.cpu().float() - ref).abs().max()) <= tol(dtype, ref)
    # bias + activation + residual epilogue
    _lib.call("rb_linear", cuda.ctx, P(x), P(w), P(b), P(r), P(out), m, n, k, _lib.ACT_GELU_TANH, DT[dtype])
    cuda.synchronize()
    ref = rai_cpu.new_gelu(rai_cpu.linear(x.cpu().float(), w.cpu().float(), b.cpu().float())) + r.cpu().float()
    assert float((out.cpu().float() - ref).abs().max()) <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("act", [_lib.ACT_SILU, _lib.ACT_GELU_TANH])
@pytest.mark.parametrize("m,n,k", [(2, 40, 256), (2, 80, 256), (80, 40, 256), (1, 256, 128), (16, 200, 192), (64, 640, 896), (128, 384, 256), (130, 384, 256),
                                   (512, 1024, 512), (300, 328, 136)])
def test_gated_linear_matches_oracle(cuda, dtype, act, m, n, k):
    x, w, w2, _, _ = make(m, n, k, dtype, m + n + act)
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    _lib.call("rb_gated_linear", cuda.ctx, P(x), P(w), P(w2), P(out), m, n, k, act, DT[dtype])
    cuda.synchronize()
    xf = x.cpu().float()
    ref = ACTS[act](xf @ w.cpu().float().t()) * (xf @ w2.cpu().float().t())
    assert float((out.cpu().float() - ref).abs().max()) <= tol(dtype, ref)


@pytest.mark.parametrize("m,n,k,splits", [(64, 512, 896, 4), (8, 256, 2560, 5), (1, 128, 640, 3), (200, 384, 1024, 2),
                                          (64, 256, 192, 7)])
def test_linear_partials_sum_to_the_product(cuda, m, n, k, splits):
    x, w, _, _, _ = make(m, n, k, torch.bfloat16, k)
    part = torch.full((splits, m, n), float("nan"), dtype=torch.float32, device="cuda")
    _lib.call("rb_linear_partials", cuda.ctx, P(x), P(w), P(part), m, n, k, splits)
    cuda.synchronize()
    ref = x.cpu().float() @ w.cpu().float().t()
    got = part.sum(0).cpu()
    assert torch.isfinite(got).all()
    assert float((got - ref).abs().max()) <= 1e-4 * float(ref.abs().max()) + 1e-5  # float32 partials


def test_pick_splits_fills_the_gpu(cuda):
    sms = cuda.sm_count()
    s = _lib.lib().rb_linear_pick_splits(cuda.ctx, 64, 3584, 3584)
    assert 1 < s <= 16 and 28 * s <= sms
    assert _lib.lib().rb_linear_pick_splits(cuda.ctx, 64, 37888, 3584) == 1
    assert _lib.lib().rb_linear_pick_splits(cuda.ctx, 4096, 3584, 3584) == 1


def test_linear_is_deterministic(cuda):
    x, w, _, _, _ = make(64, 1024, 2048, torch.bfloat16, 5)
    outs = []
    for _ in range(3):
        out = torch.empty(64, 1024, dtype=torch.bfloat16, device="cuda")
        _lib.call("rb_linear", cuda.ctx, P(x), P(w), None, None, P(out), 64, 1024, 2048, _lib.ACT_NONE, _lib.BF16)
        cuda.synchronize()
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


def test_linear_rejects_bad_k(cuda):
    x, w, _, _, _ = make(4, 16, 12, torch.bfloat16, 1)
    out = torch.empty(4, 16, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.RaiB200Error):
        _lib.call("rb_linear", cuda.ctx, P(x), P(w), None, None, P(out), 4, 16, 12, _lib.ACT_NONE, _lib.BF16)


@pytest.mark.parametrize("seed", range(8))
def test_decode_sized_linear_over_many_seeds(cuda, seed):
    """The same tiny decode GEMMs on fresh data every time: a result that depends on what the previous
    launch left in shared or tensor memory would show up here."""
    for m, n, k in ((2, 192, 256), (2, 256, 64), (2, 256, 40), (2, 64, 256)):
        x, w, _, b, _ = make(m, n, k, torch.bfloat16, 1000 * seed + n + k)
        out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        _lib.call("rb_linear", cuda.ctx, P(x), P(w), P(b), None, P(out), m, n, k, _lib.ACT_NONE, _lib.BF16)
        cuda.synchronize()
        ref = rai_cpu.linear(x.cpu().float(), w.cpu().float(), b.cpu().float())
        assert float((out.cpu().float() - ref).abs().max()) <= tol(torch.bfloat16, ref), (m, n, k)
    x, w, w2, _, _ = make(2, 40, 256, torch.bfloat16, seed)
    out = torch.empty(2, 40, dtype=torch.bfloat16, device="cuda")
    _lib.call("rb_gated_linear", cuda.ctx, P(x), P(w), P(w2), P(out), 2, 40, 256, _lib.ACT_SILU, _lib.BF16)
    cuda.synchronize()
    xf = x.cpu().float()
    ref = rai_cpu.silu(xf @ w.cpu().float().t()) * (xf @ w2.cpu().float().t())
    assert float((out.cpu().float() - ref).abs().max()) <= tol(torch.bfloat16, ref)
