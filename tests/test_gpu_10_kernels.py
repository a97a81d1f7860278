"""Parity of the HBM-bound decoder kernels with the CPU oracle, through the C ABI."""
import ctypes
import math

import numpy as np
import pytest
import torch

import rai_cpu
from rai_b200 import _lib

pytestmark = pytest.mark.gpu
P = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.6e-2}


def dev(x, dtype):
    return x.to(device="cuda", dtype=dtype).contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [64, 896, 2050])
def test_embed_gather_is_bit_exact(cuda, dtype, hidden):
    g = torch.Generator().manual_seed(1)
    table = dev(torch.randn(1000, hidden, generator=g), dtype)
    ids = torch.tensor([0, 999, 5, 5, 123, 0, 7], dtype=torch.int32, device="cuda")
    out = torch.empty(len(ids), hidden, dtype=dtype, device="cuda")
    _lib.call("rb_embed_gather", cuda.ctx, P(table), DT[dtype], 1000, hidden, P(ids), len(ids), 1.0, P(out))
    cuda.synchronize()
    want = rai_cpu.embedding(table.cpu(), ids.cpu().long())
    assert torch.equal(out.cpu(), want)  # IndexSelect is a copy: bit for bit


def test_embed_gather_scale_and_empty(cuda):
    table = dev(torch.randn(50, 2048), torch.bfloat16)
    ids = torch.tensor([3, 49], dtype=torch.int32, device="cuda")
    out = torch.empty(2, 2048, dtype=torch.bfloat16, device="cuda")
    s = math.sqrt(2048.0)
    _lib.call("rb_embed_gather", cuda.ctx, P(table), _lib.BF16, 50, 2048, P(ids), 2, s, P(out))
    cuda.synchronize()
    want = (table.cpu().float()[[3, 49]] * np.float32(s)).to(torch.bfloat16)
    assert torch.equal(out.cpu(), want)
    _lib.call("rb_embed_gather", cuda.ctx, P(table), _lib.BF16, 50, 2048, P(ids), 0, 1.0, P(out))  # empty input


def test_embed_gather_out_of_range_id_is_reported_not_faulted(cuda):
    table = dev(torch.randn(10, 64), torch.float32)
    ids = torch.tensor([3, 77], dtype=torch.int32, device="cuda")
    out = torch.empty(2, 64, dtype=torch.float32, device="cuda")
    _lib.call("rb_embed_gather", cuda.ctx, P(table), _lib.F32, 10, 64, P(ids), 2, 1.0, P(out))
    with pytest.raises(_lib.RaiB200Error) as e:
        cuda.synchronize()
    assert e.value.code == -1
    cuda.synchronize()  # the status word was cleared; the context stays usable


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", [_lib.NORM_RMS, _lib.NORM_RMS_ONE_PLUS, _lib.NORM_LAYER])
@pytest.mark.parametrize("rows,hidden", [(1, 64), (7, 896), (33, 3584)])
def test_norm_matches_oracle(cuda, dtype, kind, rows, hidden):
    g = torch.Generator().manual_seed(2)
    x = dev(torch.randn(rows, hidden, generator=g), dtype)
    w = dev(1 + 0.1 * torch.randn(hidden, generator=g), dtype)
    b = dev(0.1 * torch.randn(hidden, generator=g), dtype)
    out = torch.empty_like(x)
    _lib.call("rb_norm", cuda.ctx, kind, P(x), None, None, 0, None, P(w), P(b) if kind == _lib.NORM_LAYER else None,
              1e-6, rows, hidden, P(out), None, DT[dtype])
    cuda.synchronize()
    xf, wf, bf = x.cpu().float(), w.cpu().float(), b.cpu().float()
    want = {_lib.NORM_RMS: lambda: rai_cpu.rms_norm(xf, wf, 1e-6),
            _lib.NORM_RMS_ONE_PLUS: lambda: rai_cpu.gemma_rms_norm(xf, wf, 1e-6),
            _lib.NORM_LAYER: lambda: rai_cpu.layer_norm(xf, wf, bf, 1e-6)}[kind]()
    assert float((out.cpu().float() - want).abs().max()) <= TOL[dtype] * float(want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_folds_residual_and_partials(cuda, dtype):
    """v = x + add + sum(acc) + acc_bias; sum_out = v; out = norm(v) — the residual adds of
    qwen2.rs:262,265 and the split-K reduction in one pass."""
    g = torch.Generator().manual_seed(3)
    rows, hidden, n_acc = 5, 256, 3
    x = dev(torch.randn(rows, hidden, generator=g), dtype)
    add = dev(torch.randn(rows, hidden, generator=g), dtype)
    acc = dev(torch.randn(n_acc, rows, hidden, generator=g), torch.float32)
    ab = dev(torch.randn(hidden, generator=g), dtype)
    w = dev(torch.randn(hidden, generator=g), dtype)
    out, s = torch.empty_like(x), torch.empty_like(x)
    _lib.call("rb_norm", cuda.ctx, _lib.NORM_RMS, P(x), P(add), P(acc), n_acc, P(ab), P(w), None, 1e-5, rows, hidden,
              P(out), P(s), DT[dtype])
    cuda.synchronize()
    v = (x.float() + add.float() + acc.sum(0) + ab.float()).cpu()
    assert float((s.cpu().float() - v).abs().max()) <= TOL[dtype] * float(v.abs().max())
    want = rai_cpu.rms_norm(s.cpu().float(), w.cpu().float(), 1e-5)  # normalises the stored (rounded) sum
    assert float((out.cpu().float() - want).abs().max()) <= TOL[dtype] * float(want.abs().max())
    # in place: sum_out aliases x, no norm output
    x2 = x.clone()
    _lib.call("rb_norm", cuda.ctx, _lib.NORM_RMS, P(x2), P(add), None, 0, None, None, None, 1e-5, rows, hidden, None,
              P(x2), DT[dtype])
    cuda.synchronize()
    assert torch.equal(x2, (x.float() + add.float()).to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [7, 640, 152064])
def test_argmax_rows_is_bit_exact_with_last_index_ties(cuda, dtype, cols):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(9, cols, generator=g)
    x[0, :] = 0.25                     # every element ties: the last index wins
    if cols > 5:
        x[1, 3] = x[1, cols - 2] = 50.0    # two equal maxima
    x[2, 0] = float("inf")
    x[3, :] = -1.0
    x[3, cols // 2] = -0.0             # -0.0 < +0.0 under total order but both beat -1
    xd = dev(x, dtype)
    out = torch.empty(9, dtype=torch.int32, device="cuda")
    _lib.call("rb_argmax_rows", cuda.ctx, P(xd), DT[dtype], 9, cols, P(out))
    cuda.synchronize()
    xr = xd.cpu().float()
    want = [rai_cpu.sample_argmax(xr[i]) for i in range(9)]
    assert out.cpu().tolist() == want
    assert want[0] == cols - 1


def test_rope_tables_match_oracle(cuda):
    for recipe, name, dim, theta in ((0, "qwen2", 128, 1e6), (1, "phi2", 32, 1e4), (2, "phi3", 96, 1e4)):
        n = 300
        cos = torch.empty(n, dim // 2, dtype=torch.float32, device="cuda")
        sin = torch.empty_like(cos)
        _lib.call("rb_rope_tables", cuda.ctx, recipe, dim, n, theta, P(cos), P(sin))
        cuda.synchronize()
        s_ref, c_ref = rai_cpu.rope_tables(dim, n, theta, name)
        assert float((cos.cpu() - c_ref[:, : dim // 2]).abs().max()) < 2e-5
        assert float((sin.cpu() - s_ref[:, : dim // 2]).abs().max()) < 2e-5


def test_pooled_stream_ordered_allocation(cuda):
    """rb_malloc_async / rb_free_async: no synchronisation, blocks reused in stream order, contents intact."""
    import ctypes
    import time
    import numpy as np
    from rai_b200 import _lib
    n = 1 << 20
    host = np.arange(n, dtype=np.float32)
    back = np.empty_like(host)
    seen = set()
    t0 = time.perf_counter()
    for i in range(200):
        p = ctypes.c_void_p()
        _lib.call("rb_malloc_async", cuda.ctx, n * 4, ctypes.byref(p))
        assert p.value and p.value % 256 == 0
        seen.add(p.value)
        if i % 50 == 0:
            _lib.call("rb_upload", cuda.ctx, p, host.ctypes.data_as(ctypes.c_void_p), n * 4)
            _lib.call("rb_download", cuda.ctx, back.ctypes.data_as(ctypes.c_void_p), p, n * 4)
            assert np.array_equal(back, host)
        _lib.call("rb_free_async", cuda.ctx, p)
    cuda.synchronize()
    assert len(seen) <= 4, "freed blocks should be reused by the next allocation on the stream"
    assert time.perf_counter() - t0 < 2.0
    empty = ctypes.c_void_p(1)
    _lib.call("rb_malloc_async", cuda.ctx, 0, ctypes.byref(empty))
    assert not empty.value
    _lib.call("rb_free_async", cuda.ctx, None)
