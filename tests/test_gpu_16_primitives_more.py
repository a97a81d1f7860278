"""The rest of the primitive set (rai-core/src/dispatch.rs:41-157) on `Cuda` through the Tensor mirror, against the
same operations of torch on the CPU: comparisons, sign / log2 / log10, log-softmax, arg-min, reductions over several
dims, gather along any dim, scatter-add / index-add, convolutions (1-D, 2-D, transposed), pooling, nearest upsampling."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from rai_b200 import _lib
from rai_b200.tensor import Tensor

pytestmark = pytest.mark.gpu


def T(a, cuda, dtype=_lib.F32):
    a = np.asarray(a)
    return Tensor.from_array(a, a.shape, cuda, dtype)


def close(got, want, tol=1e-5):
    want = want.numpy() if isinstance(want, torch.Tensor) else np.asarray(want)
    assert list(got.shape) == list(want.shape), (got.shape, want.shape)
    np.testing.assert_allclose(got, want, rtol=tol, atol=tol)


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def test_comparisons_give_u8_with_broadcast(cuda):
    a, b = rnd(3, 1, 5, seed=1), rnd(4, 5, seed=2)
    a[0, 0, 0] = b[0, 0]                      # an exact tie
    ta, tb = T(a.numpy(), cuda), T(b.numpy(), cuda)
    for name, ref in (("eq", torch.eq), ("ne", torch.ne), ("gt", torch.gt), ("ge", torch.ge), ("lt", torch.lt), ("le", torch.le)):
        got = getattr(ta, name)(tb)
        assert got.dtype == _lib.U8
        assert np.array_equal(got.as_vec().astype(np.uint8), ref(a, b).to(torch.uint8).numpy()), name
    assert np.array_equal(ta.gt(0.0).as_vec().astype(bool), (a > 0).numpy())


def test_sign_logs_abs_minimum(cuda):
    x = rnd(7, 9, seed=3)
    x[0, 0] = 0.0
    t = T(x.numpy(), cuda)
    close(t.sign().as_vec(), torch.sign(x))
    close(t.abs().as_vec(), x.abs())
    pos = x.abs() + 0.1
    tp = T(pos.numpy(), cuda)
    close(tp.log().as_vec(), pos.log())
    close(tp.log2().as_vec(), pos.log2())
    close(tp.log10().as_vec(), pos.log10(), 2e-5)
    close(t.minimum(T(rnd(9, seed=4).numpy(), cuda)).as_vec(), torch.minimum(x, rnd(9, seed=4)))


@pytest.mark.parametrize("dim", [-1, 0, 1])
def test_log_softmax_and_argmin_over_any_dim(cuda, dim):
    x = rnd(5, 6, 7, seed=5)
    t = T(x.numpy(), cuda)
    close(t.log_softmax(dim).as_vec(), F.log_softmax(x, dim), 2e-5)
    assert np.array_equal(t.argmin(dim).as_vec().astype(np.int64), x.argmin(dim).numpy())


def test_argmin_takes_the_first_of_equal_minima(cuda):
    x = torch.tensor([[3.0, -1.0, 5.0, -1.0, 2.0], [0.0, 0.0, 0.0, 0.0, 0.0]])
    assert T(x.numpy(), cuda).argmin(-1).as_vec().tolist() == [1, 0]


@pytest.mark.parametrize("dims,keep", [((0, 2), False), ((1,), True), ((0, 1, 2), False), ((-1, 0), True)])
def test_reductions_over_several_dims(cuda, dims, keep):
    x = rnd(4, 5, 6, seed=6)
    t = T(x.numpy(), cuda)
    close(t.sum(dims, keep).as_vec(), x.sum(dim=dims, keepdim=keep), 2e-5)
    close(t.max(dims, keep).as_vec(), x.amax(dim=dims, keepdim=keep))
    close(t.min(dims, keep).as_vec(), x.amin(dim=dims, keepdim=keep))


def test_gather_along_any_dim(cuda):
    x = rnd(4, 5, 6, seed=7)
    for dim in (0, 1, 2):
        shape = list(x.shape)
        shape[dim] = 3
        idx = torch.randint(0, x.shape[dim], shape, generator=torch.Generator().manual_seed(dim))
        got = T(x.numpy(), cuda).gather(dim, T(idx.numpy().astype(np.int32), cuda, _lib.U32))
        close(got.as_vec(), x.gather(dim, idx))


@pytest.mark.parametrize("dim", [0, 1, 2])
def test_scatter_add_and_index_add(cuda, dim):
    x = rnd(4, 5, 6, seed=8)
    src_shape = list(x.shape)
    src_shape[dim] = 7
    src = rnd(*src_shape, seed=9)
    idx = torch.randint(0, x.shape[dim], src_shape, generator=torch.Generator().manual_seed(10))      # duplicates on purpose
    got = T(x.numpy(), cuda).scatter_add(dim, T(idx.numpy().astype(np.int32), cuda, _lib.U32), T(src.numpy(), cuda))
    close(got.as_vec(), x.scatter_add(dim, idx, src), 1e-5)
    idx1 = torch.randint(0, x.shape[dim], (7,), generator=torch.Generator().manual_seed(11))
    got = T(x.numpy(), cuda).index_add(dim, T(idx1.numpy().astype(np.int32), cuda, _lib.U32), T(src.numpy(), cuda))
    close(got.as_vec(), x.index_add(dim, idx1, src), 1e-5)


@pytest.mark.parametrize("pad,stride,dil", [((0, 0), (1, 1), (1, 1)), ((1, 2), (2, 1), (1, 1)), ((2, 2), (1, 2), (2, 1))])
def test_conv2d_and_conv1d(cuda, pad, stride, dil):
    x, w = rnd(2, 3, 9, 11, seed=12), rnd(4, 3, 3, 2, seed=13)
    got = T(x.numpy(), cuda).conv2d(T(w.numpy(), cuda), pad, stride, dil)
    close(got.as_vec(), F.conv2d(x, w, None, stride, pad, dil), 2e-5)
    x1, w1 = rnd(2, 3, 17, seed=14), rnd(5, 3, 4, seed=15)
    got = T(x1.numpy(), cuda).conv1d(T(w1.numpy(), cuda), pad[1], stride[1], dil[1])
    close(got.as_vec(), F.conv1d(x1, w1, None, stride[1], pad[1], dil[1]), 2e-5)


@pytest.mark.parametrize("pad,opad,stride,dil", [((0, 0), (0, 0), (1, 1), (1, 1)), ((1, 0), (1, 0), (2, 1), (1, 1)),
                                                 ((1, 1), (0, 1), (2, 3), (1, 2))])
def test_conv_transpose2d_and_1d(cuda, pad, opad, stride, dil):
    x, w = rnd(2, 3, 5, 6, seed=16), rnd(3, 4, 3, 2, seed=17)
    got = T(x.numpy(), cuda).conv_transpose2d(T(w.numpy(), cuda), pad, opad, stride, dil)
    close(got.as_vec(), F.conv_transpose2d(x, w, None, stride, pad, opad, 1, dil), 2e-5)
    x1, w1 = rnd(2, 3, 7, seed=18), rnd(3, 2, 3, seed=19)
    got = T(x1.numpy(), cuda).conv_transpose1d(T(w1.numpy(), cuda), pad[1], opad[1], stride[1], dil[1])
    close(got.as_vec(), F.conv_transpose1d(x1, w1, None, stride[1], pad[1], opad[1], 1, dil[1]), 2e-5)


def test_pooling_and_upsampling(cuda):
    x = rnd(2, 3, 8, 10, seed=20)
    t = T(x.numpy(), cuda)
    close(t.max_pool2d((2, 3), (2, 2), (1, 1)).as_vec(), F.max_pool2d(x, (2, 3), (2, 2), (1, 1)))
    close(t.max_pool2d((3, 3), (1, 2), (0, 0), (2, 1)).as_vec(), F.max_pool2d(x, (3, 3), (1, 2), 0, (2, 1)))
    close(t.avg_pool2d((2, 2)).as_vec(), F.avg_pool2d(x, (2, 2)))
    close(t.avg_pool2d((3, 2), (1, 2)).as_vec(), F.avg_pool2d(x, (3, 2), (1, 2)))
    x1 = rnd(2, 3, 12, seed=21)
    t1 = T(x1.numpy(), cuda)
    close(t1.max_pool1d(3, 2).as_vec(), F.max_pool1d(x1, 3, 2))
    close(t1.avg_pool1d(4).as_vec(), F.avg_pool1d(x1, 4))
    close(t.upsample_nearest2d((16, 25)).as_vec(), F.interpolate(x, size=(16, 25), mode="nearest"))
    close(t1.upsample_nearest1d(30).as_vec(), F.interpolate(x1, size=30, mode="nearest"))


def test_bf16_storage_goes_through_the_same_kernels(cuda):
    x, w = rnd(1, 2, 6, 6, seed=22), rnd(3, 2, 3, 3, seed=23)
    xb, wb = x.to(torch.bfloat16).float(), w.to(torch.bfloat16).float()
    got = T(xb.numpy(), cuda, _lib.BF16).conv2d(T(wb.numpy(), cuda, _lib.BF16), (1, 1), (1, 1), (1, 1))
    close(got.as_vec(), F.conv2d(xb, wb, None, 1, 1), 2e-2)
    assert np.array_equal(T(xb.numpy(), cuda, _lib.BF16).gt(0.0).as_vec().astype(bool), (xb > 0).numpy())
