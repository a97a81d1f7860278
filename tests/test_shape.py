"""Known answers of the reference's own shape tests (rai-core/tests/shape.rs:3-64, read as text: the
reference cannot be built here) for the index helpers, plus the broadcasting, matmul and reduction shape
rules of rai-core/src/shape.rs:88-173 on the shapes the decoders use."""
import pytest

from rai_b200 import shape as S


def test_dim_known_answers():                      # tests/shape.rs:4-13
    s = [0, 1, 2, 3, 4, 5]
    assert S.dim(s, 0) == 0 and S.dim(s, 1) == 1 and S.dim(s, 2) == 2
    assert S.dim(s, -2) == len(s) - 2 and S.dim(s, -1) == len(s) - 1


def test_dims_known_answers():                     # tests/shape.rs:17-58
    s = [0, 1, 2, 3, 4, 5]
    assert S.dims(s, 0, 0) == []
    assert S.dims(s, 0, 1) == [0]
    assert S.dims(s, 2, 4) == [2, 3]
    assert S.dims(s, 4, 2) == [4, 3]
    assert S.dims(s, 4, 0) == [4, 3, 2, 1]
    assert S.dims(s, 0, 0, True) == [0]
    assert S.dims(s, 0, 1, True) == [0, 1]
    assert S.dims(s, 2, 4, True) == [2, 3, 4]
    assert S.dims(s, 4, 2, True) == [4, 3, 2]
    assert S.dims(s, 4, 0, True) == [4, 3, 2, 1, 0]
    assert S.dims(s, None, 0) == []
    assert S.dims(s, None, 1) == [0]
    assert S.dims(s, None, 2) == [0, 1]
    assert S.dims(s, None, 0, True) == [0]
    assert S.dims(s, None, 1, True) == [0, 1]
    assert S.dims(s, None, 2, True) == [0, 1, 2]
    assert S.dims(s, 0) == [0, 1, 2, 3, 4, 5]
    assert S.dims(s, 1) == [1, 2, 3, 4, 5]
    assert S.dims(s, 2) == [2, 3, 4, 5]
    assert S.dims(s) == [0, 1, 2, 3, 4, 5]
    assert S.dims(s, -1) == [5]
    assert S.dims(s, -2) == [4, 5]
    assert S.dims(s, -5) == [1, 2, 3, 4, 5]
    assert S.dims(s, -1, 0) == [5, 4, 3, 2, 1]
    assert S.dims(s, -4, -1) == [2, 3, 4]
    assert S.dims(s, -1, 0, True) == [5, 4, 3, 2, 1, 0]
    assert S.dims(s, -4, -1, True) == [2, 3, 4, 5]


def test_size_known_answer():                      # tests/shape.rs:61-64
    assert S.size([1, 2, 3, 4, 5, 6], -1) == 6


def test_broadcast_rules():
    assert S.broadcast_to([2, 1, 5], [3, 1]) == ([2, 3, 5], True, True)
    assert S.broadcast_to([4, 8], [4, 8]) == ([4, 8], False, False)
    assert S.broadcast_to([8], [2, 4, 8]) == ([2, 4, 8], True, False)
    assert S.broadcast_to([2, 14, 128, 128], [2, 1, 128, 128]) == ([2, 14, 128, 128], False, True)   # scores + mask
    with pytest.raises(ValueError):
        S.broadcast_to([2, 3], [4, 3])


def test_matmul_and_reduce_rules():
    assert S.broadcast_matmul([5, 7], [7, 3]) == ([5, 3], [5, 7], [7, 3], False, False)
    # Linear::fwd: x [B, S, in] against the weight broadcast to [B, in, out] (linear.rs:59-69)
    assert S.broadcast_matmul([2, 9, 16], [2, 16, 4])[0] == [2, 9, 4]
    out, l, r, lb, rb = S.broadcast_matmul([2, 14, 9, 64], [1, 1, 64, 9])
    assert out == [2, 14, 9, 9] and l == [2, 14, 9, 64] and r == [2, 14, 64, 9] and (lb, rb) == (False, True)
    with pytest.raises(ValueError):
        S.broadcast_matmul([2, 3], [4, 5])
    assert S.reduce([2, 9, 16], [2], True) == [2, 9, 1]          # the norms' mean over the last dimension
    assert S.reduce([2, 9, 16], [2], False) == [2, 9]
    assert S.reduce([2, 9, 16], [0, 2], False) == [9]
