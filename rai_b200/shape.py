"""The shape algebra of rai-core/src/shape.rs that the decoder graphs rely on: dimension indexing with
negative indices and (possibly reversed) ranges, broadcasting, batched-matmul and reduction shapes."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple


def dim(shape: Sequence[int], i: int) -> int:
    """Shape::dim (shape.rs:33-35): the index of a dimension, negative values counted from the end."""
    rank = len(shape)
    j = i + rank if i < 0 else i
    if not 0 <= j < rank:
        raise IndexError(f"dimension {i} out of range for rank {rank}")
    return j


def size(shape: Sequence[int], i: int) -> int:
    """Shape::size (shape.rs:13-15)."""
    return int(shape[dim(shape, i)])


def dims(shape: Sequence[int], start: Optional[int] = None, stop: Optional[int] = None, inclusive: bool = False) -> List[int]:
    """Shape::dims over a range (shape.rs:43-45): `start..stop` (or `start..=stop`); open ends default to the first
    dimension and to one past the last; a range whose start lies after its end walks backwards."""
    rank = len(shape)

    def resolve(v: int) -> int:
        return v + rank if v < 0 else v

    a = 0 if start is None else resolve(start)
    if stop is None:
        return list(range(a, rank))
    b = resolve(stop)
    if a <= b:
        return list(range(a, b + 1 if inclusive else b))
    return list(range(a, b - 1 if inclusive else b, -1))


def broadcast_to(lhs: Sequence[int], rhs: Sequence[int]) -> Tuple[List[int], bool, bool]:
    """Shape::shape_broadcast_to (shape.rs:88-127): the common shape and which side had to be broadcast."""
    l, r = list(lhs), list(rhs)
    lb = rb = False
    if len(l) < len(r):
        l, lb = [1] * (len(r) - len(l)) + l, True
    elif len(l) > len(r):
        r, rb = [1] * (len(l) - len(r)) + r, True
    out = []
    for a, b in zip(l, r):
        if a == b:
            out.append(a)
        elif a == 1:
            out.append(b)
            lb = True
        elif b == 1:
            out.append(a)
            rb = True
        else:
            raise ValueError(f"incompatible shapes {list(lhs)} and {list(rhs)}")
    return out, lb, rb


def broadcast_matmul(lhs: Sequence[int], rhs: Sequence[int]):
    """Shape::shape_broadcast_matmul (shape.rs:129-160): (out, lhs as batched, rhs as batched, lhs broadcast?, rhs broadcast?)."""
    l, r = list(lhs), list(rhs)
    if len(l) < 2 or len(r) < 2 or l[-1] != r[-2]:
        raise ValueError(f"incompatible shapes {l} and {r}")
    m, k, n = l[-2], l[-1], r[-1]
    if len(l) == 2 and len(r) == 2:
        return [m, n], l, r, False, False
    batching, lb, rb = broadcast_to(l[:-2], r[:-2])
    return batching + [m, n], batching + [m, k], batching + [k, n], lb, rb


def reduce(shape: Sequence[int], which: Sequence[int], keep_dim: bool) -> List[int]:
    """Shape::shape_reduce (shape.rs:162-173)."""
    out = []
    for i in range(len(shape)):
        if i not in which:
            out.append(int(shape[i]))
        elif keep_dim:
            out.append(1)
    return out
