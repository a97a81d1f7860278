"""rai-nn modules over `rai_b200.tensor.Tensor`: Linear, Embedding, RmsNorm, LayerNorm, Activation, each
`fwd` written as the reference composes it from primitives (rai-nn/src/{linear,embedding,rms_norm,
layer_norm,activations}.rs).  These are the unfused forms; the decoder driver runs the fused kernels."""
from __future__ import annotations

import math
from typing import Optional

from .tensor import Tensor


class Linear:
    """rai-nn/src/linear.rs:8-69: y = x . W^T (+ b), W is [out, in]."""

    def __init__(self, weight: Tensor, bias: Optional[Tensor] = None):
        self.weight, self.bias = weight, bias

    def fwd(self, x: Tensor) -> Tensor:
        # broadcast_left over the batch dims, then .t() (linear.rs:60-64)
        w = self.weight.broadcast_to(list(x.shape[:-2]) + list(self.weight.shape)).t() if len(x.shape) > 2 else self.weight.t()
        y = x.matmul(w)
        return y + self.bias if self.bias is not None else y

    forward = fwd


class Embedding:
    """rai-nn/src/embedding.rs:6-30: flatten the ids, index_select(0), reshape."""

    def __init__(self, weight: Tensor):
        self.weight = weight

    def fwd(self, ids: Tensor) -> Tensor:
        out_dims = list(ids.shape) + [self.weight.size(-1)]
        return self.weight.index_select(0, ids.flatten()).reshape(out_dims)

    forward = fwd


class RmsNorm:
    """rai-nn/src/rms_norm.rs:6-22."""

    def __init__(self, weight: Tensor, eps: float):
        self.weight, self.eps = weight, eps

    def fwd(self, x: Tensor) -> Tensor:
        s = 1.0 / math.sqrt(x.size(-1))
        n = ((x * s).square().sum(-1, True) + self.eps).rsqrt()
        return self.weight * x * n

    forward = fwd


class LayerNorm:
    """rai-nn/src/layer_norm.rs:6-42 (population variance, hlops/var.rs:33-38)."""

    def __init__(self, weight: Optional[Tensor], bias: Optional[Tensor], eps: float):
        self.weight, self.bias, self.eps = weight, bias, eps

    def fwd(self, x: Tensor) -> Tensor:
        mean = x.mean(-1, True)
        var = x.var(-1, True)
        y = (x - mean) * (var + self.eps).rsqrt()
        return self.weight * y + self.bias if self.weight is not None else y

    forward = fwd


class Activation:
    """rai-nn/src/activations.rs:5-30; names are the serde names."""
    _FNS = {"gelu": Tensor.gelu, "gelu_new": Tensor.new_gelu, "newgelu": Tensor.new_gelu, "relu": Tensor.relu,
            "silu": Tensor.silu}

    def __init__(self, name: str):
        self.name = name

    def fwd(self, x: Tensor) -> Tensor:
        return self._FNS[self.name](x)

    forward = fwd
