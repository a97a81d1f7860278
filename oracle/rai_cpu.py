"""CPU oracle: an op-for-op PyTorch-CPU float32 restatement of the decoder forward pass of
cksac/rai (qwen2, phi2, phi3, gemma), with the KV cache grown by concatenation as the
reference does.

THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA path is compared against and
the timed CPU baseline; nothing in the product package imports it.

PARITY UNPINNED: the reference holds no golden vectors, known-answer tests or recorded logits
for this path (its ops/layer tests print without asserting), and the reference itself cannot be
built in this environment (no Rust toolchain).  The arithmetic of the reference lives in the
third-party crate candle-core ("0.6", not vendored, no lockfile); this file restates rai's own
graph (which is in the tree) with IEEE float32 torch ops, one torch op per rai primitive, in the
reference's order.  The restatement is cross-checked by self-consistency properties in
tests/ (cached decode == full recompute, GQA == explicit repeat_kv, shape algebra against the
asserts of rai-core/tests/shape.rs).

Deliberate deviations from the reference text, each needed by the benchmark configurations:
  * qwen2 builds k_proj/v_proj as hidden->hidden with num_kv_groups = 1
    (rai-models/src/llm/qwen2.rs:138-139,150), which only works for MHA checkpoints.  The GQA
    form of gemma/phi3 (gemma.rs:167-172,191-201; phi3.rs:136,152-161) is used instead.
  * RoPE tables are built in float32 whatever the model dtype (the reference builds them in the
    model dtype, qwen2.rs:45-59).
  * tie_word_embeddings is honoured for qwen2 by loading one matrix under both names.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

F32 = torch.float32


# --------------------------------------------------------------------------------------
# rai-core primitives / hlops that have a recipe of their own
# --------------------------------------------------------------------------------------

def rsqrt(x: torch.Tensor) -> torch.Tensor:
    """rai-core/src/backend/candle.rs:545-553 — Rsqrt is sqrt() followed by recip()."""
    return x.sqrt().reciprocal()


def softmax_last(x: torch.Tensor) -> torch.Tensor:
    """rai-core/src/backend/candle.rs:792-803 — max_keepdim, broadcast_sub, exp, sum_keepdim,
    broadcast_div, all in the tensor's dtype."""
    m = x.max(dim=-1, keepdim=True).values
    e = (x - m).exp()
    return e / e.sum(dim=-1, keepdim=True)


def silu(x: torch.Tensor) -> torch.Tensor:
    """rai-core/src/hlops/activations.rs:30-32 — x / (exp(-x) + 1)."""
    return x / (x.neg().exp() + 1.0)


def gelu(x: torch.Tensor) -> torch.Tensor:
    """rai-core/src/hlops/activations.rs:20-22 — x * 0.5 * (1 + erf(x / sqrt(2)))."""
    return x * 0.5 * (1.0 + (x / math.sqrt(2.0)).erf())


def new_gelu(x: torch.Tensor) -> torch.Tensor:
    """rai-core/src/hlops/activations.rs:25-27 — tanh form."""
    c = torch.tensor(math.sqrt(2.0 / math.pi), dtype=F32).item()
    return 0.5 * x * (1.0 + (c * (x + 0.044715 * x.pow(3.0))).tanh())


def relu(x: torch.Tensor) -> torch.Tensor:
    """rai-core/src/hlops/activations.rs:5-7."""
    return torch.maximum(x, torch.zeros_like(x))


ACTIVATIONS = {
    # names follow the serde names of rai-nn/src/activations.rs:5-17
    "gelu": gelu,
    "gelu_new": new_gelu,
    "newgelu": new_gelu,
    "relu": relu,
    "silu": silu,
}


def mean_last(x: torch.Tensor) -> torch.Tensor:
    """rai-core/src/hlops/mean.rs:4-7 — sum / count."""
    return x.sum(dim=-1, keepdim=True) / float(x.shape[-1])


def var_last(x: torch.Tensor) -> torch.Tensor:
    """rai-core/src/hlops/var.rs:33-38 — population variance (ddof 0), mean recomputed."""
    m = mean_last(x)
    s = (x - m).square().sum(dim=-1, keepdim=True)
    return s / float(x.shape[-1])


# --------------------------------------------------------------------------------------
# rai-nn modules
# --------------------------------------------------------------------------------------

def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    """rai-nn/src/linear.rs:59-69 — y = x . W^T (+ b), W is [out, in], broadcast over batch."""
    y = x.matmul(w.t())
    return y + b if b is not None else y


def embedding(weight: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """rai-nn/src/embedding.rs:25-30 — flatten, index_select(0), reshape."""
    out_dims = list(ids.shape) + [weight.shape[-1]]
    return weight.index_select(0, ids.flatten().long()).reshape(out_dims)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """rai-nn/src/rms_norm.rs:18-22 — w * x * rsqrt(sum((x / sqrt(H))^2) + eps)."""
    s = 1.0 / math.sqrt(x.shape[-1])
    n = rsqrt((x * s).square().sum(dim=-1, keepdim=True) + eps)
    return w * x * n


def gemma_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """rai-models/src/llm/gemma.rs:42-54 — f32 internally, x / sqrt(mean(x^2) + eps), * (w + 1)."""
    h = x.shape[-1]
    xf = x.to(F32)
    norm_x = xf.square().sum(dim=-1, keepdim=True) / float(h)
    x_normed = xf / (norm_x + eps).sqrt()
    return x_normed.to(x.dtype) * (w + 1.0)


def layer_norm(x: torch.Tensor, w: Optional[torch.Tensor], b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """rai-nn/src/layer_norm.rs:32-42."""
    mean = mean_last(x)
    var = var_last(x)
    x = (x - mean) * rsqrt(var + eps)
    if w is not None:
        return w * x + b
    return x


# --------------------------------------------------------------------------------------
# shared pieces of the four decoders
# --------------------------------------------------------------------------------------

def rope_tables(dim: int, max_pos: int, theta: float, recipe: str):
    """sin/cos tables [max_pos, dim] (the two halves repeat).

    recipe "qwen2" (also gemma): inv_freq = 1f32 / (theta^(i/dim) in f64, cast to f32)
        qwen2.rs:45-59, gemma.rs:76-90
    recipe "phi2": theta is f32 and powf runs in f32     phi2.rs:48-63
    recipe "phi3": f64 throughout, cast to the table dtype phi3.rs:45-60
    """
    idx = list(range(0, dim, 2))
    if recipe == "qwen2":
        inv = [float(torch.tensor(1.0, dtype=F32) / torch.tensor(theta ** (i / dim), dtype=F32)) for i in idx]
    elif recipe == "phi2":
        th = torch.tensor(theta, dtype=F32)
        inv = [float(torch.tensor(1.0, dtype=F32) / th.pow(torch.tensor(i, dtype=F32) / torch.tensor(dim, dtype=F32)))
               for i in idx]
    elif recipe == "phi3":
        inv = [1.0 / (theta ** (i / dim)) for i in idx]
    else:
        raise ValueError(recipe)
    inv_freq = torch.tensor(inv, dtype=torch.float64).to(F32).reshape(1, -1)
    t = torch.arange(0, max_pos, dtype=torch.int64).to(F32).reshape(max_pos, 1)
    freqs = t.matmul(inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.sin(), emb.cos()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """qwen2.rs:33-38 / gemma.rs:64-69."""
    last = x.shape[-1]
    x1 = x.narrow(-1, 0, last // 2)
    x2 = x.narrow(-1, last // 2, last - last // 2)
    return torch.cat([x2.neg(), x1], dim=-1)


def rope_full(q, k, sin, cos, offset):
    """qwen2.rs:62-71 / gemma.rs:93-102 — whole head rotated."""
    s = q.shape[2]
    c = cos.narrow(0, offset, s).unsqueeze(0).unsqueeze(0)
    sn = sin.narrow(0, offset, s).unsqueeze(0).unsqueeze(0)
    return q * c + rotate_half(q) * sn, k * c + rotate_half(k) * sn


def rope_partial(x, sin, cos, dim, offset):
    """phi2.rs:66-77 / phi3.rs:63-74 — first `dim` lanes rotated, the rest passed through."""
    s, hd = x.shape[2], x.shape[3]
    x_rot = x.narrow(3, 0, dim)
    x_pass = x.narrow(3, dim, hd - dim)
    x1, x2 = x_rot.chunk(2, dim=-1)
    c = cos.narrow(0, offset, s)
    sn = sin.narrow(0, offset, s)
    rh = torch.cat([x2.neg(), x1], dim=-1)
    x_rot = x_rot * c + rh * sn
    return torch.cat([x_rot, x_pass], dim=-1)


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """gemma.rs:191-201 / phi3.rs:152-161 / phi2.rs:190-200."""
    if n_rep == 1:
        return x
    b, nkv, t, d = x.shape
    return x.unsqueeze(2).expand(b, nkv, n_rep, t, d).reshape(b, nkv * n_rep, t, d)


def additive_causal_mask(b: int, tgt: int, offset: int, window: Optional[int] = None) -> torch.Tensor:
    """qwen2.rs:306-336 (with the sliding-window term) / phi3.rs:286-306 / gemma.rs:341-362."""
    i = torch.arange(tgt).reshape(tgt, 1)
    j = torch.arange(tgt).reshape(1, tgt)
    masked = i < j
    if window is not None:
        masked = masked | ((j + window) < i)
    mask = torch.where(masked, torch.tensor(float("-inf")), torch.tensor(0.0)).to(F32)
    if offset > 0:
        mask = torch.cat([torch.zeros(tgt, offset, dtype=F32), mask], dim=-1)
    return mask.expand(b, 1, tgt, tgt + offset)


@dataclass
class Config:
    """Union of the four reference Config structs (qwen2.rs:8-24, phi2.rs:9-24, phi3.rs:9-24,
    gemma.rs:12-27); `arch` selects the decoder."""
    arch: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    max_position_embeddings: int
    rope_theta: float
    norm_eps: float
    hidden_act: str
    tie_word_embeddings: bool = False
    partial_rotary_factor: float = 1.0
    sliding_window: int = 1 << 30
    attention_bias: bool = False

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


class _Decoder:
    def __init__(self, cfg: Config, params: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.p = {k: v.to(F32) for k, v in params.items()}
        self.kv: List[Optional[tuple]] = [None] * cfg.num_hidden_layers

    def clear_kv_cache(self):
        self.kv = [None] * self.cfg.num_hidden_layers

    def _w(self, name):
        return self.p[name + ".weight"]

    def _b(self, name):
        return self.p.get(name + ".bias")

    def _lin(self, name, x):
        return linear(x, self._w(name), self._b(name))

    def _cache(self, layer, k, v):
        prev = self.kv[layer]
        if prev is not None:
            k = torch.cat([prev[0], k], dim=2)
            v = torch.cat([prev[1], v], dim=2)
        self.kv[layer] = (k, v)
        return k, v

    def _split_heads(self, x, n):
        b, s, _ = x.shape
        return x.reshape(b, s, n, self.cfg.head_dim).transpose(1, 2)


class Qwen2(_Decoder):
    """rai-models/src/llm/qwen2.rs (GQA form, see module docstring)."""

    def __init__(self, cfg, params):
        super().__init__(cfg, params)
        self.sin, self.cos = rope_tables(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_theta, "qwen2")
        self.act = ACTIVATIONS[cfg.hidden_act]

    def _attn(self, i, xs, mask, offset):  # qwen2.rs:170-221
        cfg, pre = self.cfg, f"model.layers.{i}.self_attn."
        b, s, _ = xs.shape
        q = self._split_heads(self._lin(pre + "q_proj", xs), cfg.num_attention_heads)
        k = self._split_heads(self._lin(pre + "k_proj", xs), cfg.num_key_value_heads)
        v = self._split_heads(self._lin(pre + "v_proj", xs), cfg.num_key_value_heads)
        q, k = rope_full(q, k, self.sin, self.cos, offset)
        k, v = self._cache(i, k, v)
        n_rep = cfg.num_attention_heads // cfg.num_key_value_heads
        k, v = repeat_kv(k, n_rep), repeat_kv(v, n_rep)
        scale = 1.0 / math.sqrt(cfg.head_dim)
        w = q.matmul(k.transpose(2, 3)) * scale
        if mask is not None:
            w = w + mask
        w = softmax_last(w)
        o = w.matmul(v)
        o = o.transpose(1, 2).reshape(b, s, cfg.num_attention_heads * cfg.head_dim)
        return self._lin(pre + "o_proj", o)

    def _mlp(self, i, xs):  # qwen2.rs:100-104
        pre = f"model.layers.{i}.mlp."
        lhs = self.act(self._lin(pre + "gate_proj", xs))
        rhs = self._lin(pre + "up_proj", xs)
        return self._lin(pre + "down_proj", lhs * rhs)

    def _norm(self, name, x):
        return rms_norm(x, self._w(name), self.cfg.norm_eps)

    def _embed(self, ids):
        return embedding(self._w("model.embed_tokens"), ids)

    def _mask(self, b, s, offset):
        return additive_causal_mask(b, s, offset, self.cfg.sliding_window)

    def _head(self, xs):
        return linear(xs, self._w("lm_head"), None)

    def forward(self, ids: torch.Tensor, offset: int) -> torch.Tensor:  # qwen2.rs:338-359
        b, s = ids.shape
        mask = None if s <= 1 else self._mask(b, s, offset)
        xs = self._embed(ids)
        for i in range(self.cfg.num_hidden_layers):  # qwen2.rs:253-266
            pre = f"model.layers.{i}."
            residual = xs
            h = self._norm(pre + "input_layernorm", xs)
            h = self._attn(i, h, mask, offset)
            xs = h + residual
            residual = xs
            h = self._mlp(i, self._norm(pre + "post_attention_layernorm", xs))
            xs = residual + h
        xs = xs.narrow(1, s - 1, 1)
        return self._head(self._norm("model.norm", xs))


class Gemma(Qwen2):
    """rai-models/src/llm/gemma.rs — own RmsNorm (1 + w), embeddings * sqrt(H), tied lm_head."""

    def _norm(self, name, x):
        return gemma_rms_norm(x, self._w(name), self.cfg.norm_eps)

    def _embed(self, ids):  # gemma.rs:378-379
        return embedding(self._w("model.embed_tokens"), ids) * math.sqrt(self.cfg.hidden_size)

    def _mask(self, b, s, offset):
        return additive_causal_mask(b, s, offset, None)

    def _head(self, xs):  # gemma.rs:330
        return linear(xs, self._w("model.embed_tokens"), None)


class Phi3(_Decoder):
    """rai-models/src/llm/phi3.rs — fused qkv_proj and gate_up_proj."""

    def __init__(self, cfg, params):
        super().__init__(cfg, params)
        self.sin, self.cos = rope_tables(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_theta, "phi3")
        self.act = ACTIVATIONS[cfg.hidden_act]

    def _attn(self, i, xs, mask, offset):  # phi3.rs:163-211
        cfg, pre = self.cfg, f"model.layers.{i}.self_attn."
        b, s, _ = xs.shape
        nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        qkv = self._lin(pre + "qkv_proj", xs)
        q = self._split_heads(qkv.narrow(-1, 0, nq * d), nq)
        k = self._split_heads(qkv.narrow(-1, nq * d, nkv * d), nkv)
        v = self._split_heads(qkv.narrow(-1, nq * d + nkv * d, nkv * d), nkv)
        q = rope_partial(q, self.sin, self.cos, d, offset)
        k = rope_partial(k, self.sin, self.cos, d, offset)
        k, v = self._cache(i, k, v)
        k, v = repeat_kv(k, nq // nkv), repeat_kv(v, nq // nkv)
        scale = float(torch.tensor(1.0, dtype=F32) / torch.tensor(float(d), dtype=F32).sqrt())
        w = q.matmul(k.transpose(2, 3)) * scale
        if mask is not None:
            w = w + mask
        o = softmax_last(w).matmul(v)
        return self._lin(pre + "o_proj", o.transpose(1, 2).flatten(2))

    def _mlp(self, i, xs):  # phi3.rs:101-107
        pre, isz = f"model.layers.{i}.mlp.", self.cfg.intermediate_size
        up = self._lin(pre + "gate_up_proj", xs)
        gate = up.narrow(-1, 0, isz)
        up = up.narrow(-1, isz, isz)
        return self._lin(pre + "down_proj", up * self.act(gate))

    def forward(self, ids, offset):  # phi3.rs:308-323
        b, s = ids.shape
        mask = None if s <= 1 else additive_causal_mask(b, s, offset, None)
        xs = embedding(self._w("model.embed_tokens"), ids)
        eps = self.cfg.norm_eps
        for i in range(self.cfg.num_hidden_layers):  # phi3.rs:243-251
            pre = f"model.layers.{i}."
            residual = xs
            h = self._attn(i, rms_norm(xs, self._w(pre + "input_layernorm"), eps), mask, offset)
            xs = h + residual
            residual = xs
            h = self._mlp(i, rms_norm(xs, self._w(pre + "post_attention_layernorm"), eps))
            xs = residual + h
        xs = xs.narrow(1, s - 1, 1)
        return linear(rms_norm(xs, self._w("model.norm"), eps), self._w("lm_head"), None)


class Phi2(_Decoder):
    """rai-models/src/llm/phi2.rs — parallel attention + MLP under one LayerNorm, partial rotary,
    f32 scores with the scale folded into K^T, u8 mask + where."""

    def __init__(self, cfg, params):
        super().__init__(cfg, params)
        self.rot = int(cfg.partial_rotary_factor * cfg.head_dim)
        self.sin, self.cos = rope_tables(self.rot, cfg.max_position_embeddings, cfg.rope_theta, "phi2")
        self.act = ACTIVATIONS[cfg.hidden_act]

    def _attn(self, i, xs, mask):  # phi2.rs:202-264
        cfg, pre = self.cfg, f"model.layers.{i}.self_attn."
        b, s, _ = xs.shape
        nq, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
        q = self._split_heads(self._lin(pre + "q_proj", xs), nq)
        k = self._split_heads(self._lin(pre + "k_proj", xs), nkv)
        v = self._split_heads(self._lin(pre + "v_proj", xs), nkv)
        offset = 0 if self.kv[i] is None else self.kv[i][0].shape[2]
        q = rope_partial(q, self.sin, self.cos, self.rot, offset)
        k = rope_partial(k, self.sin, self.cos, self.rot, offset)
        k, v = self._cache(i, k, v)
        k, v = repeat_kv(k, nq // nkv), repeat_kv(v, nq // nkv)
        scale = 1.0 / math.sqrt(cfg.head_dim)
        w = q.to(F32).matmul(k.to(F32).transpose(-1, -2) * scale)
        if mask is not None:
            w = torch.where(mask.expand(b, nq, s, s), torch.tensor(float("-inf")), w)
        w = softmax_last(w).to(v.dtype)
        o = w.matmul(v).transpose(1, 2)
        return self._lin(pre + "dense", o.reshape(b, s, -1))

    def _mlp(self, i, xs):  # phi2.rs:99-101
        pre = f"model.layers.{i}.mlp."
        return self._lin(pre + "fc2", self.act(self._lin(pre + "fc1", xs)))

    def forward(self, ids, offset=None):  # phi2.rs:334-347 (offset comes from the cache length)
        b, s = ids.shape
        xs = embedding(self._w("model.embed_tokens"), ids)
        mask = None
        if s > 1:  # phi2.rs:104-109
            mask = (torch.arange(s).reshape(1, s) > torch.arange(s).reshape(s, 1))
        eps = self.cfg.norm_eps
        for i in range(self.cfg.num_hidden_layers):  # phi2.rs:293-299
            pre = f"model.layers.{i}."
            residual = xs
            h = layer_norm(xs, self._w(pre + "input_layernorm"), self._b(pre + "input_layernorm"), eps)
            xs = self._attn(i, h, mask) + self._mlp(i, h) + residual
        xs = layer_norm(xs, self._w("model.final_layernorm"), self._b("model.final_layernorm"), eps)
        xs = xs.narrow(1, s - 1, 1)
        return self._lin("lm_head", xs).squeeze(1)


ARCHS = {"qwen2": Qwen2, "gemma": Gemma, "phi3": Phi3, "phi2": Phi2}


def build(cfg: Config, params: Dict[str, torch.Tensor]):
    return ARCHS[cfg.arch](cfg, params)


# --------------------------------------------------------------------------------------
# generation loop of the examples (examples/qwen2/src/main.rs:32-53,74-99)
# --------------------------------------------------------------------------------------

def total_order_keys(values) -> "np.ndarray":
    """f32::total_cmp as an unsigned key: flip all bits of negatives, set the sign bit of the rest, so
    that -NaN < -inf < ... < -0.0 < +0.0 < ... < +inf < +NaN compares as plain integers."""
    import numpy as np
    u = np.ascontiguousarray(np.asarray(values, dtype=np.float32)).view(np.uint32)
    return np.where(u & np.uint32(0x80000000), ~u, u | np.uint32(0x80000000))


def sample_argmax(logits: torch.Tensor) -> int:
    """examples/qwen2/src/main.rs:32-40 — `max_by(total_cmp)`: the maximum under the IEEE total order,
    and the LAST index among equal maxima (Iterator::max_by returns the last of equal elements)."""
    import numpy as np
    k = total_order_keys(logits.reshape(-1).float().numpy())
    return int(np.nonzero(k == k.max())[0].max())


def apply_repeat_penalty(logits: torch.Tensor, penalty: float, context) -> torch.Tensor:
    """examples/qwen2/src/main.rs:42-53: every token id present in `context` (a set, so once each) has
    its float32 logit divided by the float32 penalty when >= 0 and multiplied by it otherwise."""
    import numpy as np
    out = logits.float().clone().numpy()
    p = np.float32(penalty)
    for t in set(int(c) for c in context):
        out[t] = np.float32(out[t]) / p if out[t] >= 0 else np.float32(out[t]) * p
    return torch.from_numpy(out)


def generate_with_penalty(model, prompt: torch.Tensor, steps: int, penalty: float, last_n: int, eos: int = -1,
                          collect_logits: bool = False):
    """The generation loop of examples/qwen2/src/main.rs:74-99 for each row of a batch: logits to float32,
    repeat penalty over the last `last_n` tokens of (prompt + generated) when penalty >= 1, argmax, stop at
    `eos`.  A finished row keeps emitting `eos` so that the batch stays rectangular (the example handles one
    sequence and leaves the loop).  Returns [B, steps] tokens (and the raw per-step logits when asked)."""
    model.clear_kv_cache()
    b, s = prompt.shape
    tokens = [[int(t) for t in prompt[i]] for i in range(b)]
    finished = [False] * b
    out, all_logits = [], []
    ids, pos = prompt, 0
    for _ in range(steps):
        logits = model.forward(ids, pos).reshape(b, -1).float()
        pos += ids.shape[1]
        nxt = []
        for i in range(b):
            row = logits[i]
            if penalty >= 1.0:
                row = apply_repeat_penalty(row, penalty, tokens[i][max(0, len(tokens[i]) - last_n):])
            t = eos if finished[i] else sample_argmax(row)
            finished[i] = finished[i] or t == eos
            tokens[i].append(t)
            nxt.append(t)
        out.append(torch.tensor(nxt, dtype=torch.int64))
        if collect_logits:
            all_logits.append(logits.clone())
        ids = out[-1].reshape(b, 1)
    res = torch.stack(out, dim=1)
    return (res, torch.stack(all_logits)) if collect_logits else res


def greedy_generate(model, prompt: torch.Tensor, steps: int, collect_logits: bool = False):
    """Prefill once, then one token per step, argmax on the host (no repeat penalty, which is what
    the benchmark configurations call "greedy").  prompt is [B, S] int64; returns [B, steps] tokens
    (and the per-step logits [steps, B, V] when asked)."""
    model.clear_kv_cache()
    b, s = prompt.shape
    toks, all_logits = [], []
    ids, pos = prompt, 0
    for _ in range(steps):
        logits = model.forward(ids, pos).reshape(b, -1)
        pos += ids.shape[1]
        nxt = torch.tensor([sample_argmax(logits[i]) for i in range(b)], dtype=torch.int64)
        toks.append(nxt)
        if collect_logits:
            all_logits.append(logits.clone())
        ids = nxt.reshape(b, 1)
    out = torch.stack(toks, dim=1)
    return (out, torch.stack(all_logits)) if collect_logits else out
