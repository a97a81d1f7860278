"""ctypes front of oracle/rai_ref.c, the plain-C restatement of the decoder forward pass.  TEST INFRASTRUCTURE,
like the rest of this directory; parity unpinned (see the header of rai_ref.c)."""
import ctypes
from typing import Dict, Optional

import numpy as np

import build_ref

_ARCH = {"qwen2": 0, "phi2": 1, "phi3": 2, "gemma": 3}
_ACT = {"silu": 1, "gelu_new": 2, "gelu_pytorch_tanh": 2, "gelu": 2}


class _Config(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("arch", "vocab", "hidden", "inter", "layers", "q_heads", "kv_heads", "head_dim",
                                              "rot", "act", "max_pos")] + [("theta", ctypes.c_double), ("eps", ctypes.c_double)]


_LAYER_FIELDS = ("ln1_w", "ln1_b", "ln2_w", "q_w", "q_b", "k_w", "k_b", "v_w", "v_b", "o_w", "o_b", "gate_w", "up_w", "up_b",
                 "down_w", "down_b")


class _Layer(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in _LAYER_FIELDS]


def _lib():
    lib = ctypes.CDLL(str(build_ref.build()))
    lib.ref_create.restype = ctypes.c_void_p
    lib.ref_create.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int32]
    lib.ref_destroy.argtypes = [ctypes.c_void_p]
    lib.ref_clear_kv_cache.argtypes = [ctypes.c_void_p]
    lib.ref_forward.restype = ctypes.c_int32
    lib.ref_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    return lib


class RefModel:
    """cfg: a configuration dict (rai_b200.configs); weights: checkpoint name -> float32 numpy array."""

    def __init__(self, cfg: dict, weights: Dict[str, np.ndarray], batch_cap: int = 8):
        self._lib = _lib()
        self.cfg = cfg
        a = cfg["arch"]
        nq = cfg["num_attention_heads"]
        nkv = cfg.get("num_key_value_heads") or nq
        d = cfg.get("head_dim") or cfg["hidden_size"] // nq
        rot = int(cfg.get("partial_rotary_factor", 1.0) * d) if a == "phi2" else d
        eps = cfg["layer_norm_eps"] if a == "phi2" else cfg["rms_norm_eps"]
        self._keep = []  # arrays the C side points into

        def arr(x) -> Optional[int]:
            if x is None:
                return None
            x = np.ascontiguousarray(x, dtype=np.float32)
            self._keep.append(x)
            return x.ctypes.data

        def get(name):
            return weights.get(name)

        layers = (_Layer * cfg["num_hidden_layers"])()
        isz = cfg["intermediate_size"]
        for i in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{i}."
            f = dict.fromkeys(_LAYER_FIELDS)
            f["ln1_w"], f["ln1_b"] = get(p + "input_layernorm.weight"), get(p + "input_layernorm.bias")
            f["ln2_w"] = get(p + "post_attention_layernorm.weight")
            if a == "phi3":  # narrow() on the fused projections' outputs == row ranges of their weights (phi3.rs:172-176,103-105)
                qkv = weights[p + "self_attn.qkv_proj.weight"]
                f["q_w"], f["k_w"], f["v_w"] = qkv[: nq * d], qkv[nq * d:(nq + nkv) * d], qkv[(nq + nkv) * d:]
                gu = weights[p + "mlp.gate_up_proj.weight"]
                f["gate_w"], f["up_w"] = gu[:isz], gu[isz:]
                f["o_w"], f["down_w"] = get(p + "self_attn.o_proj.weight"), get(p + "mlp.down_proj.weight")
            else:
                for h in "qkv":
                    f[h + "_w"], f[h + "_b"] = get(p + f"self_attn.{h}_proj.weight"), get(p + f"self_attn.{h}_proj.bias")
                if a == "phi2":
                    f["o_w"], f["o_b"] = get(p + "self_attn.dense.weight"), get(p + "self_attn.dense.bias")
                    f["up_w"], f["up_b"] = get(p + "mlp.fc1.weight"), get(p + "mlp.fc1.bias")
                    f["down_w"], f["down_b"] = get(p + "mlp.fc2.weight"), get(p + "mlp.fc2.bias")
                else:
                    f["o_w"] = get(p + "self_attn.o_proj.weight")
                    f["gate_w"], f["up_w"] = get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")
                    f["down_w"] = get(p + "mlp.down_proj.weight")
            for k, v in f.items():
                setattr(layers[i], k, arr(v))
        fn = "model.final_layernorm" if a == "phi2" else "model.norm"
        tied = a == "gemma" or bool(cfg.get("tie_word_embeddings", False))
        head = weights["model.embed_tokens.weight"] if tied else weights["lm_head.weight"]
        c = _Config(_ARCH[a], cfg["vocab_size"], cfg["hidden_size"], isz, cfg["num_hidden_layers"], nq, nkv, d, rot,
                    _ACT[cfg["hidden_act"]], cfg["max_position_embeddings"], float(cfg["rope_theta"]), float(eps))
        self._layers = layers
        self._m = self._lib.ref_create(ctypes.byref(c), arr(weights["model.embed_tokens.weight"]), arr(get(fn + ".weight")),
                                       arr(get(fn + ".bias")), arr(head), arr(get("lm_head.bias")), layers, batch_cap)

    def clear_kv_cache(self):
        self._lib.ref_clear_kv_cache(self._m)

    def forward(self, ids: np.ndarray, offset: int) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        b, s = ids.shape
        out = np.empty((b, self.cfg["vocab_size"]), dtype=np.float32)
        st = self._lib.ref_forward(self._m, ids.ctypes.data, b, s, int(offset), out.ctypes.data)
        if st != 0:
            raise ValueError("ref_forward: bad arguments (batch, position or token id out of range)")
        return out

    def close(self):
        if self._m:
            self._lib.ref_destroy(self._m)
            self._m = None

    def __del__(self):
        self.close()
