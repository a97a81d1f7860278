"""ctypes binding of librai_b200.so.

The prototypes are read from include/rai_b200.h, so the binding cannot drift from the header:
every function the header declares is bound, with argument and return types taken from the
declaration.  There is no CPU implementation behind this module: if the shared library is missing
or no B200 is present, calls fail with an exception that says so.
"""
from __future__ import annotations

import ctypes
import re
from pathlib import Path
from typing import Dict, List, Tuple

PKG = Path(__file__).resolve().parent
HEADER = PKG.parent / "include" / "rai_b200.h"
# RAI_B200_DEBUG_AIDS=1 selects the developer build (python -m rai_b200.build --debug-aids), a file of its own
LIB_PATH = PKG / ("librai_b200_dbg.so" if __import__("os").environ.get("RAI_B200_DEBUG_AIDS") == "1" else "librai_b200.so")

# status codes / tags of the header, mirrored for Python callers
RB_OK = 0
U8, U32, I64, F16, BF16, F32, F64 = range(7)
ACT_NONE, ACT_SILU, ACT_GELU_TANH, ACT_GELU_ERF, ACT_RELU = range(5)
NORM_RMS, NORM_RMS_ONE_PLUS, NORM_LAYER = range(3)
ARCH_QWEN2, ARCH_PHI2, ARCH_PHI3, ARCH_GEMMA = range(4)
(UN_NEG, UN_EXP, UN_SQRT, UN_RSQRT, UN_SQUARE, UN_TANH, UN_ERF, UN_SIN, UN_COS, UN_POWF, UN_SILU, UN_GELU_TANH,
 UN_GELU_ERF, UN_RELU, UN_LOG, UN_ABS, UN_RECIP, UN_ADD_SCALAR, UN_MUL_SCALAR, UN_SIGN, UN_LOG2, UN_LOG10) = range(22)
CMP_EQ, CMP_NE, CMP_GT, CMP_GE, CMP_LT, CMP_LE = range(6)
BIN_ADD, BIN_SUB, BIN_MUL, BIN_DIV, BIN_MAXIMUM, BIN_MINIMUM = range(6)
RED_SUM, RED_MAX, RED_MIN = range(3)

ERROR_NAMES = {-1: "invalid argument", -2: "incompatible shape", -3: "unsupported dtype", -4: "out of device memory",
               -5: "CUDA error", -6: "device-side wait gave up", -7: "unimplemented", -8: "parameter not found"}


class RaiB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"rai_b200 error {code} ({ERROR_NAMES.get(code, '?')}): {message}")
        self.code = code


class ModelConfig(ctypes.Structure):
    """struct rb_model_config of include/rai_b200.h."""
    _fields_ = [(n, ctypes.c_int32) for n in (
        "arch", "dtype", "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
        "num_attention_heads", "num_key_value_heads", "max_position_embeddings", "rotary_dim", "hidden_act",
        "tie_word_embeddings", "max_batch", "max_seq", "max_tokens", "tp_rank", "tp_size", "sliding_window", "reserved0")] + [
        ("rope_theta", ctypes.c_double), ("norm_eps", ctypes.c_double)]


_SCALARS = {"int32_t": ctypes.c_int32, "int64_t": ctypes.c_int64, "size_t": ctypes.c_size_t, "float": ctypes.c_float,
            "double": ctypes.c_double, "uint32_t": ctypes.c_uint32, "uint8_t": ctypes.c_uint8}


def _ctype_of(decl: str):
    decl = decl.strip()
    if "*" in decl:
        return ctypes.c_char_p if decl.count("*") == 1 and re.match(r"^const\s+char\s*\*", decl) else ctypes.c_void_p
    base = decl.split()[0] if not decl.startswith("const") else decl.split()[1]
    return _SCALARS[base]


def parse_header(path: Path = HEADER) -> Dict[str, Tuple[object, List[object]]]:
    """name -> (restype, argtypes) for every function the header declares."""
    text = re.sub(r"/\*.*?\*/", "", path.read_text(), flags=re.S)
    out = {}
    for m in re.finditer(r"^([A-Za-z_][\w\s\*]*?)\b(rb_\w+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.M | re.S):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        if ret.startswith("typedef"):
            continue
        restype = None if ret == "void" else _ctype_of(ret if "*" in ret else ret + " x")
        argtypes = [] if args in ("", "void") else [_ctype_of(a) for a in args.split(",")]
        out[name] = (restype, argtypes)
    return out


_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library with prototypes attached.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RaiB200Error(-7, f"{LIB_PATH} is missing: build it with `python -m rai_b200.build` "
                                   "(there is no CPU fallback)")
        cdll = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in parse_header().items():
            fn = getattr(cdll, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = cdll
    return _lib


def check(status: int) -> None:
    if status != RB_OK:
        raise RaiB200Error(status, lib().rb_last_error().decode("utf-8", "replace"))


def call(name: str, *args):
    """Calls an int32-status entry point and raises RaiB200Error on failure."""
    check(getattr(lib(), name)(*args))
