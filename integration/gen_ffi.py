"""Emits the Rust `extern "C"` declarations of every entry point of include/rai_b200.h, the block that
integration/b200.rs carries between its `// <ffi>` and `// </ffi>` markers.

    python integration/gen_ffi.py            # print the block
    python integration/gen_ffi.py --write    # rewrite the block inside integration/b200.rs

The mapping is mechanical (int32_t -> i32, const void* -> *const c_void, rb_ctx** -> *mut *mut rb_ctx, ...), so the
binding cannot drift from the header; tests/test_abi.py checks that the committed block is what this script emits.
"""
from __future__ import annotations

import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "rai_b200.h"
SHIM = Path(__file__).resolve().parent / "b200.rs"

SCALARS = {"int32_t": "i32", "int64_t": "i64", "uint32_t": "u32", "uint8_t": "u8", "uint64_t": "u64", "size_t": "usize", "float": "f32",
           "double": "f64", "char": "c_char", "void": "c_void"}
OPAQUE = ("rb_ctx", "rb_kv_cache", "rb_model", "rb_safetensors", "rb_model_config")


def rust_type(decl: str) -> str:
    """C parameter or return type (without the parameter name) -> Rust."""
    decl = decl.strip()
    stars = decl.count("*")
    core = decl.replace("*", " ").split()
    const = "const" in core
    base = [t for t in core if t != "const"][0]
    ty = SCALARS.get(base, base if base in OPAQUE else None)
    if ty is None:
        raise ValueError(f"unknown C type in {decl!r}")
    if stars == 0:
        return ty
    # `const T*` is *const T; `const T* const*` and `T**` add a level; out-parameters are *mut
    out = ty
    for level in range(stars):
        innermost = level == 0
        out = ("*const " if (const and innermost) else "*mut ") + out
    if decl.replace(" ", "").endswith("*const*"):      # const char* const* paths
        out = "*const *const " + ty
    return out


def split_param(p: str):
    p = p.strip()
    m = re.match(r"^(.*?)(\b[A-Za-z_]\w*)$", p)
    if not m or m.group(1).strip() == "":
        return p, "_"
    return m.group(1).strip(), m.group(2)


def prototypes():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    for m in re.finditer(r"^([A-Za-z_][\w\s\*]*?)\b(rb_\w+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.M | re.S):
        ret, name, args = m.group(1).strip(), m.group(2), " ".join(m.group(3).split())
        if ret.startswith("typedef"):
            continue
        params = [] if args in ("", "void") else [split_param(a) for a in args.split(",")]
        yield ret, name, params


def emit() -> str:
    lines = ["extern \"C\" {"]
    for ret, name, params in prototypes():
        ps = ", ".join(f"{('r#' + n) if n in ('type', 'in', 'fn', 'ref', 'mod') else n}: {rust_type(t)}" for t, n in params)
        r = "" if ret == "void" else f" -> {rust_type(ret)}"
        lines.append(f"    pub fn {name}({ps}){r};")
    lines.append("}")
    return "\n".join(lines) + "\n"


def main():
    block = emit()
    if "--write" in sys.argv:
        src = SHIM.read_text()
        a, b = src.index("// <ffi>\n") + len("// <ffi>\n"), src.index("// </ffi>")
        SHIM.write_text(src[:a] + block + src[b:])
    else:
        sys.stdout.write(block)


if __name__ == "__main__":
    main()
