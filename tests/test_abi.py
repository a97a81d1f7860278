"""The C-ABI library loads and exports exactly what include/rai_b200.h declares (no GPU needed)."""
import ctypes
import subprocess

import pytest

from rai_b200 import _lib, build, configs, synth


@pytest.fixture(scope="module")
def library():
    build.build()
    return _lib.lib()


def test_header_parses_every_prototype():
    protos = _lib.parse_header()
    text = _lib.HEADER.read_text()
    declared = set()
    import re
    for m in re.finditer(r"\b(rb_[a-z0-9_]+)\s*\(", re.sub(r"/\*.*?\*/", "", text, flags=re.S)):
        declared.add(m.group(1))
    assert declared == set(protos), declared ^ set(protos)
    assert len(protos) >= 50


def test_library_exports_every_declared_symbol(library):
    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], capture_output=True, text=True, check=True)
    exported = {line.split()[-1] for line in out.stdout.splitlines() if " T " in line}
    missing = set(_lib.parse_header()) - exported
    assert not missing, f"declared in the header but not exported: {sorted(missing)}"
    extra = {s for s in exported if s.startswith("rb_")} - set(_lib.parse_header())
    assert not extra, f"exported but not declared: {sorted(extra)}"


def test_every_prototype_cites_the_reference():
    """Each declaration is preceded by a comment naming the reference file it stands in for."""
    text = _lib.HEADER.read_text()
    assert text.count(".rs:") >= 40


def test_model_config_struct_matches_header():
    import re
    text = _lib.HEADER.read_text()
    body = re.search(r"typedef struct rb_model_config \{(.*?)\} rb_model_config;", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = [ln.split()[-1].rstrip(";") for ln in body.splitlines() if ln.strip().endswith(";")]
    assert fields == [f[0] for f in _lib.ModelConfig._fields_]


def test_no_cpu_fallback_without_gpu(library):
    """On a machine without a GPU the context cannot be created and the error says why."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    ctx = ctypes.c_void_p()
    status = library.rb_init(0, ctypes.byref(ctx))
    assert status == -5
    assert b"no CPU path" in library.rb_last_error()
    with pytest.raises(_lib.RaiB200Error):
        _lib.call("rb_init", 0, ctypes.byref(ctx))


def test_null_arguments_are_rejected_not_dereferenced(library):
    assert library.rb_init(0, None) == -1
    assert library.rb_sync(None) == -1
    assert library.rb_linear(None, None, None, None, None, None, 1, 1, 8, 0, _lib.BF16) == -1
    assert library.rb_model_forward(None, None, 1, 1, 0, None) == -1
    assert library.rb_kv_cache_reset(None) == -1
    assert b"null" in library.rb_last_error()


def test_param_names_follow_the_derive_rule():
    names = [n for n, _, _ in synth.param_shapes(configs.get("tiny-qwen2"))]
    assert names[0] == "model.embed_tokens.weight"
    assert "model.layers.1.self_attn.q_proj.bias" in names
    assert "model.layers.0.post_attention_layernorm.weight" in names
    assert names[-1] == "lm_head.weight"
    phi2 = [n for n, _, _ in synth.param_shapes(configs.get("tiny-phi2"))]
    assert "model.layers.0.self_attn.dense.bias" in phi2 and "model.final_layernorm.bias" in phi2
    assert "lm_head.bias" in phi2
    phi3 = [n for n, _, _ in synth.param_shapes(configs.get("tiny-phi3"))]
    assert "model.layers.0.self_attn.qkv_proj.weight" in phi3 and "model.layers.1.mlp.gate_up_proj.weight" in phi3
    gemma = [n for n, _, _ in synth.param_shapes(configs.get("tiny-gemma"))]
    assert "lm_head.weight" not in gemma  # shares model.embed_tokens.weight (gemma.rs:330)


def test_baseline_config_sizes():
    """Parameter counts of the five benchmark configurations (bf16 bytes streamed per decode step)."""
    def count(name):
        return sum(int(__import__("numpy").prod(s)) for _, s, _ in synth.param_shapes(configs.get(name)))
    assert abs(count("qwen2-7b") * 2 / 1e9 - 15.23) < 0.05      # 14.14 GB streamed + 1.09 GB embedding table
    assert abs(count("qwen2-0.5b") * 2 / 1e9 - 0.988) < 0.01
    assert abs(count("gemma-2b") * 2 / 1e9 - 5.012) < 0.02


def test_rust_shim_declares_every_export():
    """integration/b200.rs carries an `extern "C"` block generated from the header: it must be exactly what the
    generator emits now (so it lists every entry point with the header's own types) and every library call the shim
    makes must be one of them."""
    import importlib.util
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("gen_ffi", os.path.join(root, "integration", "gen_ffi.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    src = open(os.path.join(root, "integration", "b200.rs")).read()
    block = src[src.index("// <ffi>\n") + len("// <ffi>\n"):src.index("// </ffi>")]
    assert block == gen.emit(), "run `python integration/gen_ffi.py --write`"
    declared = set(re.findall(r"pub fn (rb_\w+)\(", block))
    assert declared == set(_lib.parse_header())
    used = set(re.findall(r"\b(rb_[a-z0-9_]+)\(", src[src.index("// </ffi>"):]))
    assert used <= declared, used - declared
