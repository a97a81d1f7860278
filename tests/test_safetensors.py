"""The .safetensors reader under rb_model_load_safetensors (Module::update_by_safetensors,
rai-core/src/nn.rs:39-55): listing and bytes of well-formed files, files written by the `safetensors`
package itself, and the malformed headers safetensors::SafeTensors::deserialize rejects."""
import json
import struct

import numpy as np
import pytest

from rai_b200 import _lib
from rai_b200.safetensors_io import SafetensorsFile, bf16_bytes, write_safetensors


def _raw(path, header, data=b"", pad=0):
    js = (header if isinstance(header, bytes) else json.dumps(header).encode()) + b" " * pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)) + js + data)


def test_lists_entries_in_file_order_with_their_bytes(tmp_path):
    g = np.random.default_rng(0)
    t = {"model.b": g.standard_normal((3, 5)).astype(np.float32), "model.a": g.standard_normal((7,)).astype(np.float32),
         "empty": np.zeros((0, 4), np.float32), "scalar": np.float32(2.5).reshape(())}
    p = tmp_path / "w.safetensors"
    write_safetensors(str(p), t, "F32", metadata={"format": "pt", "note": 'quote " and \\ and é'})
    with SafetensorsFile(str(p)) as f:
        assert [e[0] for e in f.entries] == ["model.b", "model.a", "empty", "scalar"]
        assert f.entries[0][1:] == ("F32", (3, 5), 60) and f.entries[2][1:] == ("F32", (0, 4), 0) and f.entries[3][2] == ()
        for name, a in t.items():
            assert f.read_bytes(name) == np.ascontiguousarray(a).tobytes()


@pytest.mark.parametrize("dtype", ["F64", "F16", "BF16"])
def test_other_float_types(tmp_path, dtype):
    a = np.random.default_rng(1).standard_normal((4, 6)).astype(np.float32)
    p = tmp_path / "w.safetensors"
    write_safetensors(str(p), {"x": a}, dtype)
    with SafetensorsFile(str(p)) as f:
        assert f.entries == [("x", dtype, (4, 6), 24 * {"F64": 8, "F16": 2, "BF16": 2}[dtype])]
        want = bf16_bytes(a) if dtype == "BF16" else a.astype({"F64": np.float64, "F16": np.float16}[dtype]).tobytes()
        assert f.read_bytes("x") == want


def test_reads_what_the_safetensors_package_writes(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    import torch
    t = {"w.bf16": torch.randn(5, 8).to(torch.bfloat16), "w.f32": torch.randn(2, 3), "w.f16": torch.randn(9).half(),
         "ids": torch.arange(6, dtype=torch.int64).reshape(2, 3), "i32": torch.arange(4, dtype=torch.int32)}
    p = tmp_path / "pkg.safetensors"
    st.save_file(t, str(p), metadata={"who": "package"})
    with SafetensorsFile(str(p)) as f:
        got = {e[0]: e for e in f.entries}
        assert set(got) == set(t)
        assert got["w.bf16"][1:3] == ("BF16", (5, 8)) and got["ids"][1:3] == ("I64", (2, 3))
        assert got["i32"][1] is None and got["i32"][3] == 16           # a type without a tag is listed, not rejected
        for name, v in t.items():
            assert f.read_bytes(name) == v.contiguous().view(torch.uint8).numpy().tobytes()


def test_unicode_names_and_escapes(tmp_path):
    p = tmp_path / "u.safetensors"
    _raw(str(p), b'{"caf\\u00e9 \\ud83d\\ude00\\n": {"dtype":"U8","shape":[2],"data_offsets":[0,2]}, "__metadata__": {"a": "b"}}', b"\x01\x02")
    with SafetensorsFile(str(p)) as f:
        assert f.entries[0][0] == "café \U0001F600\n" and f.read_bytes(f.entries[0][0]) == b"\x01\x02"


@pytest.mark.parametrize("case", ["short", "header_longer_than_file", "huge_header", "not_json", "offsets_outside", "size_mismatch",
                                  "begin_after_end", "missing_shape", "unknown_dtype", "trailing", "nine_dims", "float_offset"])
def test_malformed_files_are_rejected_with_a_message(tmp_path, case):
    p = str(tmp_path / "bad.safetensors")
    ok = {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}
    data = b"\0" * 16
    if case == "short":
        open(p, "wb").write(b"\x01\x02\x03")
    elif case == "header_longer_than_file":
        open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    elif case == "huge_header":
        open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    elif case == "not_json":
        _raw(p, b'{"x": [1, 2', data)
    elif case == "offsets_outside":
        _raw(p, {"x": dict(ok, data_offsets=[8, 24])}, data)
    elif case == "size_mismatch":
        _raw(p, {"x": dict(ok, shape=[2, 3])}, data)
    elif case == "begin_after_end":
        _raw(p, {"x": dict(ok, shape=[0], data_offsets=[8, 4])}, data)
    elif case == "missing_shape":
        _raw(p, {"x": {"dtype": "F32", "data_offsets": [0, 16]}}, data)
    elif case == "unknown_dtype":
        _raw(p, {"x": dict(ok, dtype="F33")}, data)
    elif case == "trailing":
        _raw(p, json.dumps({"x": ok}).encode() + b" {}", data)
    elif case == "nine_dims":
        _raw(p, {"x": dict(ok, shape=[1] * 9, data_offsets=[0, 4])}, data)
    elif case == "float_offset":
        _raw(p, b'{"x": {"dtype":"F32","shape":[2,2],"data_offsets":[0,16.0]}}', data)
    with pytest.raises(_lib.RaiB200Error) as e:
        SafetensorsFile(p)
    assert "safetensors" in str(e.value)


def test_missing_file(tmp_path):
    with pytest.raises(_lib.RaiB200Error, match="cannot open"):
        SafetensorsFile(str(tmp_path / "nope.safetensors"))
