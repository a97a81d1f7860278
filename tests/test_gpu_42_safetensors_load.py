"""rb_model_load_safetensors (Module::update_by_safetensors, rai-core/src/nn.rs:39-55) on the GPU: a model
loaded from files must be the same model as one given the same tensors by name — identical logits, bit for
bit — for every stored float type, for several files, and for a tensor-parallel rank's shard."""
import os

import numpy as np
import pytest
import torch

from rai_b200 import _lib, configs, synth
from rai_b200.models import Model
from rai_b200.safetensors_io import write_safetensors

pytestmark = pytest.mark.gpu


def _logits(m, cfg, batch=2, prompt=9):
    ids = synth.prompt(cfg, batch, prompt, 3)
    a = m.forward(ids, 0).float().cpu()
    b = m.forward(ids[:, :1], prompt).float().cpu()
    return torch.cat([a.reshape(batch, -1), b.reshape(batch, -1)])


def _by_name(cuda, cfg, dtype, w, **kw):
    m = Model(cfg, dtype, cuda, 2, 64, 32, **kw)
    m.update_params(w)
    out = _logits(m, cfg)
    m.close()
    return out


def _from_files(cuda, cfg, dtype, files, **kw):
    m = Model(cfg, dtype, cuda, 2, 64, 32, **kw)
    m.update_by_safetensors(files)
    out = _logits(m, cfg)
    m.close()
    return out


@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-qwen2-tied", "tiny-phi2", "tiny-phi3", "tiny-gemma"])
@pytest.mark.parametrize("dtype", [_lib.BF16, _lib.F32])
def test_float32_file_gives_the_same_model(cuda, tmp_path, name, dtype):
    cfg = configs.get(name)
    w = synth.weights(cfg, 11)
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, w, "F32", metadata={"format": "pt"})
    assert torch.equal(_from_files(cuda, cfg, dtype, [p]), _by_name(cuda, cfg, dtype, w))


@pytest.mark.parametrize("stored,np_dtype", [("BF16", None), ("F16", np.float16), ("F64", np.float64)])
def test_other_stored_types_are_cast_like_the_reference(cuda, tmp_path, stored, np_dtype):
    """update_by_name casts the stored tensor to the model dtype (nn.rs:197-199): storing as T then loading
    equals loading the T-rounded values."""
    cfg = configs.get("tiny-qwen2")
    w = synth.weights(cfg, 12)
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, w, stored)
    if stored == "BF16":
        rounded = {k: torch.from_numpy(v).to(torch.bfloat16).float().numpy() for k, v in w.items()}
    else:
        rounded = {k: v.astype(np_dtype).astype(np.float32) for k, v in w.items()}
    for dtype in (_lib.BF16, _lib.F32):
        assert torch.equal(_from_files(cuda, cfg, dtype, [p]), _by_name(cuda, cfg, dtype, rounded))


def test_several_files_extra_names_and_override(cuda, tmp_path):
    cfg = configs.get("tiny-qwen2")
    w = synth.weights(cfg, 13)
    names = list(w)
    first = {k: w[k] for k in names[: len(names) // 2]}
    second = {k: w[k] for k in names[len(names) // 2:]}
    victim = names[0]
    first[victim] = np.full_like(w[victim], 9.0)                 # overridden by the later file
    second[victim] = w[victim]
    second["optimizer.step"] = np.zeros((3,), np.float32)        # not a parameter of the model: ignored
    a, b = str(tmp_path / "a.safetensors"), str(tmp_path / "b.safetensors")
    write_safetensors(a, first, "F32")
    write_safetensors(b, second, "BF16")
    want = {k: (torch.from_numpy(v).to(torch.bfloat16).float().numpy() if k in second else v) for k, v in w.items()}
    assert torch.equal(_from_files(cuda, cfg, _lib.F32, [a, b]), _by_name(cuda, cfg, _lib.F32, want))


def test_tensor_larger_than_one_staging_chunk(cuda, tmp_path):
    cfg = configs.get("tiny-qwen2")
    cfg["vocab_size"] = 40000                                    # embedding 40000 x 256 float32 = 41 MB: two chunks
    w = synth.weights(cfg, 14)
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, w, "F32")
    assert torch.equal(_from_files(cuda, cfg, _lib.BF16, [p]), _by_name(cuda, cfg, _lib.BF16, w))


def test_missing_and_misshapen_parameters_fail_by_name(cuda, tmp_path):
    cfg = configs.get("tiny-qwen2")
    w = synth.weights(cfg, 15)
    gone = "model.layers.1.mlp.down_proj.weight"
    p = str(tmp_path / "missing.safetensors")
    write_safetensors(p, {k: v for k, v in w.items() if k != gone}, "F32")
    m = Model(cfg, _lib.BF16, cuda, 2, 64, 32)
    with pytest.raises(_lib.RaiB200Error, match=gone.replace(".", r"\.")):
        m.update_by_safetensors([p])
    bad = dict(w)
    bad[gone] = w[gone][:, :-1]
    q = str(tmp_path / "shape.safetensors")
    write_safetensors(q, bad, "F32")
    with pytest.raises(_lib.RaiB200Error, match="expected"):
        m.update_by_safetensors([q])
    with pytest.raises(_lib.RaiB200Error, match="cannot open"):
        m.update_by_safetensors([str(tmp_path / "nope.safetensors")])
    m.close()


@pytest.mark.parametrize("name,tp,rank", [("tiny-qwen2", 2, 1), ("tiny-qwen2-28h", 8, 5), ("tiny-phi2", 2, 0)])
def test_tensor_parallel_rank_keeps_the_same_shard(cuda, tmp_path, name, tp, rank):
    """One rank's shard, read back parameter by parameter: the shard built from the files, where only the rows the
    rank keeps are uploaded, must equal the shard built from whole tensors, and both must be the rectangle the shard
    plan names (zeros elsewhere).  A forward pass of a rank without its group is refused, not attempted."""
    from rai_b200 import tp as tp_plan
    cfg = configs.get(name)
    w = synth.weights(cfg, 16)
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, w, "BF16")
    rounded = {k: torch.from_numpy(v).to(torch.bfloat16).float().numpy() for k, v in w.items()}
    a = Model(cfg, _lib.BF16, cuda, 2, 64, 32, tp_rank=rank, tp_size=tp)
    a.update_by_safetensors([p])
    b = Model(cfg, _lib.BF16, cuda, 2, 64, 32, tp_rank=rank, tp_size=tp)
    b.update_params(rounded)
    kept_any = False
    for n in a.param_names():
        ta, tb = a.read_param(n), b.read_param(n)
        assert torch.equal(ta, tb), n
        full = torch.from_numpy(rounded[n]).to(torch.bfloat16)
        nz = ta != 0
        assert torch.equal(ta[nz], full[nz]), n      # what the rank keeps is the checkpoint's values
        kept_any = kept_any or bool(nz.any())
    assert kept_any
    if cfg["arch"] != "phi2":
        plan = tp_plan.plan(cfg, rank, tp)
        got = a.read_param("model.layers.0.mlp.gate_proj.weight")
        want = torch.zeros_like(got)
        want[plan.inter] = torch.from_numpy(rounded["model.layers.0.mlp.gate_proj.weight"]).to(torch.bfloat16)[plan.inter]
        assert torch.equal(got, want)
    with pytest.raises(_lib.RaiB200Error, match="rb_model_tp_init"):
        a.forward(synth.prompt(cfg, 2, 4, 3), 0)
    a.close()
    b.close()


def test_parameters_round_trip_through_to_safetensors(cuda, tmp_path):
    """Module::to_safetensors then update_by_safetensors gives the same model (rai-core/src/nn.rs:31-55)."""
    cfg = configs.get("tiny-qwen2")
    w = synth.weights(cfg, 23)
    m = Model(cfg, _lib.BF16, cuda, 2, 64, 32)
    m.update_params(w)
    first = _logits(m, cfg)
    path = str(tmp_path / "saved.safetensors")
    m.to_safetensors(path)
    m.close()
    again = _from_files(cuda, cfg, _lib.BF16, [path])
    assert torch.equal(first, again)
