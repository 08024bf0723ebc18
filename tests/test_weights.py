"""Weights: the container, loading by name, the one collected error, random folders (no GPU)."""
import json
import os
import struct

import pytest
import torch

from helpers import CONFIGS, config_dict
from rocmforge_b200.config import Qwen2Config, architecture_for
from rocmforge_b200.weights import (ModelFiles, ParamSpec, SafetensorsError, WeightError, check_folder,
                                    load_folder, target_dtype, write_model_folder, write_safetensors)


def spec_of(name):
    c = Qwen2Config.from_dict(config_dict(CONFIGS[name]))
    return c, architecture_for(c.architecture).build(c)


def test_random_folder_reads_back_with_the_safetensors_package(folders):
    from safetensors.torch import load_file
    folder = folders("A", "bfloat16")
    theirs = load_file(os.path.join(folder, "model.safetensors"))
    ours = ModelFiles(folder)
    assert set(theirs) == set(ours.names())
    for name, t in theirs.items():
        assert t.dtype == torch.bfloat16
        assert torch.equal(t, ours.tensor(name))
    assert "lm_head.weight" not in theirs                      # tied: not stored
    cfg = json.load(open(os.path.join(folder, "config.json")))
    assert cfg["architectures"] == ["Qwen2ForCausalLM"] and cfg["torch_dtype"] == "bfloat16"


def test_random_weights_follow_seed_and_scheme(tmp_path):
    c, spec = spec_of("B")
    write_model_folder(str(tmp_path / "a"), c.to_dict(), spec.param_specs(), 1, torch.float32)
    write_model_folder(str(tmp_path / "b"), c.to_dict(), spec.param_specs(), 1, torch.float32)
    write_model_folder(str(tmp_path / "c"), c.to_dict(), spec.param_specs(), 2, torch.float32)
    a, b, d = (ModelFiles(str(tmp_path / x)) for x in "abc")
    w = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(a.tensor(w), b.tensor(w)) and not torch.equal(a.tensor(w), d.tensor(w))
    assert abs(float(a.tensor(w).std()) - 0.02) < 2e-3 and abs(float(a.tensor(w).mean())) < 2e-3
    assert torch.all(a.tensor("model.layers.0.input_layernorm.weight") == 1)
    assert float(a.tensor("model.layers.0.self_attn.q_proj.bias").std()) > 0.005
    assert "lm_head.weight" in set(a.names())                  # untied: stored


def test_random_values_depend_on_seed_name_and_index_alone():
    """The generator behind the random-weights mode: an element is a function of (seed, tensor name, index), so it
    does not depend on the tensor's length, on how the work is cut into chunks, or on other tensors; the values are
    close to normal with the asked deviation."""
    from rocmforge_b200.weights.random_init import fill_normal_host, normal_table, tensor_key
    key = tensor_key(7, "model.layers.3.mlp.up_proj.weight")
    a = fill_normal_host(5000, key, 0.02, torch.float32)
    assert torch.equal(a[:1234], fill_normal_host(1234, key, 0.02, torch.float32))
    assert torch.equal(a, fill_normal_host(5000, key, 0.02, torch.float32, chunk=777))
    assert not torch.equal(a, fill_normal_host(5000, tensor_key(8, "model.layers.3.mlp.up_proj.weight"), 0.02, torch.float32))
    assert not torch.equal(a, fill_normal_host(5000, tensor_key(7, "model.layers.4.mlp.up_proj.weight"), 0.02, torch.float32))
    assert torch.equal(a.bfloat16(), fill_normal_host(5000, key, 0.02, torch.bfloat16))
    big = fill_normal_host(1 << 20, key, 0.5, torch.float32).double()
    assert abs(float(big.mean())) < 3e-3 and abs(float(big.std()) - 0.5) < 3e-3
    assert abs(float((big ** 4).mean()) / 0.5 ** 4 - 3.0) < 0.05          # the fourth moment of a normal variable
    t = normal_table()
    assert t.shape == (65537,) and torch.all(t[1:] > t[:-1]) and float(t[32768]) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_model_made_on_the_device_equals_the_folder_written_on_the_host(tmp_path, dtype):
    """``Model.random(config, seed)`` fills its tensors with a kernel, ``write_model_folder`` with host arithmetic:
    the same bits, tensor by tensor (what the parts fuse at load time is compared after the same fusion)."""
    import rocmforge_b200 as rf
    c, spec = spec_of("D")
    write_model_folder(str(tmp_path), c.to_dict(), spec.param_specs(), 5, dtype)
    a = rf.Model.from_folder(str(tmp_path), dtype=dtype)
    b = rf.Model.random(c, seed=5, dtype=dtype)
    for (pa, xa), (pb, xb) in zip(a.spec.named_parts().items(), b.spec.named_parts().items()):
        for attr in ("weight", "qkv", "o", "gate_up", "down", "linear"):
            ta, tb = getattr(xa, attr, None), getattr(xb, attr, None)
            ta, tb = getattr(ta, "weight", ta), getattr(tb, "weight", tb)
            if isinstance(ta, torch.Tensor):
                assert torch.equal(ta, tb), f"{pa}{attr} differs between the folder and the device-made model"
    toks = list(range(40))
    ca, cb = a.new_cache(max_tokens=64), b.new_cache(max_tokens=64)
    la = a.step(ca, [rf.StepRequest(ca.alloc_slot(), toks, [39])])
    lb = b.step(cb, [rf.StepRequest(cb.alloc_slot(), toks, [39])])
    assert torch.equal(la, lb)


def test_load_keeps_dtypes(folders):
    c, spec = spec_of("A")
    got = load_folder(folders("A", "bfloat16"), spec.param_specs(), torch.bfloat16, "cpu")
    assert all(t.dtype == torch.bfloat16 for t in got.values())
    assert got["lm_head.weight"].data_ptr() == got["model.embed_tokens.weight"].data_ptr()   # tied = alias
    got32 = load_folder(folders("A", "bfloat16"), spec.param_specs(), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in got32.values())
    # a vector stored in 32-bit stays 32-bit on the bfloat16 path; matrices become bfloat16
    mixed = load_folder(folders("A", "float32"), spec.param_specs(), torch.bfloat16, "cpu")
    assert mixed["model.norm.weight"].dtype == torch.float32
    assert mixed["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32
    assert mixed["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert target_dtype(ParamSpec((4,), kind="int_table"), torch.int64, torch.bfloat16) == torch.int32


def test_one_error_lists_everything(tmp_path, folders):
    c, spec = spec_of("B")
    src = ModelFiles(folders("B", "float32"))
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    del tensors["model.layers.2.self_attn.k_proj.bias"]
    del tensors["lm_head.weight"]                               # untied: must be there
    tensors["model.layers.0.mlp.up_proj.weight"] = torch.zeros(7, 3)
    tensors["model.layers.1.input_layernorm.weight"] = torch.zeros(97)
    tensors["model.layers.9.extra.weight"] = torch.zeros(2)
    tensors["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    with pytest.raises(WeightError) as e:
        load_folder(str(tmp_path), spec.param_specs(), torch.float32, "cpu")
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.2.self_attn.k_proj.bias"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert {n for n, _, _ in err.wrong_shape} == {"model.layers.0.mlp.up_proj.weight",
                                                  "model.layers.1.input_layernorm.weight"}
    assert [n for n, _ in err.wrong_dtype] == ["model.norm.weight"]
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "[7, 3]", "[240, 96]", "model.norm.weight"):
        assert needle in text


def test_tied_head_may_be_absent_untied_may_not(folders):
    c, spec = spec_of("A")
    check_folder(ModelFiles(folders("A")), spec.param_specs())
    raw = config_dict(CONFIGS["A"])
    raw["tie_word_embeddings"] = False
    c2 = Qwen2Config.from_dict(raw)
    with pytest.raises(WeightError) as e:
        check_folder(ModelFiles(folders("A")), architecture_for(c2.architecture).build(c2).param_specs())
    assert e.value.missing == ["lm_head.weight"]


def test_container_faults(tmp_path):
    p = tmp_path / "model.safetensors"
    with pytest.raises(SafetensorsError):
        ModelFiles(str(tmp_path))                               # nothing there
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError):
        ModelFiles(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError):
        ModelFiles(str(tmp_path))                               # header longer than the file
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        ModelFiles(str(tmp_path))                               # data ends beyond the file
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        ModelFiles(str(tmp_path))                               # byte count does not fit the shape


def test_shards_and_duplicates(tmp_path):
    write_safetensors(str(tmp_path / "a.safetensors"), [("x", torch.ones(2)), ("y", torch.zeros(3))])
    write_safetensors(str(tmp_path / "b.safetensors"), [("z", torch.arange(4, dtype=torch.int32))])
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "a.safetensors", "y": "a.safetensors", "z": "b.safetensors"}}))
    f = ModelFiles(str(tmp_path))
    assert sorted(f.names()) == ["x", "y", "z"] and f.tensor("z").tolist() == [0, 1, 2, 3]
    write_safetensors(str(tmp_path / "b.safetensors"), [("x", torch.ones(2))])
    with pytest.raises(SafetensorsError):
        ModelFiles(str(tmp_path))


def test_a_stale_index_names_the_shard(tmp_path):
    """An index that sends a tensor to a shard which does not hold it: the error names tensor and shard."""
    write_safetensors(str(tmp_path / "a.safetensors"), [("x", torch.ones(2))])
    write_safetensors(str(tmp_path / "b.safetensors"), [("z", torch.zeros(1))])
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "a.safetensors", "y": "b.safetensors", "z": "b.safetensors"}}))
    with pytest.raises(SafetensorsError) as e:
        ModelFiles(str(tmp_path))
    assert "y (index says b.safetensors)" in str(e.value)
