"""Safetensors reading and writing, the loader's one error, random weights (no GPU)."""
import json
import os
import struct

import pytest
import torch

from hos_b200 import models  # noqa: F401
from hos_b200.errors import FormatError, IoError, MissingTensorError, WeightMismatchError
from hos_b200.model import weight_specs_for
from hos_b200.registry import config_from_dict
from hos_b200.weights import (RandomSource, SafetensorsFolder, check_against, load_tensors,
                              write_model_folder, write_safetensors)
from helpers import TINY_A, TINY_B, make_folder


def test_written_folder_reads_back_and_agrees_with_the_safetensors_package(tmp_path):
    import safetensors.torch as st
    d = make_folder(tmp_path, "A")
    ours = SafetensorsFolder(d)
    theirs = st.load_file(os.path.join(d, "model.safetensors"))
    assert set(ours.names()) == set(theirs)
    for name, t in theirs.items():
        dt, shape = ours.info(name)
        assert dt == torch.bfloat16 and tuple(shape) == tuple(t.shape)
        assert torch.equal(ours.read(name), t)
    with open(os.path.join(d, "config.json")) as f:
        assert config_from_dict(json.load(f)) == config_from_dict(TINY_A)


def test_a_file_of_the_safetensors_package_reads_here(tmp_path):
    import safetensors.torch as st
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).view(2, 3)}
    st.save_file(tensors, str(tmp_path / "model.safetensors"))
    f = SafetensorsFolder(str(tmp_path))
    for k, v in tensors.items():
        assert torch.equal(f.read(k), v)
    with pytest.raises(MissingTensorError, match="nope"):
        f.read("nope")


def test_random_weights_depend_on_seed_and_name_only():
    specs = weight_specs_for(config_from_dict(TINY_B))
    a, b, c = RandomSource(specs, 1), RandomSource(list(reversed(specs)), 1), RandomSource(specs, 2)
    name = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(a.read(name), b.read(name)) and not torch.equal(a.read(name), c.read(name))
    assert a.read(name).dtype == torch.bfloat16
    assert abs(a.read(name).float().std().item() - 0.02) < 0.002
    assert abs(a.read("model.norm.weight").float().std().item() - 0.1) < 0.03
    assert "lm_head.weight" not in a.names()          # tied: the embedding table serves


def test_sharded_folder(tmp_path):
    specs = weight_specs_for(config_from_dict(TINY_A))
    src = RandomSource(specs, 3)
    names = src.names()
    half = len(names) // 2
    write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), [(n, src.read(n)) for n in names[:half]])
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), [(n, src.read(n)) for n in names[half:]])
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    f = SafetensorsFolder(str(tmp_path))
    assert sorted(f.names()) == sorted(names)
    assert torch.equal(f.read(names[-1]), src.read(names[-1]))
    tensors = load_tensors(specs, f, torch.device("cpu"))
    assert tensors["lm_head.weight"] is tensors["model.embed_tokens.weight"]


def _write_raw(path, header: bytes, data: bytes = b""):
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + data)


def test_malformed_files_raise_format_errors(tmp_path):
    p = str(tmp_path / "model.safetensors")
    with pytest.raises(FormatError, match="no safetensors"):
        SafetensorsFolder(str(tmp_path))
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(FormatError, match="too small"):
        SafetensorsFolder(str(tmp_path))
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(FormatError, match="header out of bounds"):
        SafetensorsFolder(str(tmp_path))
    _write_raw(p, b"{not json")
    with pytest.raises(FormatError, match="bad header json"):
        SafetensorsFolder(str(tmp_path))
    _write_raw(p, json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode(), b"\0" * 8)
    with pytest.raises(FormatError, match="out of bounds"):
        SafetensorsFolder(str(tmp_path))
    _write_raw(p, json.dumps({"t": {"dtype": "Q4_K", "shape": [4], "data_offsets": [0, 16]}}).encode(), b"\0" * 16)
    with pytest.raises(FormatError, match="unsupported"):
        SafetensorsFolder(str(tmp_path))
    _write_raw(p, json.dumps({"t": {"dtype": "F32", "shape": [5], "data_offsets": [0, 16]}}).encode(), b"\0" * 16)
    with pytest.raises(FormatError, match="do not hold"):
        SafetensorsFolder(str(tmp_path))
    _write_raw(p, json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [16, 0]}}).encode(), b"\0" * 16)
    with pytest.raises(FormatError, match="out of bounds"):
        SafetensorsFolder(str(tmp_path))
    _write_raw(p, json.dumps({"__metadata__": {"x": "y"}, "t": {"dtype": "F32", "shape": [4],
                                                               "data_offsets": [0, 16]}}).encode(), b"\0" * 16)
    assert SafetensorsFolder(str(tmp_path)).names() == ["t"]
    (tmp_path / "config.json").write_text("{broken")
    from hos_b200.config import read_config_json
    with pytest.raises(FormatError):
        read_config_json(str(tmp_path))
    with pytest.raises(IoError):
        read_config_json(str(tmp_path / "absent"))


def test_truncation_anywhere_never_crashes(tmp_path):
    d = make_folder(tmp_path, "A")
    blob = open(os.path.join(d, "model.safetensors"), "rb").read()
    t = tmp_path / "cut"
    t.mkdir()
    for cut in (0, 4, 8, 9, 100, len(blob) // 2, len(blob) - 1):
        (t / "model.safetensors").write_bytes(blob[:cut])
        with pytest.raises(FormatError):
            SafetensorsFolder(str(t))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    specs = weight_specs_for(config_from_dict(TINY_A))
    src = RandomSource(specs, 0)
    tensors = {n: src.read(n) for n in src.names()}
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.9.extra.weight"] = torch.zeros(2, 2, dtype=torch.bfloat16)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(8, 64, dtype=torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    with pytest.raises(WeightMismatchError) as e:
        check_against(specs, SafetensorsFolder(str(tmp_path)))
    err = e.value
    assert err.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.1.self_attn.k_proj.weight", (32, 64), (8, 64))]
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "expected [32, 64] found [8, 64]",
                  "model.norm.weight", "model.layers.9.extra.weight"):
        assert piece in text


def test_untied_head_is_used_when_present_and_dtypes_are_kept(tmp_path):
    specs = weight_specs_for(config_from_dict(TINY_A))
    src = RandomSource(specs, 0)
    tensors = {n: src.read(n) for n in src.names()}
    tensors["lm_head.weight"] = torch.ones(256, 64, dtype=torch.bfloat16)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()          # stored in 32-bit
    tensors["model.layers.0.input_layernorm.weight"] = tensors["model.layers.0.input_layernorm.weight"].half()
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    got = load_tensors(specs, SafetensorsFolder(str(tmp_path)), torch.device("cpu"))
    assert got["lm_head.weight"] is not got["model.embed_tokens.weight"]
    assert torch.equal(got["lm_head.weight"], tensors["lm_head.weight"])
    assert got["model.norm.weight"].dtype == torch.float32                        # stays 32-bit
    assert got["model.layers.0.input_layernorm.weight"].dtype == torch.bfloat16   # float16 -> bfloat16
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16
