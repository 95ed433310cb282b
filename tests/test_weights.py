"""Weights by name: the file format, the one error, the random-weights folder (CPU)."""

import json
import struct

import pytest
import torch
from safetensors.torch import load_file, save_file

from mini_llm_stack_b200.config import build_model, config_from_dict, config_from_folder
from mini_llm_stack_b200.weights import (SafetensorsFile, SafetensorsFormatError, WeightError,
                                         load_tensors, random_tensors, write_random_model,
                                         write_safetensors)
from mini_llm_stack_b200.weights.loader import device_dtype
from tiny_configs import CONFIGS, NORM_STD, TINY_A, TINY_B


def _folder(tmp_path, raw, dtype="float32", seed=3, norm_std=0.0):
    cfg = config_from_dict(dict(raw, dtype=dtype))
    write_random_model(tmp_path, cfg, seed, norm_std)
    return cfg


def test_writer_is_read_by_the_safetensors_package_and_back(tmp_path):
    cfg = _folder(tmp_path, TINY_B, "bfloat16", norm_std=0.1)
    theirs = load_file(str(tmp_path / "model.safetensors"))
    specs = build_model(cfg).tensor_specs()
    assert set(theirs) == set(specs)
    with SafetensorsFile(tmp_path / "model.safetensors") as f:
        for n, t in theirs.items():
            assert t.dtype == torch.bfloat16 and tuple(t.shape) == tuple(specs[n].shape)
            assert torch.equal(f.read(n), t)
    # and a file written by the package is read by ours
    save_file({"a": torch.arange(6, dtype=torch.float32).view(2, 3),
               "t": torch.tensor([1, 2, 3], dtype=torch.int64)}, str(tmp_path / "x.safetensors"))
    with SafetensorsFile(tmp_path / "x.safetensors") as f:
        assert f.read("a").tolist() == [[0, 1, 2], [3, 4, 5]] and f.read("t").dtype == torch.int64


def test_same_seed_same_folder_and_distribution(tmp_path):
    cfg = config_from_dict(dict(TINY_A, dtype="float32"))
    a = dict(random_tensors(cfg, 11))
    b = dict(random_tensors(cfg, 11))
    c = dict(random_tensors(cfg, 12))
    assert all(torch.equal(a[n], b[n]) for n in a)
    assert not torch.equal(a["embed.weight"], c["embed.weight"])
    # N(0, 0.02^2) for matrices, ones for norms (train/model.py:232-236, :27)
    assert abs(a["embed.weight"].std().item() - 0.02) < 2e-3
    assert torch.equal(a["final_norm.weight"], torch.ones(64))
    d = dict(random_tensors(cfg, 11, norm_std=0.1))
    assert 0.05 < (d["final_norm.weight"] - 1).std().item() < 0.2


def test_loads_by_name_with_run_dtype_rules(tmp_path):
    cfg = _folder(tmp_path, TINY_A, "bfloat16")
    m = build_model(cfg)
    t16 = load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.bfloat16, "cpu")
    assert all(t.dtype == torch.bfloat16 for t in t16.values())
    t32 = load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in t32.values())
    assert torch.equal(t32["embed.weight"], t16["embed.weight"].float())
    # stored in 32 bits: stays so in a bfloat16 run; integer tables become int32
    assert device_dtype(torch.float32, "matrix", torch.bfloat16) == torch.float32
    assert device_dtype(torch.float16, "matrix", torch.bfloat16) == torch.bfloat16
    assert device_dtype(torch.bfloat16, "vector", torch.float32) == torch.float32
    assert device_dtype(torch.int64, "table", torch.bfloat16) == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = _folder(tmp_path, TINY_B)
    path = str(tmp_path / "model.safetensors")
    w = load_file(path)
    del w["blocks.1.attn.wq.weight"]
    del w["final_norm.weight"]
    w["blocks.9.extra"] = torch.zeros(2)
    w["blocks.0.mlp.w_up.weight"] = torch.zeros(5, 5)
    w["embed.weight"] = torch.zeros(96, 97)
    save_file(w, path)
    m = build_model(cfg)
    with pytest.raises(WeightError) as err:
        load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.float32, "cpu")
    e = err.value
    assert sorted(e.missing) == ["blocks.1.attn.wq.weight", "final_norm.weight"]
    assert e.unexpected == ["blocks.9.extra"]
    assert sorted(n for n, _, _ in e.wrong_shape) == ["blocks.0.mlp.w_up.weight", "embed.weight"]
    text = str(e)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)",
                 "blocks.9.extra", "expected [97, 96], file has [96, 97]"):
        assert word in text


def test_a_file_may_use_the_usual_folder_spellings_of_the_names(tmp_path):
    cfg = _folder(tmp_path, TINY_B)
    path = str(tmp_path / "model.safetensors")
    m = build_model(cfg)
    # copies: the file is written over below, and tensors read from it are views of its mapping
    want = {n: t.clone() for n, t in load_tensors(tmp_path, m.tensor_specs(), m.tied_names(),
                                                  torch.float32, "cpu").items()}
    aliases = m.name_aliases()
    assert aliases["blocks.2.attn.wk.weight"] == ["model.layers.2.self_attn.k_proj.weight"]
    assert aliases["embed.weight"] == ["model.embed_tokens.weight"] and "lm_head.weight" not in aliases
    w = {n: t.clone() for n, t in load_file(path).items()}
    renamed = {aliases.get(n, [n])[0]: t.clone() for n, t in w.items()}
    assert set(renamed).isdisjoint(set(w) - {"lm_head.weight"})
    save_file(renamed, path)
    with pytest.raises(WeightError):                       # not without the table
        load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.float32, "cpu")
    got = load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.float32, "cpu",
                       aliases=aliases)
    assert set(got) == set(want) and all(torch.equal(got[n], want[n]) for n in want)
    # errors speak the model's names; a leftover tensor keeps the file's
    renamed["model.layers.0.mlp.up_proj.weight"] = torch.zeros(3, 3)
    del renamed["model.norm.weight"]
    renamed["model.layers.7.rotary.inv_freq"] = torch.zeros(4)
    save_file(renamed, path)
    with pytest.raises(WeightError) as err:
        load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.float32, "cpu",
                     aliases=aliases)
    e = err.value
    assert e.missing == ["final_norm.weight"] and e.unexpected == ["model.layers.7.rotary.inv_freq"]
    assert [n for n, _, _ in e.wrong_shape] == ["blocks.0.mlp.w_up.weight"]
    # a name of the model's own wins over its other spelling
    both = dict(w)
    both["model.embed_tokens.weight"] = torch.zeros_like(w["embed.weight"])
    save_file(both, path)
    with pytest.raises(WeightError) as err:
        load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.float32, "cpu",
                     aliases=aliases)
    assert err.value.unexpected == ["model.embed_tokens.weight"]


def test_weights_spread_over_several_files_with_an_index(tmp_path):
    cfg = _folder(tmp_path, TINY_A, "bfloat16")
    m = build_model(cfg)
    want = load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.bfloat16, "cpu")
    names = sorted(want)
    parts = {"model-00001-of-00002.safetensors": names[::2],
             "model-00002-of-00002.safetensors": names[1::2]}
    for fname, own in parts.items():
        save_file({n: want[n].clone() for n in own}, str(tmp_path / fname))
    (tmp_path / "model.safetensors").unlink()
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"metadata": {}, "weight_map": {n: f for f, own in parts.items() for n in own}}))
    got = load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.bfloat16, "cpu")
    assert set(got) == set(want) and all(torch.equal(got[n], want[n]) for n in want)
    # an index that names a tensor its file does not hold
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {names[0]: "model-00002-of-00002.safetensors"}}))
    with pytest.raises(SafetensorsFormatError, match="does not hold"):
        load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.bfloat16, "cpu")


def test_tied_head_in_the_file_is_accepted_only_if_equal(tmp_path):
    cfg = _folder(tmp_path, TINY_A)
    path = str(tmp_path / "model.safetensors")
    m = build_model(cfg)
    w = load_file(path)
    w["lm_head.weight"] = w["embed.weight"].clone()     # the reference's state_dict holds both
    save_file(w, path)
    load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.float32, "cpu")
    w["lm_head.weight"] = w["embed.weight"] + 1
    save_file(w, path)
    with pytest.raises(WeightError, match="ties it to embed.weight"):
        load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.float32, "cpu")


def test_float_where_a_table_is_needed_is_an_error(tmp_path):
    cfg = _folder(tmp_path, TINY_A)
    path = str(tmp_path / "model.safetensors")
    w = load_file(path)
    w["final_norm.weight"] = torch.ones(64, dtype=torch.int32)
    save_file(w, path)
    m = build_model(cfg)
    with pytest.raises(WeightError, match="floating tensor"):
        load_tensors(tmp_path, m.tensor_specs(), m.tied_names(), torch.float32, "cpu")


def test_broken_files(tmp_path):
    with pytest.raises(FileNotFoundError):
        SafetensorsFile(tmp_path / "none.safetensors")
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsFormatError, match="header length"):
        SafetensorsFile(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsFormatError, match="inconsistent"):
        SafetensorsFile(p)


def test_folder_has_config_and_weights(tmp_path):
    for key, raw in CONFIGS.items():
        d = tmp_path / key
        cfg = _folder(d, raw, norm_std=NORM_STD[key])
        assert config_from_folder(d) == cfg
        assert (d / "model.safetensors").is_file()


def test_writer_checks_what_it_is_given(tmp_path):
    with pytest.raises(ValueError, match="declared"):
        write_safetensors(tmp_path / "w.safetensors", [("a", torch.float32, (2,))],
                          lambda n: torch.zeros(3))
