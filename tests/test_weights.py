"""Weights: the safetensors format, binding by name, the one error that lists
everything wrong, storage dtypes, random model folders."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file as st_save

import tiny_configs
from gollmgo_b200.parts import manifest_for_config
from gollmgo_b200.weights import (SafetensorsError, WeightError, WeightSpec, check_manifest,
                                  checkpoint_source, open_model_files, save_file, storage_dtype,
                                  write_random_model)


def test_roundtrip_against_the_safetensors_package(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int64).view(2, 3), "d": torch.randn(2, 2).to(torch.float16)}
    ours = str(tmp_path / "ours.safetensors")
    save_file(t.items(), ours, metadata={"k": "v"})
    back = load_file(ours)                         # their reader, our writer
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    theirs = str(tmp_path / "theirs.safetensors")
    st_save(t, theirs)
    idx = open_model_files(theirs)                 # our reader, their writer
    for k in t:
        f, e = idx[k]
        got = f.tensor(k)
        assert got.dtype == t[k].dtype and torch.equal(got, t[k])


def test_folder_of_shards_later_file_wins(tmp_path):
    save_file([("x", torch.zeros(2)), ("y", torch.ones(2))], str(tmp_path / "a.safetensors"))
    save_file([("x", torch.full((2,), 5.0))], str(tmp_path / "b.safetensors"))
    idx = open_model_files(str(tmp_path))
    assert idx["x"][0].tensor("x").tolist() == [5.0, 5.0] and idx["y"][0].tensor("y").tolist() == [1.0, 1.0]


def test_bad_files(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError):
        open_model_files(str(p))
    p2 = tmp_path / "hdr.safetensors"
    p2.write_bytes((10 ** 12).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        open_model_files(str(p2))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p3 = tmp_path / "size.safetensors"
    p3.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        open_model_files(str(p3))
    with pytest.raises(SafetensorsError):
        open_model_files(str(tmp_path / "empty_dir_that_is_missing"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg, *_ = tiny_configs.get("tiny_a")
    d = write_random_model(str(tmp_path / "m"), cfg, seed=1, dtype="float32")
    w = load_file(os.path.join(d, "model.safetensors"))
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 60)
    w["model.layers.7.extra.weight"] = torch.zeros(2)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)     # ignorable
    st_save(w, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        checkpoint_source(d, manifest_for_config(cfg), torch.float32, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 60), (64, 64))]
    msg = str(err)
    for word in ("missing", "unexpected", "wrong shape", "up_proj", "extra", "[64, 60]"):
        assert word in msg


def test_tied_model_needs_no_head_but_untied_does(tmp_path):
    cfg, *_ = tiny_configs.get("tiny_b")
    d = write_random_model(str(tmp_path / "tied"), cfg, seed=1)
    assert "lm_head.weight" not in load_file(os.path.join(d, "model.safetensors"))
    checkpoint_source(d, manifest_for_config(cfg), torch.bfloat16, "cpu")
    cfg["tie_word_embeddings"] = False
    with pytest.raises(WeightError) as e:
        checkpoint_source(d, manifest_for_config(cfg), torch.bfloat16, "cpu")
    assert e.value.missing == ["lm_head.weight"]


def test_storage_dtypes():
    bf, f32 = torch.bfloat16, torch.float32
    assert storage_dtype(bf, "float", bf) == bf
    assert storage_dtype(f32, "float", bf) == f32          # stored in 32-bit stays so
    assert storage_dtype(torch.float16, "float", bf) == bf
    assert storage_dtype(bf, "float", f32) == f32          # the float32 mode widens everything
    assert storage_dtype(torch.int64, "int", bf) == torch.int32
    with pytest.raises(WeightError):
        check_manifest({"t": WeightSpec((2,))}, {"t": ((2,), torch.int64)})


def test_checkpoint_source_delivers_storage_dtype(tmp_path):
    cfg, *_ = tiny_configs.get("tiny_a")
    d = write_random_model(str(tmp_path / "m"), cfg, seed=1, dtype="bfloat16")
    m = manifest_for_config(cfg)
    get = checkpoint_source(d, m, torch.bfloat16, "cpu")
    assert get("model.embed_tokens.weight").dtype == torch.bfloat16
    get32 = checkpoint_source(d, m, torch.float32, "cpu")
    t = get32("model.embed_tokens.weight")
    assert t.dtype == torch.float32 and torch.equal(t, get("model.embed_tokens.weight").float())


def test_random_model_depends_only_on_seed_and_name(tmp_path):
    cfg, *_ = tiny_configs.get("tiny_a")
    a = load_file(os.path.join(write_random_model(str(tmp_path / "a"), cfg, 4, "float32", std=0.1), "model.safetensors"))
    b = load_file(os.path.join(write_random_model(str(tmp_path / "b"), cfg, 4, "float32", std=0.1), "model.safetensors"))
    c = load_file(os.path.join(write_random_model(str(tmp_path / "c"), cfg, 5, "float32", std=0.1), "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert abs(float(a["model.embed_tokens.weight"].std()) - 0.1) < 0.01
    assert torch.equal(a["model.norm.weight"], torch.ones(64))
    with open(tmp_path / "a" / "config.json") as f:
        assert json.load(f)["hidden_size"] == 64
