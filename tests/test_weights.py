"""Weights: safetensors container, by-name loading, one error for all mismatches (no GPU)."""
import json
import os
import struct

import pytest
import torch

from mdma_b200.config import load_config
from mdma_b200.engine.model import DecoderModel
from mdma_b200.weights import (CheckpointError, WeightsError, load_tensors, read_header,
                               write_random_model, write_safetensors)
from mdma_b200.weights.safetensors_io import SafetensorsFile
from tiny import TINY_A, TINY_B, make_model


def expected_of(cfg):
    arch, c = load_config(cfg)
    return DecoderModel(arch.describe(c)).expected_tensors()


def test_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t)
    f = SafetensorsFile(path)
    for k, v in t.items():
        assert torch.equal(f.tensor(k), v) and f.tensor(k).dtype == v.dtype


def test_random_model_is_seeded_and_loadable():
    d1, c, t1 = make_model(TINY_A, 3, torch.float32, norm_jitter=0)      # the random mode as it writes: norm weights 1.0
    d2, _, t2 = make_model(TINY_A, 3, torch.float32, norm_jitter=0)
    d3, _, t3 = make_model(TINY_A, 4, torch.float32, norm_jitter=0)
    assert all(torch.equal(t1[k], t2[k]) for k in t1)
    assert not torch.equal(t1["model.embed_tokens.weight"], t3["model.embed_tokens.weight"])
    assert torch.all(t1["model.norm.weight"] == 1.0)
    assert abs(t1["model.layers.0.mlp.up_proj.weight"].std().item() - 0.02) < 0.002
    loaded = load_tensors(d1, expected_of(TINY_A), torch.float32)
    assert set(loaded) == set(t1)


def test_dtype_rules():
    d, _, _ = make_model(TINY_B, 1, torch.float32)
    exp = expected_of(TINY_B)
    bf = load_tensors(d, exp, torch.bfloat16)
    assert bf["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16      # matrices in bfloat16
    assert bf["model.norm.weight"].dtype == torch.float32                            # stored 32-bit stays so
    d2, _, _ = make_model(TINY_B, 1, torch.bfloat16)
    bf2 = load_tensors(d2, exp, torch.bfloat16)
    assert bf2["model.norm.weight"].dtype == torch.bfloat16
    f32 = load_tensors(d2, exp, torch.float32)
    assert all(v.dtype == torch.float32 for v in f32.values())


def test_tied_model_has_no_separate_head():
    exp = expected_of(TINY_B)
    assert "lm_head.weight" not in exp and "model.embed_tokens.weight" in exp
    assert "lm_head.weight" in expected_of(TINY_A)


def test_one_error_lists_everything(tmp_path):
    d, _, tensors = make_model(TINY_A, 0, torch.float32)
    del tensors["model.layers.1.mlp.down_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 63)
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as e:
        load_tensors(d, expected_of(TINY_A), torch.float32)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 63), (32, 64))]
    assert [w[0] for w in err.wrong_dtype] == ["lm_head.weight"]
    text = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "q_proj.bias",
                   "is [32, 63], expected [32, 64]"):
        assert needle in text


def test_container_faults(tmp_path):
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, {"a": torch.randn(4, 4)})
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[:-5])                          # truncated
    with pytest.raises(CheckpointError, match="inside|fill"):
        read_header(path)
    open(path, "wb").write(raw + b"\0" * 8)                   # trailing bytes
    with pytest.raises(CheckpointError, match="do not fill the file"):
        read_header(path)
    open(path, "wb").write(struct.pack("<Q", 1 << 40) + raw[8:])   # absurd header length
    with pytest.raises(CheckpointError, match="header claims"):
        read_header(path)
    open(path, "wb").write(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(CheckpointError, match="not JSON"):
        read_header(path)
    with pytest.raises(CheckpointError, match="neither"):
        load_tensors(str(tmp_path / "nowhere"), {}, torch.float32)


def test_sharded_folder(tmp_path):
    d, _, tensors = make_model(TINY_A, 0, torch.float32)
    os.remove(os.path.join(d, "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(os.path.join(d, "s1.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(os.path.join(d, "s2.safetensors"), {n: tensors[n] for n in names[half:]})
    wm = {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    loaded = load_tensors(d, expected_of(TINY_A), torch.float32)
    assert all(torch.equal(loaded[n], tensors[n]) for n in names)


def test_the_container_agrees_with_the_safetensors_package(tmp_path):
    """The folder writer and the reader of this library against the `safetensors` package (a file-format
    library, not model code): it reads what we write, we read what it writes, tensor for tensor."""
    st = pytest.importorskip("safetensors.torch")
    d, _, tensors = make_model(TINY_B, 1, torch.bfloat16)
    theirs = st.load_file(os.path.join(d, "model.safetensors"))
    assert set(theirs) == set(tensors)
    for k, v in tensors.items():
        assert theirs[k].dtype == v.dtype and torch.equal(theirs[k], v), k
    t = {"w": torch.randn(5, 7), "b": torch.randn(9).bfloat16(), "i": torch.arange(12, dtype=torch.int32).reshape(3, 4)}
    path = str(tmp_path / "theirs.safetensors")
    st.save_file(t, path)
    f = SafetensorsFile(path)
    for k, v in t.items():
        assert torch.equal(f.tensor(k), v) and f.tensor(k).dtype == v.dtype


def test_seeded_weights_do_not_depend_on_the_order_or_the_piece(tmp_path):
    """Element i of a tensor is a function of (seed, name, i): a tensor made alone, in pieces, or as part of a
    model has the same values (the device fills with the same arithmetic; a GPU test compares the bits)."""
    from mdma_b200.spec import TensorSpec
    from mdma_b200.weights.random_init import normal_values, random_tensor, tensor_key
    _, _, t = make_model(TINY_A, 7, torch.float32)
    name = "model.layers.1.mlp.down_proj.weight"
    alone = random_tensor(name, TensorSpec(tuple(t[name].shape)), 7, torch.float32)
    assert torch.equal(alone, t[name])
    key = tensor_key(7, name)
    whole = normal_values(key, 0, 1000, 0.02)
    pieces = [normal_values(key, lo, 250, 0.02) for lo in range(0, 1000, 250)]
    assert (whole == __import__("numpy").concatenate(pieces)).all()
    assert torch.equal(torch.from_numpy(whole), t[name].flatten()[:1000])
