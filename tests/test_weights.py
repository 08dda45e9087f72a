"""Safetensors reading and writing, the by-name loader and its one error, random folders (no GPU)."""
import json
import os
import struct

import pytest
import torch

import tiny
from prelude_b200.config import load_model_config
from prelude_b200.parts.model import DecoderModel
from prelude_b200.weights.loader import TensorReq, WeightError, WeightStore
from prelude_b200.weights.random_init import random_tensors, write_random_model
from prelude_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, find_shards, write_safetensors


def test_round_trip_against_the_safetensors_package(tmp_path):
    tensors = {"a.weight": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int64).reshape(2, 3), "h": torch.randn(4).to(torch.float16),
               "e": torch.zeros(0, 4)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors)
    from safetensors import safe_open
    with safe_open(path, framework="pt") as f:                      # the library reads what we wrote
        for k, v in tensors.items():
            assert torch.equal(f.get_tensor(k), v)
    from safetensors.torch import save_file
    other = str(tmp_path / "other.safetensors")
    save_file({k: v for k, v in tensors.items()}, other)             # we read what the library wrote
    mine = SafetensorsFile(other)
    for k, v in tensors.items():
        assert torch.equal(mine.tensor(k), v) and mine.info(k) == (v.dtype, tuple(v.shape))


def test_storage_types_kept(tmp_path):
    write_safetensors(str(tmp_path / "model.safetensors"),
                      {"bf": torch.ones(2, dtype=torch.bfloat16), "f32": torch.ones(2), "i64": torch.ones(2, dtype=torch.int64),
                       "f16": torch.ones(2, dtype=torch.float16), "f64": torch.ones(2, dtype=torch.float64)})
    st = WeightStore.open(str(tmp_path))
    assert st.get("bf").dtype == torch.bfloat16      # bfloat16 is kept
    assert st.get("f32").dtype == torch.float32      # a tensor stored in 32-bit stays so
    assert st.get("i64").dtype == torch.int32        # integer tables as int32
    assert st.get("f16").dtype == torch.bfloat16 and st.get("f64").dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = tiny.make_folder(tmp_path, "A")
    tensors = tiny.read_weights(folder)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(17)
    tensors["model.embed_tokens.weight"] = torch.zeros(256, 60)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    model = DecoderModel(load_model_config(folder).to_model_spec())
    req, opt = model.tensors()
    with pytest.raises(WeightError) as e:
        WeightStore.open(folder).check(req, opt)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["model.embed_tokens.weight", "model.layers.0.self_attn.q_norm.weight"]
    text = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (2)", "expected [16] got [17]", "expected [256, 64] got [256, 60]"):
        assert word in text


def test_tied_head_copy_is_tolerated_untied_head_is_required(tmp_path):
    folder = tiny.make_folder(tmp_path, "A")                          # tied
    tensors = tiny.read_weights(folder)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    req, opt = DecoderModel(load_model_config(folder).to_model_spec()).tensors()
    WeightStore.open(folder).check(req, opt)
    folder_b = tiny.make_folder(tmp_path, "B")                        # separate head
    tensors = tiny.read_weights(folder_b)
    del tensors["lm_head.weight"]
    write_safetensors(os.path.join(folder_b, "model.safetensors"), tensors)
    req, opt = DecoderModel(load_model_config(folder_b).to_model_spec()).tensors()
    with pytest.raises(WeightError, match="lm_head.weight"):
        WeightStore.open(folder_b).check(req, opt)


def test_integer_tensor_where_a_float_is_needed():
    st = WeightStore.from_tensors({"w": torch.zeros(2, 2, dtype=torch.int64)})
    with pytest.raises(WeightError, match="wrong type"):
        st.check({"w": TensorReq((2, 2))})


def test_shard_discovery(tmp_path):
    with pytest.raises(SafetensorsError, match="no .safetensors files were resolved"):
        find_shards(str(tmp_path))
    write_safetensors(str(tmp_path / "b.safetensors"), {"x": torch.zeros(1)})
    write_safetensors(str(tmp_path / "a.safetensors"), {"y": torch.zeros(1)})
    assert [os.path.basename(p) for p in find_shards(str(tmp_path))] == ["a.safetensors", "b.safetensors"]
    write_safetensors(str(tmp_path / "model.safetensors"), {"z": torch.zeros(1)})
    assert [os.path.basename(p) for p in find_shards(str(tmp_path))] == ["model.safetensors"]
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"y": "a.safetensors", "x": "b.safetensors", "y2": "a.safetensors"}}))
    assert [os.path.basename(p) for p in find_shards(str(tmp_path))] == ["a.safetensors", "b.safetensors"]
    st = WeightStore.open(str(tmp_path))
    assert st.names() == ["x", "y"]
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"y": "../a.safetensors"}}))
    with pytest.raises(SafetensorsError, match="leaves the model folder"):
        find_shards(str(tmp_path))


def test_corrupt_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 10_000) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="do not fit shape"):
        SafetensorsFile(str(p))


def test_random_folder_is_seeded_and_by_role(tmp_path):
    a1 = random_tensors(tiny.TINY_A, seed=0, std=0.02, norm_jitter=0.1)
    a2 = random_tensors(tiny.TINY_A, seed=0, std=0.02, norm_jitter=0.1)
    a3 = random_tensors(tiny.TINY_A, seed=1, std=0.02, norm_jitter=0.1)
    assert all(torch.equal(a1[k], a2[k]) for k in a1)
    assert not torch.equal(a1["model.embed_tokens.weight"], a3["model.embed_tokens.weight"])
    assert "lm_head.weight" not in a1 and "lm_head.weight" in random_tensors(tiny.TINY_B)
    w = a1["model.layers.0.mlp.gate_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = a1["model.layers.1.self_attn.q_norm.weight"]
    assert float(n.min()) >= 0.9 and float(n.max()) <= 1.1 and float(n.std()) > 0.01
    # a tensor's numbers do not depend on the rest of the model
    bigger = random_tensors(dict(tiny.TINY_A, num_hidden_layers=3), seed=0, std=0.02, norm_jitter=0.1)
    assert torch.equal(bigger["model.layers.1.mlp.down_proj.weight"], a1["model.layers.1.mlp.down_proj.weight"])
    folder = write_random_model(str(tmp_path / "m"), tiny.TINY_A, seed=0, dtype=torch.bfloat16)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    assert WeightStore.open(folder).get("model.norm.weight").dtype == torch.bfloat16
    with pytest.raises(Exception):
        write_random_model(str(tmp_path / "bad"), dict(tiny.TINY_A, head_dim=7))
    assert not os.path.exists(str(tmp_path / "bad" / "model.safetensors"))


def test_tensors_an_architecture_names_as_ignored_are_passed_over():
    """A checkpoint may carry buffers the parts never read; an architecture lists their name patterns in its model
    spec and the check passes over them (the reference ignores every extra tensor; here the rest still count)."""
    from dataclasses import replace
    from prelude_b200.config import load_model_config
    from prelude_b200.parts.model import DecoderModel
    spec = load_model_config(tiny.TINY_A).to_model_spec()
    tensors = dict(random_tensors(tiny.TINY_A, seed=0))
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    store = WeightStore.from_tensors(tensors)
    req, opt = DecoderModel(spec).tensors()
    with pytest.raises(WeightError) as e:
        store.check(req, opt, spec.ignored_tensors)
    assert e.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq", "model.layers.1.self_attn.rotary_emb.inv_freq"]
    lenient = replace(spec, ignored_tensors=("*.rotary_emb.inv_freq",))
    store.check(req, opt, lenient.ignored_tensors)
    tensors["model.extra.weight"] = torch.zeros(3)
    with pytest.raises(WeightError) as e:
        WeightStore.from_tensors(tensors).check(req, opt, lenient.ignored_tensors)
    assert e.value.unexpected == ["model.extra.weight"]


def test_the_two_ends_of_the_model_are_parts():
    from prelude_b200.config import load_model_config
    from prelude_b200.config.spec import LinearHeadSpec, TokenEmbeddingSpec
    from prelude_b200.parts.model import DecoderModel
    from prelude_b200.parts.registry import FAMILIES, part_class
    assert "embedding" in FAMILIES and "head" in FAMILIES
    for cfg, tied in ((tiny.TINY_A, True), (tiny.TINY_B, False)):
        spec = load_model_config(cfg).to_model_spec()
        assert spec.embedding_spec() == TokenEmbeddingSpec(cfg["vocab_size"], cfg["hidden_size"])
        assert spec.head_spec() == LinearHeadSpec(cfg["vocab_size"], cfg["hidden_size"], tied)
        m = DecoderModel(spec)
        assert isinstance(m.embedding, part_class("embedding", "token_embedding"))
        req, opt = m.tensors()
        assert ("lm_head.weight" in opt) == tied and ("lm_head.weight" in req) == (not tied)
