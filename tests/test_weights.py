"""Weights by tensor name: folders, the single error, random mode (CPU)."""

import json
import os

import pytest
import torch

import helpers as H
import plain_model
from servelab_b200.config import config_from_dict
from servelab_b200.models import declare_tensors
from servelab_b200.weights import (BIAS, MATRIX, NORM, FolderSource, RandomSource,
                                   SafetensorsFile, WeightsError, WeightStore, check_source,
                                   write_random_model, write_safetensors)


def _decls(cfg):
    spec = config_from_dict(cfg).to_model_spec()
    return spec, declare_tensors(spec)


def test_declared_names_are_the_checkpoint_names():
    spec, decls = _decls(H.TINY_B)
    names = {d.name: d for d in decls}
    assert names["model.embed_tokens.weight"].shape == (512, 96)
    assert names["model.layers.2.self_attn.q_proj.weight"].shape == (96, 96)
    assert names["model.layers.2.self_attn.k_proj.bias"].shape == (32,)
    assert names["model.layers.0.mlp.down_proj.weight"].shape == (96, 256)
    assert names["model.layers.1.post_attention_layernorm.weight"].role == NORM
    assert names["lm_head.weight"].shape == (512, 96)
    assert "model.layers.0.self_attn.o_proj.bias" not in names
    assert len(decls) == 1 + 3 * 12 + 1 + 1
    _, tied = _decls(H.TINY_A)
    assert "lm_head.weight" not in {d.name for d in tied}


def test_random_folder_is_complete_and_reproducible(tmp_path):
    a = H.make_model(str(tmp_path / "a"), H.TINY_A, 0)
    b = H.make_model(str(tmp_path / "b"), H.TINY_A, 0)
    c = H.make_model(str(tmp_path / "c"), H.TINY_A, 1)
    spec, decls = _decls(H.TINY_A)
    src = FolderSource(a)
    check_source(src, decls, spec.ignored_suffixes)
    ta, tb, tc = (plain_model.read_safetensors(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["model.embed_tokens.weight"], tc["model.embed_tokens.weight"])
    w = ta["model.layers.0.mlp.up_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = ta["model.layers.1.input_layernorm.weight"]
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.05 < float(n.std()) < 0.2
    assert float(ta["model.layers.0.self_attn.q_proj.bias"].abs().max()) > 0
    assert json.load(open(os.path.join(a, "config.json")))["intermediate_size"] == 172


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = H.make_model(str(tmp_path / "m"), H.TINY_A, 0)
    tensors = plain_model.read_safetensors(os.path.join(folder, "model.safetensors"))
    del tensors["model.layers.0.self_attn.k_proj.bias"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.kproj.bias"] = torch.zeros(32)
    tensors["model.layers.1.mlp.up_proj.weight"] = torch.zeros(171, 64)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)   # ignorable
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(k, tuple(v.shape), v.dtype) for k, v in tensors.items()],
                      lambda n: tensors[n])
    spec, decls = _decls(H.TINY_A)
    with pytest.raises(WeightsError) as e:
        check_source(FolderSource(folder), decls, spec.ignored_suffixes)
    err = e.value
    assert err.missing == ["model.layers.0.self_attn.k_proj.bias", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.kproj.bias"]
    assert err.wrong_shape == [("model.layers.1.mlp.up_proj.weight", (171, 64), (172, 64))]
    msg = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)",
                  "model.norm.weight", "kproj", "[171, 64] != model [172, 64]"):
        assert piece in msg


def test_tied_checkpoint_may_carry_lm_head(tmp_path):
    folder = H.make_model(str(tmp_path / "m"), H.TINY_A, 0)
    tensors = plain_model.read_safetensors(os.path.join(folder, "model.safetensors"))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(k, tuple(v.shape), v.dtype) for k, v in tensors.items()],
                      lambda n: tensors[n])
    spec, decls = _decls(H.TINY_A)
    check_source(FolderSource(folder), decls, spec.ignored_suffixes, optional=("lm_head.weight",))


def test_precision_policy(tmp_path):
    spec, decls = _decls(H.TINY_A)
    for stored in (torch.float32, torch.bfloat16):
        src = RandomSource(decls, seed=3, dtype=stored)
        store = WeightStore(src, decls, torch.bfloat16, "cpu")
        assert store.get("model.embed_tokens.weight").dtype == torch.bfloat16
        assert store.get("model.norm.weight").dtype == torch.float32          # 32-bit stays
        assert store.get("model.layers.0.self_attn.q_proj.bias").dtype == torch.float32
        store32 = WeightStore(src, decls, torch.float32, "cpu")
        assert store32.get("model.embed_tokens.weight").dtype == torch.float32
    fused = store.cat(["model.layers.0.self_attn.q_proj.weight",
                       "model.layers.0.self_attn.k_proj.weight",
                       "model.layers.0.self_attn.v_proj.weight"])
    assert fused.shape == (64 + 32 + 32, 64)


def test_sharded_folder_and_corrupt_header(tmp_path):
    t = {"a": torch.randn(4, 4), "b": torch.randn(3)}
    write_safetensors(str(tmp_path / "s1.safetensors"), [("a", (4, 4), torch.float32)], lambda n: t[n])
    write_safetensors(str(tmp_path / "s2.safetensors"), [("b", (3,), torch.float32)], lambda n: t[n])
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    src = FolderSource(str(tmp_path))
    assert sorted(src.names()) == ["a", "b"] and torch.equal(src.read("b"), t["b"])
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\xff" * 16)
    with pytest.raises(ValueError, match="corrupt"):
        SafetensorsFile(str(bad))
    with pytest.raises(FileNotFoundError):
        FolderSource(str(tmp_path / "empty"))


def test_a_state_dict_checkpoint_is_read_by_name_like_a_safetensors_one(tmp_path):
    """``pytorch_model.bin`` (a state dict from ``torch.save``, the form the reference's tests
    write): the same tensors by the same names, checked and loaded like a safetensors folder;
    a file that is no dict of tensors is refused."""
    folder = H.make_model(str(tmp_path / "st"), H.TINY_A, 3)
    tensors = plain_model.read_safetensors(os.path.join(folder, "model.safetensors"))
    other = tmp_path / "bin"
    other.mkdir()
    torch.save(dict(tensors), str(other / "pytorch_model.bin"))
    (other / "config.json").write_text(open(os.path.join(folder, "config.json")).read())
    spec, decls = _decls(H.TINY_A)
    src = FolderSource(str(other))
    check_source(src, decls, spec.ignored_suffixes)
    assert sorted(src.names()) == sorted(tensors)
    for name, t in tensors.items():
        assert src.shape(name) == tuple(t.shape) and src.stored_dtype(name) == t.dtype
        assert torch.equal(src.read(name), t)
    bad = tmp_path / "bad"
    bad.mkdir()
    torch.save([1, 2, 3], str(bad / "pytorch_model.bin"))
    with pytest.raises(ValueError, match="state dict"):
        FolderSource(str(bad))


def _raw_file(path, header: dict, payload: bytes):
    import struct
    blob = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(blob)) + blob + payload)


def test_an_entry_whose_byte_range_does_not_fit_its_shape_is_refused(tmp_path):
    """Offsets inside the file are not enough: a range shorter than shape x element size
    would hand out the neighbouring tensor's bytes."""
    ok = {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]},
          "b": {"dtype": "F32", "shape": [4], "data_offsets": [16, 32]}}
    _raw_file(tmp_path / "ok.safetensors", ok, bytes(32))
    assert SafetensorsFile(str(tmp_path / "ok.safetensors")).shape("b") == (4,)
    short = {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 8]},
             "b": {"dtype": "F32", "shape": [4], "data_offsets": [8, 24]}}
    _raw_file(tmp_path / "short.safetensors", short, bytes(32))
    with pytest.raises(ValueError, match="tensor a spans 8 bytes"):
        SafetensorsFile(str(tmp_path / "short.safetensors"))
    negative = {"a": {"dtype": "F32", "shape": [4], "data_offsets": [-16, 0]}}
    _raw_file(tmp_path / "neg.safetensors", negative, bytes(32))
    with pytest.raises(ValueError, match="outside the file"):
        SafetensorsFile(str(tmp_path / "neg.safetensors"))
