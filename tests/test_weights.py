"""safetensors container, weight store errors, random-weights mode (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from conftest import SEEDS, TINY
from mimirmind_b200.weights import (SafetensorsError, SafetensorsFolder, WeightsError, expected_tensors, load_spec,
                                    load_tensors, random_tensors, write_random_model, write_safetensors)
from mimirmind_b200.weights.safetensors_io import parse_header


def _file(header: dict, data: bytes = b"") -> bytes:
    blob = json.dumps(header).encode()
    return struct.pack("<Q", len(blob)) + blob + data


def _parse(raw: bytes):
    return parse_header(raw, len(raw), "t")


def test_header_valid():
    raw = _file({"__metadata__": {"a": "b"}, "x": {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 24]}}, b"\0" * 24)
    recs, start = _parse(raw)
    assert recs["x"].shape == (2, 3) and start == len(raw) - 24


# the reference's malformed-file matrix (tests/safetensors_tests.cpp:150-197)
@pytest.mark.parametrize("raw,msg", [
    (b"\x01\x02", "shorter"),
    (struct.pack("<Q", 1000) + b"{}", "past the end"),
    (struct.pack("<Q", 5) + b"{bad}", "not valid JSON"),
    (_file({"x": {"dtype": "F7", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4), "unknown dtype"),
    (_file({"x": {"dtype": "F32", "shape": [1], "data_offsets": [0, 400]}}, b"\0" * 4), "past the data region"),
    (_file({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4), "needs 8"),
    (_file({"x": {"dtype": "F32", "shape": [1], "data_offsets": [4, 0]}}, b"\0" * 4), "invalid data_offsets|begin"),
    (_file({"x": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 4]}}, b"\0" * 4), "invalid shape"),
    (_file({"x": {"dtype": "F32", "shape": [1]}}, b"\0" * 4), "lacks"),
])
def test_header_malformed(raw, msg):
    with pytest.raises(SafetensorsError, match=msg):
        _parse(raw)


def test_duplicate_name_rejected():
    blob = b'{"x":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"x":{"dtype":"F32","shape":[1],"data_offsets":[4,8]}}'
    raw = struct.pack("<Q", len(blob)) + blob + b"\0" * 8
    with pytest.raises(SafetensorsError, match="twice"):
        _parse(raw)


def test_write_read_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3)}
    p = tmp_path / "model.safetensors"
    write_safetensors(str(p), t)
    with SafetensorsFolder(str(tmp_path)) as f:
        assert set(f.names()) == {"a", "b", "c"}
        for k in t:
            assert torch.equal(f.tensor(k), t[k]) and f.tensor(k).dtype == t[k].dtype


def test_sharded_folder(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.ones(2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    with SafetensorsFolder(str(tmp_path)) as f:
        assert torch.equal(f.tensor("b"), torch.zeros(3))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "s2.safetensors"}}))
    with pytest.raises(SafetensorsError, match="not in it"):
        SafetensorsFolder(str(tmp_path))
    write_safetensors(str(tmp_path / "s2.safetensors"), {"a": torch.zeros(2), "b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    with pytest.raises(SafetensorsError, match="two shards"):
        SafetensorsFolder(str(tmp_path))


def test_names_with_escapes_and_metadata_round_trip(tmp_path):
    # a name with a quote, a backslash, a control character and letters beyond ASCII (two and four bytes in UTF-8)
    odd = 'w"\\\t\u00e9\U0001d11e.weight'
    t = {odd: torch.arange(4, dtype=torch.int32), "empty": torch.zeros(0, 3), "scalar": torch.tensor(2.5)}
    p = tmp_path / "model.safetensors"
    write_safetensors(str(p), t, metadata={"format": "pt", 'k"ey': "v\nal"})
    raw = p.read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])                 # a standard reader agrees with what was written
    assert header["__metadata__"] == {"format": "pt", 'k"ey': "v\nal"} and set(header) == set(t) | {"__metadata__"}
    assert (8 + hlen) % 8 == 0                           # the data region starts on an 8-byte boundary
    with SafetensorsFolder(str(tmp_path)) as f:
        assert torch.equal(f.tensor(odd), t[odd]) and f.shape("empty") == (0, 3) and f.shape("scalar") == ()
        assert f.tensor("empty").numel() == 0 and float(f.tensor("scalar")) == 2.5
    # the same header written by a standard writer with \u escapes (surrogate pair included) reads back to the same name
    blob = json.dumps({odd: {"dtype": "I32", "shape": [4], "data_offsets": [0, 16]}}, ensure_ascii=True).encode()
    recs, _ = _parse(struct.pack("<Q", len(blob)) + blob + b"\0" * 16)
    assert list(recs) == [odd]


def test_files_of_the_safetensors_package_both_ways(tmp_path):
    """The container as the widely used writer makes it (header padded with spaces) reads here, and what is written here
    reads there.  Skipped where that package is not installed."""
    st = pytest.importorskip("safetensors.torch")
    t = {"a.weight": torch.randn(5, 7).to(torch.bfloat16), "b": torch.arange(10, dtype=torch.int64), "c": torch.randn(3), "h": torch.randn(2, 2).half()}
    st.save_file(t, str(tmp_path / "model.safetensors"), metadata={"format": "pt"})
    with SafetensorsFolder(str(tmp_path)) as f:
        assert set(f.names()) == set(t)
        for k in t:
            assert torch.equal(f.tensor(k), t[k]) and f.tensor(k).dtype == t[k].dtype
    write_safetensors(str(tmp_path / "ours.safetensors"), t, metadata={"format": "pt"})
    back = st.load_file(str(tmp_path / "ours.safetensors"))
    for k in t:
        assert torch.equal(back[k], t[k])


def test_a_file_that_shrank_after_opening_is_an_error(tmp_path):
    p = tmp_path / "model.safetensors"
    write_safetensors(str(p), {"a": torch.ones(1024)})
    with SafetensorsFolder(str(tmp_path)) as f:
        os.truncate(p, os.path.getsize(p) - 100)
        with pytest.raises(SafetensorsError, match="read failed"):
            f.tensor("a")


def test_empty_folder(tmp_path):
    with pytest.raises(SafetensorsError, match="neither"):
        SafetensorsFolder(str(tmp_path))


# ---- store -----------------------------------------------------------------------

def test_expected_tensor_names_are_hf_names(model_folders):
    _, spec = load_spec(model_folders("B"))
    names = expected_tensors(spec)
    assert "model.layers.2.self_attn.k_proj.bias" in names and names["model.layers.2.self_attn.k_proj.bias"].shape == (32,)
    assert names["model.layers.0.mlp.down_proj.weight"].shape == (192, 352)
    assert names["lm_head.weight"].shape == (384, 192) and not names["lm_head.weight"].optional
    _, specA = load_spec(model_folders("A"))
    assert expected_tensors(specA)["lm_head.weight"].optional      # tied: head may be absent


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_folders, tmp_path):
    src = model_folders("A")
    with SafetensorsFolder(src) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    del tensors["model.layers.1.self_attn.q_proj.bias"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.mlp.up_proj.weight"] = torch.zeros(5, 64)
    (tmp_path / "config.json").write_text(open(os.path.join(src, "config.json")).read())
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    _, spec = load_spec(str(tmp_path))
    with pytest.raises(WeightsError) as e:
        load_tensors(str(tmp_path), spec, torch.float32, "cpu")
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.self_attn.q_proj.bias" in msg and "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.0.extra.weight" in msg
    assert "wrong shapes (1)" in msg and "file has [5, 64], config needs [176, 64]" in msg


def test_precision_policy(model_folders, tmp_path):
    src = model_folders("A", "bfloat16")
    _, spec = load_spec(src)
    t = load_tensors(src, spec, torch.bfloat16, "cpu")
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    t32 = load_tensors(src, spec, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t32.values())
    assert torch.equal(t32["model.norm.weight"], t["model.norm.weight"].float())
    # a tensor stored in 32 bits stays so in a bfloat16 run
    with SafetensorsFolder(src) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    (tmp_path / "config.json").write_text(open(os.path.join(src, "config.json")).read())
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    t = load_tensors(str(tmp_path), spec, torch.bfloat16, "cpu")
    assert t["model.norm.weight"].dtype == torch.float32
    assert t["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16


def test_random_weights_are_seeded_and_distributed(tmp_path):
    a, b = tmp_path / "a", tmp_path / "b"
    write_random_model(str(a), TINY["B"], 7, "float32")
    write_random_model(str(b), TINY["B"], 7, "float32")
    assert open(a / "model.safetensors", "rb").read() == open(b / "model.safetensors", "rb").read()
    write_random_model(str(b), TINY["B"], 8, "float32")
    assert open(a / "model.safetensors", "rb").read() != open(b / "model.safetensors", "rb").read()
    cfg = json.load(open(a / "config.json"))
    assert cfg["hidden_size"] == 192 and cfg["torch_dtype"] == "float32"
    with SafetensorsFolder(str(a)) as f:
        w = f.tensor("model.layers.0.mlp.gate_proj.weight")
        n = f.tensor("model.layers.1.input_layernorm.weight")
        bias = f.tensor("model.layers.1.self_attn.q_proj.bias")
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    assert abs(n.mean().item() - 1.0) < 0.05 and abs(n.std().item() - 0.1) < 0.03
    assert abs(bias.std().item() - 0.02) < 0.006


def test_unknown_architecture_is_named(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY["A"], architectures=["FooForCausalLM"])))
    with pytest.raises(KeyError, match="FooForCausalLM"):
        load_spec(str(tmp_path))
