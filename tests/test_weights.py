"""Weights: the container, binding by name, the one error, random folders (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from helpers import TINY_A, TINY_B, make_folder
from mynah_slm_b200.engine.model import Model
from mynah_slm_b200.registry import parse_config, read_config_folder
from mynah_slm_b200.weights.loader import WeightError, check, kept_dtype
from mynah_slm_b200.weights.safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors


def _write_raw(path, header: bytes, payload: bytes = b"", hlen=None):
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header) if hlen is None else hlen))
        f.write(header)
        f.write(payload)


def test_round_trip_all_dtypes(tmp_path):
    p = str(tmp_path / "t.safetensors")
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
               "d": torch.randn(2, 2).to(torch.float16), "e": torch.zeros(0, 4)}
    write_safetensors(p, tensors, metadata={"k": "v"})
    f = SafetensorsFile(p)
    assert f.metadata == {"k": "v"} and f.payload_offset % 8 == 0
    for k, v in tensors.items():
        got = f.tensor(k)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)


@pytest.mark.parametrize("case,match", [
    ("short", "shorter than"), ("long_header", "longer than the file"), ("not_json", "not valid JSON"),
    ("not_object", "not a JSON object"), ("reversed", "reversed offsets"), ("past_end", "past the payload"),
    ("bytes", "its shape and dtype need"), ("no_dtype", "has no dtype"), ("no_offsets", "has no data_offsets"),
    ("bad_dtype", "unsupported dtype"),
])
def test_malformed_files_are_refused(tmp_path, case, match):
    p = str(tmp_path / "bad.safetensors")
    ok = {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}
    if case == "short":
        open(p, "wb").write(b"abc")
    elif case == "long_header":
        _write_raw(p, b"{}", hlen=1000)
    elif case == "not_json":
        _write_raw(p, b'{"x": ')
    elif case == "not_object":
        _write_raw(p, b"[1,2]")
    else:
        t = dict(ok)
        if case == "reversed":
            t["data_offsets"] = [8, 0]
        elif case == "past_end":
            t["data_offsets"] = [0, 16]; t["shape"] = [4]
        elif case == "bytes":
            t["shape"] = [3]
        elif case == "no_dtype":
            del t["dtype"]
        elif case == "no_offsets":
            del t["data_offsets"]
        elif case == "bad_dtype":
            t["dtype"] = "Q4_K"
        _write_raw(p, json.dumps({"x": t}).encode(), b"\0" * 8)
    with pytest.raises(SafetensorsError, match=match):
        SafetensorsFile(p)


def test_sharded_folder_and_duplicates(tmp_path):
    d = str(tmp_path)
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), {"a": torch.ones(2)})
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), {"b": torch.zeros(3)})
    json.dump({"weight_map": {"a": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}},
              open(os.path.join(d, "model.safetensors.index.json"), "w"))
    c = Checkpoint(d)
    assert sorted(c.names()) == ["a", "b"] and torch.equal(c.tensor("b"), torch.zeros(3))
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), {"a": torch.zeros(2)})
    with pytest.raises(SafetensorsError, match="appears in both"):
        Checkpoint(d)


def test_random_folder_reads_back(tmp_path):
    folder = make_folder(tmp_path, "B", torch.bfloat16)
    typed = read_config_folder(folder)
    assert typed == parse_config(TINY_B)
    model = Model(typed.model_spec())
    ckpt = Checkpoint(folder)
    check(model.tensor_specs(), ckpt)              # every name and shape fits
    assert len(ckpt.entries) == 3 * 11 + 3          # untied: embedding, norm, head
    w = ckpt.tensor("model.layers.0.self_attn.q_proj.weight").float()
    g = ckpt.tensor("model.layers.1.self_attn.q_norm.weight").float()
    assert w.shape == (6 * 32, 96) and abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    assert g.shape == (32,) and abs(g.mean().item() - 1.0) < 0.1
    # the same seed writes the same bytes; another seed does not
    again = make_folder(tmp_path / "again", "B", torch.bfloat16)
    other = make_folder(tmp_path / "other", "B", torch.bfloat16, seed=99)
    a = open(os.path.join(folder, "model.safetensors"), "rb").read()
    assert a == open(os.path.join(again, "model.safetensors"), "rb").read()
    assert a != open(os.path.join(other, "model.safetensors"), "rb").read()


def test_tied_model_has_no_head_and_tolerates_one(tmp_path):
    folder = make_folder(tmp_path, "A", torch.float32)
    ckpt = Checkpoint(folder)
    assert "lm_head.weight" not in ckpt.entries
    model = Model(read_config_folder(folder).model_spec())
    check(model.tensor_specs(), ckpt)
    # the official tied checkpoint ships a duplicate head: tolerated, not "unexpected"
    tensors = {n: ckpt.tensor(n).clone() for n in ckpt.names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    check(model.tensor_specs(), Checkpoint(folder))


def test_one_error_lists_everything(tmp_path):
    folder = make_folder(tmp_path, "B", torch.float32)
    ckpt = Checkpoint(folder)
    tensors = {n: ckpt.tensor(n).clone() for n in ckpt.names()}
    del tensors["model.layers.2.mlp.down_proj.weight"]
    del tensors["lm_head.weight"]                                   # untied: required
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 95)
    tensors["model.layers.1.self_attn.q_norm.weight"] = torch.zeros(16)
    tensors["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    tensors["extra.bias"] = torch.zeros(3)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    model = Model(read_config_folder(folder).model_spec())
    with pytest.raises(WeightError) as ei:
        check(model.tensor_specs(), Checkpoint(folder))
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.2.mlp.down_proj.weight"]
    assert e.unexpected == ["extra.bias", "model.layers.7.mlp.up_proj.weight"]
    assert sorted(n for n, _, _ in e.wrong_shape) == ["model.layers.0.self_attn.k_proj.weight",
                                                      "model.layers.1.self_attn.q_norm.weight"]
    msg = str(e)
    for needle in ("missing tensors (2)", "unexpected tensors (2)", "shape [64, 95], expected [64, 96]",
                   "shape [16], expected [32]"):
        assert needle in msg, msg


def test_kept_dtypes():
    bf, f32 = torch.bfloat16, torch.float32
    assert kept_dtype("matrix", bf, bf) == bf and kept_dtype("matrix", f32, bf) == bf
    assert kept_dtype("matrix", bf, f32) == f32
    assert kept_dtype("gain", f32, bf) == f32          # stored in 32-bit stays so
    assert kept_dtype("gain", bf, bf) == bf and kept_dtype("gain", bf, f32) == f32
    assert kept_dtype("table", torch.int64, bf) == torch.int32
