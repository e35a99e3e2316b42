"""Weights: safetensors reading and writing, binding by name, the one error that lists everything (no GPU)."""
import json
import os

import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
from ghost_infer_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_model_tensors,
                                      save_safetensors, write_random_model)
from conftest import TINY_A, TINY_B
import plain_llama as pl


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    p = str(tmp_path / "x.safetensors")
    save_safetensors(p, t, metadata={"k": "v"})
    f = SafetensorsFile(p)
    assert set(f.names()) == {"a", "b", "c"} and f.metadata["k"] == "v"
    for k in t:
        got = f.get(k)
        assert got.dtype == t[k].dtype and torch.equal(got, t[k])
    # the independent reader of the plain implementation agrees
    plain = pl.read_safetensors(p) if False else None
    w = {k: v for k, v in t.items() if v.is_floating_point()}
    save_safetensors(p, w)
    plain = pl.read_safetensors(p)
    for k in w:
        assert np.array_equal(plain[k], w[k].double().numpy())


def test_safetensors_bad_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)   # data shorter than the header says
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))


def test_random_model_folder_is_reproducible(tmp_path):
    a, b, c = (str(tmp_path / n) for n in "abc")
    write_random_model(a, TINY_A, seed=5)
    write_random_model(b, TINY_A, seed=5)
    write_random_model(c, TINY_A, seed=6)
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    n = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(fa.get(n), fb.get(n)) and not torch.equal(fa.get(n), fc.get(n))
    assert fa.get(n).dtype == torch.bfloat16
    assert torch.all(fa.get("model.norm.weight") == 1)
    assert abs(fa.get(n).float().std().item() - 0.02) < 0.002
    assert json.load(open(os.path.join(a, "config.json")))["hidden_size"] == 64


def test_bind_errors_list_everything(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, TINY_A, seed=0, dtype="float32")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.get(n).clone() for n in f.names()}
    del t["model.layers.0.self_attn.q_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.7.extra.weight"] = torch.zeros(3)
    t["model.layers.1.mlp.down_proj.weight"] = torch.zeros(64, 175)
    t["lm_head.weight"] = torch.zeros(255, 64)
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    model = gi.Model.from_config_dict(TINY_A)
    with pytest.raises(WeightsError) as e:
        load_model_tensors(d, model.weight_manifest(), model.ignorable_tensors())
    err = e.value
    assert set(err.missing) == {"model.layers.0.self_attn.q_proj.weight", "model.norm.weight"}
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert len(err.wrong) == 2 and "[64, 175]" in str(err) and "[255, 64]" in str(err)
    for name in ("model.norm.weight", "model.layers.7.extra.weight", "model.layers.1.mlp.down_proj.weight"):
        assert name in str(err)


def test_tied_model_may_carry_an_unused_head(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, TINY_B, seed=1)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    assert "lm_head.weight" not in set(f.names())
    t = {n: f.get(n).clone() for n in f.names()}
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    model = gi.Model.from_config_dict(TINY_B)
    got = load_model_tensors(d, model.weight_manifest(), model.ignorable_tensors())
    assert "lm_head.weight" not in got and "model.embed_tokens.weight" in got


def test_stored_precision_is_kept():
    from ghost_infer_b200.parts import Runtime
    rt16 = Runtime(torch.device("cpu"), torch.bfloat16)
    rt32 = Runtime(torch.device("cpu"), torch.float32)
    assert rt16.place(torch.zeros(2, dtype=torch.bfloat16)).dtype == torch.bfloat16
    assert rt16.place(torch.zeros(2, dtype=torch.float32)).dtype == torch.float32    # stored in 32-bit stays so
    assert rt16.place(torch.zeros(2, dtype=torch.float16)).dtype == torch.bfloat16
    assert rt32.place(torch.zeros(2, dtype=torch.bfloat16)).dtype == torch.float32
    assert rt16.place(torch.zeros(2, dtype=torch.int64)).dtype == torch.int32        # integer tables as int32
