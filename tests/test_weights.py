"""Weights: the safetensors reader and writer, the one error that lists everything wrong, the
element-type policy and the random-weights mode (no GPU)."""

import json
import os

import pytest
import torch

from rust_llm_inference_server_b200.models import build_model
from rust_llm_inference_server_b200.weights import (Checkpoint, SafetensorsError, WeightError,
                                                    open_model_dir, random_tensors, save_file,
                                                    write_random_model)
from tests.tiny_configs import TINY_A, TINY_B


def test_writer_is_read_by_the_safetensors_package_and_back(tmp_path):
    from safetensors.torch import load_file, save_file as st_save
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32),
         "c": torch.randn(4), "d.e": torch.randn(2, 2, 2).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p, {"k": "v"})
    back = load_file(p)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    st_save(t, str(tmp_path / "y.safetensors"))
    ck = open_model_dir(str(tmp_path))
    for k in t:
        assert ck.dtype(k) == t[k].dtype and ck.shape(k) == tuple(t[k].shape)
        assert torch.equal(ck.get(k), t[k])


def test_bad_files_are_refused(tmp_path):
    with pytest.raises(SafetensorsError):
        open_model_dir(str(tmp_path))
    (tmp_path / "bad.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{not json")
    with pytest.raises(SafetensorsError):
        open_model_dir(str(tmp_path))


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    model = build_model(TINY_B, "float32", "cpu")
    t = random_tensors(TINY_B, 1, "bfloat16")
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(96, 95, dtype=torch.bfloat16)
    t["model.layers.9.extra.weight"] = torch.zeros(1)
    with pytest.raises(WeightError) as e:
        model.load(Checkpoint(tensors=t))
    msg = str(e.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "model.layers.9.extra.weight" in msg
    assert "q_proj.weight: expected shape [96, 96], checkpoint has [96, 95]" in msg
    assert "missing tensors (2)" in msg and "unexpected tensors (1)" in msg


def test_tied_model_ignores_a_stored_lm_head_and_untied_needs_it():
    t = random_tensors(TINY_A, 0)
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    m = build_model(TINY_A, "bfloat16", "cpu")
    m.load(Checkpoint(tensors=t))
    assert m.lm_head.weight is m.embedding.weight
    tb = random_tensors(TINY_B, 2)
    del tb["lm_head.weight"]
    with pytest.raises(WeightError):
        build_model(TINY_B, "bfloat16", "cpu").load(Checkpoint(tensors=tb))


def test_element_type_policy():
    t = random_tensors(TINY_A, 0, "bfloat16")
    m16 = build_model(TINY_A, "bfloat16", "cpu")
    m16.load(Checkpoint(tensors=t))
    m32 = build_model(TINY_A, "float32", "cpu")
    m32.load(Checkpoint(tensors=t))
    a16, a32 = m16.blocks[0].mixer, m32.blocks[0].mixer
    assert a16.w_qkv.dtype == torch.bfloat16 and a32.w_qkv.dtype == torch.float32
    assert torch.equal(a16.w_qkv.float(), a32.w_qkv)                 # widening is exact
    assert a16.w_qkv.shape == ((4 + 2 * 2) * 16, 64)
    assert m16.blocks[0].norm1.weight.dtype == torch.float32         # norm weights: float32
    assert torch.equal(m16.blocks[0].norm1.weight, t["model.layers.0.input_layernorm.weight"].float())
    # a checkpoint stored in 32-bit: float32 path keeps every bit
    t32 = random_tensors(TINY_A, 0, "float32")
    m = build_model(TINY_A, "float32", "cpu")
    m.load(Checkpoint(tensors=t32))
    assert torch.equal(m.embedding.weight, t32["model.embed_tokens.weight"])


def test_random_model_folder_is_seeded_and_order_independent(tmp_path):
    d1 = write_random_model(TINY_B, str(tmp_path / "m1"), 3)
    d2 = write_random_model(TINY_B, str(tmp_path / "m2"), 3)
    d3 = write_random_model(TINY_B, str(tmp_path / "m3"), 4)
    a, b, c = open_model_dir(d1), open_model_dir(d2), open_model_dir(d3)
    assert sorted(os.listdir(d1)) == ["config.json", "model.safetensors"]
    n = "model.layers.2.mlp.down_proj.weight"
    assert torch.equal(a.get(n), b.get(n)) and not torch.equal(a.get(n), c.get(n))
    assert a.dtype(n) == torch.bfloat16 and a.shape(n) == (96, 256)
    w = a.get(n).float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    g = a.get("model.norm.weight").float()
    assert abs(float(g.mean()) - 1.0) < 0.01
    cfg = json.load(open(os.path.join(d1, "config.json")))
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["hidden_size"] == 96
