"""Weights: read by name, types kept, and ONE error that lists every mismatch."""
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny
from atom_b200.config import load_model_config
from atom_b200.models import build_model_spec
from atom_b200.models.model import Model
from atom_b200.weights import WeightError, expected_tensors, load_weights, write_random_model


def _model(d):
    return Model(build_model_spec(load_model_config(d)))


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_roundtrip_values_and_stacking(model_dirs, name):
    d = model_dirs[name]
    m = _model(d)
    raw = load_file(os.path.join(d, "model.safetensors"))
    assert all(t.dtype == torch.bfloat16 for t in raw.values())
    assert set(raw) == set(expected_tensors(m))
    w = load_weights(m, d, torch.bfloat16, "cpu")
    p = "model.layers.0.self_attn"
    want = torch.cat([raw[f"{p}.q_proj.weight"], raw[f"{p}.k_proj.weight"], raw[f"{p}.v_proj.weight"]])
    assert torch.equal(w["layers.0.mixer.qkv.weight"], want)
    want = torch.cat([raw["model.layers.0.mlp.gate_proj.weight"], raw["model.layers.0.mlp.up_proj.weight"]])
    assert torch.equal(w["layers.0.ffn.gate_up.weight"], want)
    assert w["layers.0.mixer.qkv.weight"].dtype == torch.bfloat16
    w32 = load_weights(m, d, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["embedding.weight"], raw["model.embed_tokens.weight"].float())
    tied = tiny.CONFIGS[name]["tie_word_embeddings"]
    assert ("lm_head.weight" in w) == (not tied) and ("lm_head.weight" in raw) == (not tied)


def test_same_seed_same_weights(tmp_path):
    cfg = load_model_config_from("A")
    write_random_model(str(tmp_path / "x"), cfg, 5)
    write_random_model(str(tmp_path / "y"), cfg, 5)
    write_random_model(str(tmp_path / "z"), cfg, 6)
    x, y, z = (load_file(str(tmp_path / n / "model.safetensors")) for n in "xyz")
    assert all(torch.equal(x[k], y[k]) for k in x)
    assert any(not torch.equal(x[k], z[k]) for k in x)
    e = x["model.embed_tokens.weight"].float()
    assert abs(e.std().item() - 0.02) < 0.002
    n = x["model.norm.weight"].float()
    assert 0.8 <= n.min() and n.max() <= 1.2


def load_model_config_from(name):
    from atom_b200.config import config_from_dict
    return config_from_dict(tiny.CONFIGS[name])


def test_vector_stored_in_32_bit_stays_32_bit(model_dirs, tmp_path):
    d = str(tmp_path)
    raw = load_file(os.path.join(model_dirs["A"], "model.safetensors"))
    raw["model.norm.weight"] = raw["model.norm.weight"].float()
    save_file(raw, os.path.join(d, "model.safetensors"))
    os.link(os.path.join(model_dirs["A"], "config.json"), os.path.join(d, "config.json"))
    w = load_weights(_model(d), d, torch.bfloat16, "cpu")
    assert w["final_norm.weight"].dtype == torch.float32
    assert w["layers.0.mixer_norm.weight"].dtype == torch.bfloat16
    assert w["layers.0.mixer.qkv.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_dirs, tmp_path):
    d = str(tmp_path)
    raw = load_file(os.path.join(model_dirs["B"], "model.safetensors"))
    del raw["model.layers.1.mlp.up_proj.weight"]
    del raw["lm_head.weight"]
    raw["model.layers.7.extra.weight"] = torch.zeros(3)
    raw["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(5, 7, dtype=torch.bfloat16)
    raw["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(4)   # ignored, not reported
    save_file(raw, os.path.join(d, "model.safetensors"))
    os.link(os.path.join(model_dirs["B"], "config.json"), os.path.join(d, "config.json"))
    with pytest.raises(WeightError) as e:
        load_weights(_model(d), d, torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert len(err.wrong_shape) == 1 and "k_proj" in err.wrong_shape[0] and "[5, 7]" in err.wrong_shape[0]
    msg = str(err)
    assert "missing" in msg and "unexpected" in msg and "wrong shapes" in msg and "inv_freq" not in msg


def test_tied_model_refuses_a_separate_head(model_dirs, tmp_path):
    d = str(tmp_path)
    raw = load_file(os.path.join(model_dirs["A"], "model.safetensors"))
    raw["lm_head.weight"] = raw["model.embed_tokens.weight"].clone()
    save_file(raw, os.path.join(d, "model.safetensors"))
    os.link(os.path.join(model_dirs["A"], "config.json"), os.path.join(d, "config.json"))
    with pytest.raises(WeightError) as e:
        load_weights(_model(d), d, torch.bfloat16, "cpu")
    assert e.value.unexpected == ["lm_head.weight"]


def test_missing_shard_named_by_index(model_dirs, tmp_path):
    import json
    d = str(tmp_path)
    os.link(os.path.join(model_dirs["A"], "config.json"), os.path.join(d, "config.json"))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {"a": "model-00001-of-00002.safetensors"}}, f)
    with pytest.raises(FileNotFoundError):
        load_weights(_model(d), d, torch.bfloat16, "cpu")
