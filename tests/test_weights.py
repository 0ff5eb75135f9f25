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


def _with_head(model_dirs, tmp_path, head):
    d = str(tmp_path)
    raw = load_file(os.path.join(model_dirs["A"], "model.safetensors"))
    raw["lm_head.weight"] = head(raw["model.embed_tokens.weight"])
    save_file(raw, os.path.join(d, "model.safetensors"))
    os.link(os.path.join(model_dirs["A"], "config.json"), os.path.join(d, "config.json"))
    return d, raw


def test_tied_model_takes_a_head_that_equals_the_embedding(model_dirs, tmp_path):
    """A tied checkpoint that carries the output matrix as well loads, and uses the embedding table."""
    d, raw = _with_head(model_dirs, tmp_path, lambda e: e.clone())
    w = load_weights(_model(d), d, torch.bfloat16, "cpu")
    assert "lm_head.weight" not in w
    assert torch.equal(w["embedding.weight"], raw["model.embed_tokens.weight"])


def test_tied_model_refuses_a_head_that_differs(model_dirs, tmp_path):
    def other(e):
        e = e.clone()
        e[3, 5] += 1.0
        return e

    d, _ = _with_head(model_dirs, tmp_path, other)
    with pytest.raises(WeightError) as e:
        load_weights(_model(d), d, torch.bfloat16, "cpu")
    assert not e.value.unexpected and len(e.value.wrong_shape) == 1
    assert "lm_head.weight" in e.value.wrong_shape[0] and "model.embed_tokens.weight" in e.value.wrong_shape[0]


def test_untied_model_still_needs_its_own_head(model_dirs):
    m = _model(model_dirs["B"])
    assert m.spec.duplicate_tensors == () and "lm_head.weight" in expected_tensors(m)


def test_cut_off_file_is_named(model_dirs, tmp_path):
    from atom_b200.weights import WeightFileError
    d = str(tmp_path)
    with open(os.path.join(model_dirs["A"], "model.safetensors"), "rb") as f:
        data = f.read()
    with open(os.path.join(d, "model.safetensors"), "wb") as f:
        f.write(data[: len(data) // 2])
    os.link(os.path.join(model_dirs["A"], "config.json"), os.path.join(d, "config.json"))
    with pytest.raises(WeightFileError) as e:
        load_weights(_model(d), d, torch.bfloat16, "cpu")
    assert "model.safetensors" in str(e.value)


def test_after_load_runs_once_per_part_and_changes_nothing(model_dirs):
    """The hook that lets a part lay its tensors out anew is called once for every part after all are
    bound; the built-in parts leave their tensors as loaded."""
    from atom_b200.parts.base import Part, Runtime, Workspace
    d = model_dirs["B"]
    m = _model(d)
    w = load_weights(m, d, torch.bfloat16, "cpu")
    before = {k: v.clone() for k, v in w.items()}
    calls = []
    orig = Part.after_load

    def spy(self):
        assert m.rt is not None and hasattr(m.lm_head, "w_weight")     # everything is bound by now
        calls.append(self)
        return orig(self)

    Part.after_load = spy
    try:
        m.bind(w, Runtime(torch.bfloat16, torch.device("cpu"), Workspace(torch.device("cpu"))))
    finally:
        Part.after_load = orig
    parts = [p for _, p, _ in m.named_parts()]
    assert len(calls) == len(parts) and {id(c) for c in calls} == {id(p) for p in parts}
    assert all(torch.equal(before[k], w[k]) for k in w)


def test_missing_shard_named_by_index(model_dirs, tmp_path):
    import json
    d = str(tmp_path)
    os.link(os.path.join(model_dirs["A"], "config.json"), os.path.join(d, "config.json"))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {"a": "model-00001-of-00002.safetensors"}}, f)
    with pytest.raises(FileNotFoundError):
        load_weights(_model(d), d, torch.bfloat16, "cpu")


def test_parameter_stacked_side_by_side_and_parts_named_by_the_arrangement(tmp_path):
    """A parameter may be several checkpoint tensors side by side (ParamSpec.stack_dim = 1), and a layer's
    parts are those its arrangement declares: the toy architecture of tests/test_parts_gpu.py has four
    norms in a layer, and a layer without a feed-forward."""
    import test_parts_gpu as toys
    from atom_b200.config import config_from_dict
    from atom_b200.parts.spec import LayerSpec

    toys._register_sandwich()
    d = str(tmp_path)
    write_random_model(d, config_from_dict(toys._SANDWICH), seed=1)
    m = _model(d)
    raw = load_file(os.path.join(d, "model.safetensors"))
    w = load_weights(m, d, torch.bfloat16, "cpu")
    assert torch.equal(w["layers.0.mixer.qc.weight"], torch.cat([raw["l0.wq"], raw["l0.wc"]], dim=1))
    assert raw["l0.wq"].shape == (48, 12)
    names = {n for n, _, _ in m.named_parts()}
    assert {"layers.0.pre_mixer", "layers.0.post_mixer", "layers.0.pre_ffn", "layers.0.post_ffn"} <= names
    assert "layers.1.ffn" not in names and "layers.1.post_mixer" in names
    # a wrong width of one of the side-by-side tensors is a shape error that names it
    raw["l0.wc"] = torch.zeros(48, 11, dtype=torch.bfloat16)
    save_file(raw, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_weights(m, d, torch.bfloat16, "cpu")
    assert "l0.wc" in str(e.value) and "[48, 12]" in str(e.value)
    # a layer that lacks a part its arrangement needs, or names one it does not know, is refused
    spec = m.spec
    broken = {k: v for k, v in spec.layers[0].parts.items() if k != "post_mixer"}
    with pytest.raises(ValueError, match="post_mixer"):
        Model(type(spec)(**{**spec.__dict__, "layers": (LayerSpec("toy_sandwich", broken),),
                            "run_order": spec.run_order[:1]}))
    with pytest.raises(ValueError, match="gate_norm"):
        Model(type(spec)(**{**spec.__dict__, "layers": (
            LayerSpec("prenorm", {**spec.layers[0].parts, "gate_norm": spec.final_norm}),),
            "run_order": spec.run_order[:1]}))
