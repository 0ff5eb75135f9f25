"""Configuration: every key comes from config.json; bad files are refused with the key named."""
import copy
import json

import pytest

import tiny
from atom_b200.config import ConfigError, config_from_dict, load_model_config, save_model_config
from atom_b200.models import build_model_spec, registered_architectures


def test_registry_knows_qwen3():
    assert "Qwen3ForCausalLM" in registered_architectures()


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_roundtrip_and_spec(name, tmp_path):
    raw = tiny.CONFIGS[name]
    cfg = config_from_dict(raw)
    for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
              "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
        assert getattr(cfg, k) == raw[k]
    save_model_config(cfg, str(tmp_path))
    again = load_model_config(str(tmp_path))
    assert again == cfg
    spec = build_model_spec(cfg)
    assert len(spec.layers) == raw["num_hidden_layers"]
    assert [e.layer for e in spec.run_order] == list(range(raw["num_hidden_layers"]))
    for i, layer in enumerate(spec.layers):
        a = layer.parts["mixer"].args
        assert (a["num_heads"], a["num_kv_heads"], a["head_dim"]) == (
            raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"])
        assert a["norm_eps"] == raw["rms_norm_eps"] and a["position"].args["theta"] == raw["rope_theta"]
        want_window = raw["sliding_window"] if raw.get("layer_types", ["full_attention"] * 99)[i] == "sliding_attention" else None
        assert a["window"] == want_window
        assert layer.parts["ffn"].args["intermediate_size"] == raw["intermediate_size"]
    assert spec.lm_head.args["tied"] == raw["tie_word_embeddings"]


def test_head_dim_default_is_hidden_over_heads():
    raw = copy.deepcopy(tiny.CONFIGS["A"])
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == raw["hidden_size"] // raw["num_attention_heads"]


def test_rope_parameters_block():
    raw = copy.deepcopy(tiny.CONFIGS["A"])
    del raw["rope_theta"]
    raw["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert config_from_dict(raw).rope_theta == 12345.0


@pytest.mark.parametrize("mutate,needle", [
    (lambda d: d.pop("hidden_size"), "hidden_size"),
    (lambda d: d.pop("rms_norm_eps"), "rms_norm_eps"),
    (lambda d: d.pop("rope_theta"), "rope_theta"),
    (lambda d: d.pop("tie_word_embeddings"), "tie_word_embeddings"),
    (lambda d: d.update(architectures=["NoSuchModel"]), "NoSuchModel"),
    (lambda d: d.update(hidden_act="gelu"), "hidden_act"),
    (lambda d: d.update(num_key_value_heads=3), "num_key_value_heads"),
    (lambda d: d.update(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope_scaling"),
    (lambda d: d.update(vocab_size="many"), "vocab_size"),
    (lambda d: d.update(num_hidden_layers=0), "num_hidden_layers"),
    (lambda d: d.update(layer_types=["full_attention"]), "layer_types"),
    (lambda d: d.update(layer_types=["sliding_attention", "full_attention"]), "sliding_window"),
    # the older spelling of a window (from layer max_window_layers on) is refused, not run as full attention
    (lambda d: d.update(use_sliding_window=True, sliding_window=32, max_window_layers=1), "layer_types"),
])
def test_bad_config_names_the_key(mutate, needle):
    raw = copy.deepcopy(tiny.CONFIGS["A"])
    mutate(raw)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert needle in str(e.value)


def test_window_keys_without_effect_are_taken():
    """use_sliding_window false (or no window at all) beside max_window_layers: full attention, as written."""
    raw = copy.deepcopy(tiny.CONFIGS["A"])
    raw.update(use_sliding_window=False, sliding_window=32, max_window_layers=1)
    cfg = config_from_dict(raw)
    assert cfg.sliding_window is None and cfg.layer_types is None
    raw.update(use_sliding_window=True, sliding_window=None)
    assert config_from_dict(raw).sliding_window is None


def test_missing_file(tmp_path):
    with pytest.raises(ConfigError):
        load_model_config(str(tmp_path))


def test_engine_config_checks():
    from atom_b200.config import EngineConfig

    assert EngineConfig(dtype="bf16").dtype == "bfloat16" and EngineConfig(dtype="fp32").dtype == "float32"
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(kv_cache_block_size=0)


def test_cli_flags_follow_the_reference():
    import argparse
    from atom_b200.engine.arg_utils import EngineArgs

    p = EngineArgs.add_cli_args(argparse.ArgumentParser())
    a = p.parse_args(["--model", "m", "--block-size", "8", "--max-num-batched-tokens", "64", "--max-num-seqs", "3",
                      "--enforce-eager", "--gpu-memory-utilization", "0.5", "--max-model-len", "100",
                      "--no-enable_chunked_prefill", "--load_dummy"])
    e = EngineArgs.from_cli_args(a)
    kw = e._engine_kwargs()
    assert kw["kv_cache_block_size"] == 8 and kw["max_num_batched_tokens"] == 64 and kw["max_num_seqs"] == 3
    assert kw["enforce_eager"] and kw["gpu_memory_utilization"] == 0.5 and kw["max_model_len"] == 100
    assert kw["enable_chunked_prefill"] is False and kw["load_dummy"] == "random"
