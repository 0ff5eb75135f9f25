"""Tiny configurations of the architecture, differing in every size and option, and helpers
that write them as model folders with seeded random weights."""
from __future__ import annotations

import os
import zlib
from typing import Dict, List

import numpy as np
import torch

# A and B are the two acceptance configurations; C adds what Qwen3 checkpoints may carry
# and A/B lack: sliding-window layers, projection biases, as many kv heads as heads, a head
# size that is no power of two.  D has the head size of the large models (128), so that whole
# requests run through the kernels made for it (tensor-memory prefill, TMA decode).
CONFIGS: Dict[str, dict] = {
    "A": dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64,
        num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128,
        vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
        max_position_embeddings=1024, hidden_act="silu", attention_bias=False,
    ),
    "B": dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96,
        num_attention_heads=8, num_key_value_heads=2, head_dim=32, intermediate_size=160,
        vocab_size=389, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
        max_position_embeddings=2048, hidden_act="silu", attention_bias=False,
    ),
    "C": dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=4, hidden_size=80,
        num_attention_heads=5, num_key_value_heads=5, head_dim=48, intermediate_size=112,
        vocab_size=301, rope_theta=500000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
        max_position_embeddings=768, hidden_act="silu", attention_bias=True,
        sliding_window=24, use_sliding_window=True,
        layer_types=["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
    ),
    "D": dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=192,
        num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=320,
        vocab_size=517, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
        max_position_embeddings=1024, hidden_act="silu", attention_bias=False,
    ),
}
SEEDS = {"A": 0, "B": 2, "C": 11, "D": 13}
# Factor on the per-head q/k norm weights: sharpens the attention so that a wrong or missing
# key changes the output visibly instead of drowning in a near-uniform average.
QK_SHARPEN = {"A": 1.0, "B": 2.0, "C": 1.5, "D": 1.2}


def write_model(name: str, model_dir: str) -> None:
    from atom_b200.config import config_from_dict
    from atom_b200.weights import write_random_model
    from safetensors.torch import load_file, save_file

    cfg = config_from_dict(CONFIGS[name])
    write_random_model(model_dir, cfg, SEEDS[name])
    path = os.path.join(model_dir, "model.safetensors")
    t = load_file(path)
    f = QK_SHARPEN[name]
    for k in list(t):
        if k.endswith("q_norm.weight") or k.endswith("k_norm.weight"):
            t[k] = (t[k].float() * f).to(t[k].dtype)
        if k.endswith("_proj.bias"):
            g = torch.Generator().manual_seed(zlib.crc32(k.encode()))
            t[k] = (torch.randn(t[k].shape, generator=g) * 0.02).to(t[k].dtype)
    save_file(t, path, metadata={"format": "pt"})


def prompts(name: str, lengths: List[int], seed: int) -> List[List[int]]:
    rng = np.random.default_rng(seed)
    V = CONFIGS[name]["vocab_size"]
    return [rng.integers(0, V, size=n).tolist() for n in lengths]
