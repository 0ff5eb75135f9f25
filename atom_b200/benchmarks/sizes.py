"""Layer sizes of the Qwen3 dense models that the benchmarks run with random weights, and the
seed each is drawn with."""
from __future__ import annotations

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
    max_position_embeddings=40960, hidden_act="silu", attention_bias=False,
)

# name -> (config.json keys, weight seed)
SIZES = {
    "8b": (QWEN3_8B, 4),
    "4b": (dict(QWEN3_8B, hidden_size=2560, intermediate_size=9728, tie_word_embeddings=True), 5),
    "32b": (dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                 intermediate_size=25600), 7),
}
