"""The product path at the layer sizes it is measured at: hidden 4096, 32 heads, 8 kv heads, head
size 128, feed-forward 12288 (two layers, a vocabulary of 32,000 to keep the folder small), against
the plain implementation.  At these sizes a long prompt runs on the tcgen05 attention kernel with
two query tiles per CTA, decoded tokens on the TMA decode attention and on the weight-streaming
product with ranges cut inside slabs, replayed from a CUDA graph with programmatic dependent
launch: none of which the tiny configurations reach."""
import numpy as np
import pytest

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

CONFIG = dict(
    architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=4096, num_attention_heads=32,
    num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=32000, rope_theta=1000000.0,
    rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096, hidden_act="silu",
    attention_bias=False)
PROMPTS = [301, 1, 77, 140]          # lengths: 1,204 packed query rows, a single token, ...
DECODE = 6


@pytest.fixture(scope="module")
def big_model(tmp_path_factory):
    from atom_b200.config import config_from_dict
    from atom_b200.weights import write_random_model

    d = str(tmp_path_factory.mktemp("layer_sizes") / "m")
    write_random_model(d, config_from_dict(CONFIG), seed=4)
    rng = np.random.default_rng(12)
    seqs = [rng.integers(0, CONFIG["vocab_size"], n + DECODE).tolist() for n in PROMPTS]
    cfg, w = plain.read_config(d), plain.read_tensors(d)
    ref = [plain.forward(cfg, w, s).numpy() for s in seqs]
    return d, seqs, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_whole_then_decoded_together(big_model, dtype):
    from atom_b200.config import EngineConfig
    from atom_b200.engine.batch import StepEntry
    from atom_b200.engine.runner import ModelRunner

    d, seqs, ref = big_model
    runner = ModelRunner(EngineConfig(model=d, dtype=dtype, kv_cache_block_size=16, num_kvcache_blocks=96,
                                      max_num_seqs=8, enforce_eager=False, cudagraph_capture_sizes=[1, 2, 4]))
    got = [[] for _ in seqs]
    # the prompts: the long one alone (in two portions, the second continuing a cached prefix), the others together
    n0 = PROMPTS[0]
    got[0].append(runner.step([StepEntry(0, seqs[0][:200], list(range(200)))]).cpu().numpy())
    got[0].append(runner.step([StepEntry(0, seqs[0][200:n0], list(range(n0 - 200)))]).cpu().numpy())
    logits = runner.step([StepEntry(i, seqs[i][:PROMPTS[i]], list(range(PROMPTS[i]))) for i in (1, 2, 3)]).cpu().numpy()
    o = 0
    for i in (1, 2, 3):
        got[i].append(logits[o:o + PROMPTS[i]])
        o += PROMPTS[i]
    # decoded tokens of all four, one step each, from the captured graph
    for k in range(DECODE):
        logits = runner.step([StepEntry(i, [seqs[i][PROMPTS[i] + k]], (0,)) for i in range(4)]).cpu().numpy()
        for i in range(4):
            got[i].append(logits[i:i + 1])
    runner.check_status()
    assert runner.graph_replays >= DECODE
    for i in range(4):
        g, r = np.concatenate(got[i]), ref[i]
        scale = float(np.abs(r).max())
        err = float(np.abs(g - r).max())
        if dtype == "float32":
            assert err <= 2e-4 * max(1.0, scale), f"request {i}: max abs error {err:.2e} (scale {scale:.2f})"
        else:
            rms = float(np.sqrt(np.mean((g - r) ** 2)))
            assert err <= 0.08 * scale and rms <= 0.01 * scale, f"request {i}: max {err:.3f}, rms {rms:.4f}, scale {scale:.2f}"
        # the argmax agrees wherever the plain implementation's lead over the runner-up is clear
        top2 = np.sort(r, axis=-1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > (0.0 if dtype == "float32" else 0.1 * scale)
        assert (g.argmax(-1)[clear] == r.argmax(-1)[clear]).all()
    for i in range(4):
        runner.finish(i)
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


def test_a_portion_long_enough_for_the_gated_product_on_two_ctas_to_a_tile(big_model):
    """From 600 rows on the feed-forward's gated product of a portion runs, by the engine's own rule, on the
    tcgen05 kernel with two CTAs to a tile and the activation in its epilogue: a prompt of 700 tokens in one
    step gives the plain implementation's logits, and the kernel did run."""
    from atom_b200 import native
    from atom_b200.config import EngineConfig
    from atom_b200.engine.batch import StepEntry
    from atom_b200.engine.runner import ModelRunner

    d, _, _ = big_model
    n = 700
    seq = np.random.default_rng(13).integers(0, CONFIG["vocab_size"], n).tolist()
    cfg, w = plain.read_config(d), plain.read_tensors(d)
    r = plain.forward(cfg, w, seq).numpy()
    calls = [0]
    real = native.gemm_pairs

    def counted(*args, **kwargs):
        calls[0] += 1
        return real(*args, **kwargs)

    native.gemm_pairs = counted
    try:
        runner = ModelRunner(EngineConfig(model=d, dtype="bfloat16", kv_cache_block_size=16, num_kvcache_blocks=64,
                                          max_num_seqs=2, max_num_batched_tokens=1024, enforce_eager=True))
        g = runner.step([StepEntry(0, seq, list(range(n)))]).cpu().numpy()
        runner.check_status()
    finally:
        native.gemm_pairs = real
    assert calls[0] == CONFIG["num_hidden_layers"], "the portion's gated products did not run on the kernel"
    scale = float(np.abs(r).max())
    err, rms = float(np.abs(g - r).max()), float(np.sqrt(np.mean((g - r) ** 2)))
    assert err <= 0.08 * scale and rms <= 0.01 * scale, f"max {err:.3f}, rms {rms:.4f}, scale {scale:.2f}"
    top2 = np.sort(r, axis=-1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 0.1 * scale
    assert (g.argmax(-1)[clear] == r.argmax(-1)[clear]).all()
    runner.finish(0)
    assert all(grp.pool.num_used == 0 for grp in runner.cache.groups)
