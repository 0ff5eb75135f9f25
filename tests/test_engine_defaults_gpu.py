"""The engine as a user gets it when they give nothing but a model folder: the cache sized from the
memory that is left, ``max_num_seqs`` and ``max_model_len`` at their defaults, graphs captured at
start.  Also options that no other test turns: portions off, two engines in one process."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu


def _plain(model_dir):
    return plain.read_config(model_dir), plain.read_tensors(model_dir)


def _margin_check(cfg, w, prompt, out_ids, margin):
    full = list(prompt) + list(out_ids)
    logits = plain.forward(cfg, w, full[:-1]).numpy()
    for i, tok in enumerate(out_ids):
        row = logits[len(prompt) - 1 + i]
        assert row[tok] >= row.max() - margin * abs(row).max(), f"token {i}: logit {row[tok]:.4f} vs max {row.max():.4f}"


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16"), ("C", "bfloat16")])
def test_default_engine_sizes_its_cache_and_stays_within_its_share(model_dirs, name, dtype):
    """No ``num_kvcache_blocks``, no ``max_num_seqs``, no ``max_model_len``: the pool comes from a
    measured warm-up step and a bound on what the graphs take, the graphs are captured after it, and
    when all is set up the process holds no more of the device than ``gpu_memory_utilization``."""
    from atom_b200 import LLMEngine, SamplingParams

    torch.cuda.empty_cache()
    free, total = torch.cuda.mem_get_info()
    share = (total - free + (3 << 30)) / total          # what is in use already, and 3 GiB for this engine
    assert share < 0.95, "the device is too full for this test"
    eng = LLMEngine(model_dirs[name], dtype=dtype, gpu_memory_utilization=share)
    r = eng.runner
    assert r.cfg.num_kvcache_blocks == -1 and r.cfg.max_num_seqs == 512
    assert r.max_model_len == tiny.CONFIGS[name]["max_position_embeddings"]
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert total - free_after <= share * total, (r.memory, total - free_after, share * total)
    # the pool took most of the share: what the graphs really took stayed within what was set aside
    assert r.memory["graphs"] <= r.memory["graph_reserve"], r.memory
    assert r.memory["cache"] >= 0.5 * (3 << 30) - r.memory["graph_reserve"], r.memory
    assert 512 in r.graph_shapes and 1 in r.graph_shapes and any(isinstance(k, tuple) for k in r.graph_shapes)
    # and it generates what the plain implementation does
    cfg, w = _plain(model_dirs[name])
    prompts = tiny.prompts(name, [5, 40, 90, 1, 17], seed=31)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        if dtype == "float32":
            assert o["token_ids"] == plain.generate_greedy(cfg, w, p, 10)
        else:
            _margin_check(cfg, w, p, o["token_ids"], 0.08)
    assert eng.runner.graph_replays > 0
    assert all(g.pool.num_used == 0 for g in r.cache.groups)
    r.cache.check()
    del eng, r
    torch.cuda.empty_cache()


def test_step_arrays_do_not_grow_with_max_model_len(model_dirs):
    """A captured decode step copies its small arrays and the live part of its block tables: the same
    bytes whether the engine takes requests of 256 or of 2,048 tokens, and the same tokens."""
    from atom_b200 import LLMEngine, SamplingParams

    name = "B"
    prompts = tiny.prompts(name, [30, 12, 5], seed=6)
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    seen = {}
    for mml in (256, 2048):
        eng = LLMEngine(model_dirs[name], dtype="float32", kv_cache_block_size=8, num_kvcache_blocks=64,
                        max_num_seqs=4, cudagraph_capture_sizes=[1, 2, 4], max_model_len=mml)
        outs = eng.generate(prompts, sp)
        seen[mml] = ([o["token_ids"] for o in outs], eng.runner.h2d_bytes, eng.runner.graph_replays)
    assert seen[256][0] == seen[2048][0]
    assert seen[256][2] == seen[2048][2] > 10
    assert seen[256][1] == seen[2048][1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_follows_the_context_class(model_dirs, dtype):
    """A request that grows from a few tokens past 256 and on to 1,000 replays, at batch 1, the graph of
    its context class (launch plans made for 256 and for 1,024 keys); the logits stay the plain
    implementation's across the change."""
    from atom_b200.config import EngineConfig
    from atom_b200.engine.batch import StepEntry
    from atom_b200.engine.runner import ModelRunner

    name = "D"
    cfg, w = _plain(model_dirs[name])
    toks = tiny.prompts(name, [1020], seed=12)[0]
    ref = plain.forward(cfg, w, toks).numpy()
    runner = ModelRunner(EngineConfig(model=model_dirs[name], dtype=dtype, kv_cache_block_size=16,
                                      num_kvcache_blocks=80, max_num_seqs=2, enforce_eager=False,
                                      cudagraph_capture_sizes=[1], cudagraph_mixed_steps=False))
    scale = float(np.abs(ref).max())
    tol = 1e-4 * max(1.0, scale) if dtype == "float32" else 8e-2 * scale
    done = 0
    for upto, n_decode in ((240, 22), (1000, 12)):
        runner.step([StepEntry("r", toks[done:upto], ())])
        done = upto
        for _ in range(n_decode):
            got = runner.step([StepEntry("r", [toks[done]], (0,))]).cpu().numpy()[0]
            assert np.abs(got - ref[done]).max() <= tol, f"position {done}"
            done += 1
    runner.check_status()
    keys = [k for k in runner._graphs if k[0] == 1]
    if dtype == "bfloat16":                # (the 32-bit attention kernel has no plan that depends on the context)
        assert len(keys) >= 2, keys        # two context classes with plans of their own at batch 1
    assert runner.graph_replays == 34


def test_portions_off_runs_whole_prompts_only(model_dirs):
    """``enable_chunked_prefill=False``: a prompt runs in one step or waits for a step that has room
    for all of it; one that is longer than the token budget is refused with a reason."""
    from atom_b200 import LLMEngine, SamplingParams

    name = "B"
    cfg, w = _plain(model_dirs[name])
    prompts = tiny.prompts(name, [20, 9, 31, 4, 50], seed=14)
    eng = LLMEngine(model_dirs[name], dtype="float32", kv_cache_block_size=8, num_kvcache_blocks=64,
                    max_num_seqs=8, enforce_eager=True, max_num_batched_tokens=40, enable_chunked_prefill=False)
    for p in prompts:
        eng.add_request(p, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    whole = []
    while not eng.is_finished():
        before = {s.seq_id: s.num_computed for s in eng.scheduler.running}
        waiting = {s.seq_id: s.num_tokens for s in eng.scheduler.waiting}
        eng.step()
        for s in eng.scheduler.running:
            if s.seq_id in waiting:                          # admitted in this step: all of it or nothing
                whole.append(s.num_computed >= waiting[s.seq_id])
    assert whole and all(whole)
    outs = [eng._output(eng._seqs[i]) for i in sorted(eng._seqs)]
    assert outs[4]["finish_reason"].startswith("unschedulable") and "max_num_batched_tokens" in outs[4]["finish_reason"]
    for p, o in list(zip(prompts, outs))[:4]:
        assert o["token_ids"] == plain.generate_greedy(cfg, w, p, 6)
    assert all(g.pool.num_used == 0 for g in eng.runner.cache.groups)


def test_second_engine_of_a_process_samples_like_the_first(model_dirs):
    """Request ids, and with them the default random seeds, are counted per engine."""
    from atom_b200 import LLMEngine, SamplingParams

    name = "B"
    prompts = tiny.prompts(name, [7, 19], seed=2)
    sp = SamplingParams(temperature=1.0, max_tokens=12, ignore_eos=True)       # no seed given
    outs = []
    for _ in range(2):
        eng = LLMEngine(model_dirs[name], dtype="float32", kv_cache_block_size=8, num_kvcache_blocks=32,
                        max_num_seqs=4, enforce_eager=True)
        outs.append([o["token_ids"] for o in eng.generate(prompts, sp)])
    assert outs[0] == outs[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preempted_requests_still_match_plain(model_dirs, dtype):
    """A pool of 12 pages for four requests that grow by 40 tokens each: the newest are preempted and
    computed again, and every token is the plain implementation's (in bfloat16: its argmax within
    rounding, teacher-forced)."""
    from atom_b200 import LLMEngine, SamplingParams

    name = "B"
    cfg, w = _plain(model_dirs[name])
    prompts = tiny.prompts(name, [3, 5, 12, 29], seed=3)
    eng = LLMEngine(model_dirs[name], dtype=dtype, kv_cache_block_size=8, num_kvcache_blocks=12,
                    max_num_batched_tokens=24, max_num_seqs=4, cudagraph_capture_sizes=[1, 2, 4], max_model_len=128)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    assert eng.stats()["preemptions"] > 0 and eng.runner.graph_replays > 0
    for p, o in zip(prompts, outs):
        if dtype == "float32":
            assert o["token_ids"] == plain.generate_greedy(cfg, w, p, 40)
        else:
            _margin_check(cfg, w, p, o["token_ids"], 0.08)
    eng.runner.cache.check()
    assert eng.runner.cache.num_free_pages(0) == 12
