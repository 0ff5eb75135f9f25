"""The engine against the plain implementation, under every way of cutting the work:
each request alone and whole; most of it in one step and the last 32 tokens one by one; in
portions of changing size down to two tokens; and mixed, up to four live requests, with so
few pages that they are used again.  In 32-bit and in bfloat16."""
import numpy as np
import pytest

import tiny
import traces
from replay_util import make_runner, max_err, plain_logits, replay

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 7, 16, 33, 100, 70], "B": [3, 5, 12, 29, 64, 100, 131], "C": [2, 31, 77, 49, 120],
           "D": [4, 70, 150, 33, 200]}
PAGE = {"A": 16, "B": 8, "C": 16, "D": 16}
# 32-bit: the engine and the plain implementation differ by the order of float32 sums only:
# 1e-4 absolute on logits of magnitude ~1.
# bfloat16: activations are rounded to 8 bits of mantissa (relative 2^-9) between kernels.
# Over all positions the error is a fraction of a percent of the logit scale (bound: 1 % rms);
# single positions reach a few percent where a sharpened softmax (scores up to ~16)
# multiplies the rounding of q and k (bound: 8 % of the largest logit).  Faults of the cache
# or the batch are far larger, and the 32-bit runs of the same code catch the small ones.
TOL = {"float32": 1e-4, "bfloat16": 8e-2}
RMS_TOL_BF16 = 1e-2


def _seqs(name):
    ps = tiny.prompts(name, LENGTHS[name], seed={"A": 1, "B": 3, "C": 5, "D": 7}[name])
    return {f"r{i}": p for i, p in enumerate(ps)}


def _tol(dtype, ref):
    scale = max(float(np.abs(r).max()) for r in ref.values())
    return TOL[dtype] * max(1.0, scale) if dtype == "float32" else TOL[dtype] * scale


@pytest.fixture(scope="module")
def runners(model_dirs):
    cache = {}

    def get(name, dtype, max_tokens):
        key = (name, dtype, max_tokens)
        if key not in cache:
            cache[key] = make_runner(model_dirs[name], dtype, max_tokens, PAGE[name])
        return cache[key]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("cut", ["whole", "tail", "ragged", "mixed"])
def test_cut_matches_plain(model_dirs, runners, name, dtype, cut):
    seqs = _seqs(name)
    ref = plain_logits(model_dirs[name], seqs)
    if cut == "whole":
        steps, peak = traces.whole(seqs), 256
    elif cut == "tail":
        steps, peak = traces.tail_by_token(seqs, 32), 256
    elif cut == "ragged":
        steps, peak = traces.ragged(seqs), 256
    else:
        budget = 320 if name != "D" else 512
        steps, peak = traces.mixed(seqs, max_live=4, budget_tokens=budget)
        assert peak <= budget
    runner = runners(name, dtype, peak)
    got = traces.collect(steps, replay(runner, steps))
    err, rid, pos = max_err(got, ref)
    tol = _tol(dtype, ref)
    assert err <= tol, f"{name}/{dtype}/{cut}: max abs error {err:.3e} at {rid}[{pos}] > {tol:.3e}"
    if dtype == "bfloat16":
        scale = max(float(np.abs(r).max()) for r in ref.values())
        for r in ref:
            rms = float(np.sqrt(((got[r] - ref[r]) ** 2).mean()))
            assert rms <= RMS_TOL_BF16 * scale, f"{name}/{cut}: rms error {rms:.3e} in {r}"
    # every page and slot is back
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)
    if dtype == "float32":
        for r in ref:
            assert (got[r].argmax(1) == ref[r].argmax(1)).all(), f"{name}/{cut}: greedy token differs in {r}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_request_freed_and_fed_again_matches_plain(model_dirs, runners, name, dtype):
    """Two of the live requests are ended half-way, so that their pages go back while the others go on,
    and fed again from their first token under the same id (what preemption by recomputation does).
    Every row of both passes is the plain implementation's."""
    seqs = _seqs(name)
    ref = plain_logits(model_dirs[name], seqs)
    ids = list(seqs)
    budget = 320 if name != "D" else 512
    steps, peak = traces.mixed_refeed(seqs, [ids[-1], ids[-3]], max_live=4, budget_tokens=budget)
    assert peak <= budget
    runner = runners(name, dtype, peak)
    rows = traces.collect_rows(steps, replay(runner, steps))
    tol = _tol(dtype, ref)
    for rid, got in rows.items():
        assert {p for p, _ in got} == set(range(len(seqs[rid])))
        assert len(got) > len(seqs[rid]) or rid not in (ids[-1], ids[-3])     # the victims ran twice in part
        for p, row in got:
            assert np.isfinite(row).all()
            err = float(np.abs(row.astype(np.float64) - ref[rid][p]).max())
            assert err <= tol, f"{name}/{dtype}: {rid}[{p}] off by {err:.3e} > {tol:.3e}"
            if dtype == "float32":
                assert row.argmax() == ref[rid][p].argmax()
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_gated_product_of_portions_on_the_tcgen05_kernel_matches_plain(model_dirs, name):
    """Long portions run their gated product on the kernel with two CTAs to a tile (from a thousand rows on by
    itself).  Forced for every portion of more than 16 rows, whole prompts, portions of changing size and the
    mixed trace give the plain implementation's logits on every configuration (widths that end inside a block
    of 64, outputs that end inside a tile), and the kernel did run."""
    from atom_b200 import native
    from atom_b200.parts import linear

    seqs = _seqs(name)
    ref = plain_logits(model_dirs[name], seqs)
    saved = (linear.PAIRS_MIN_ROWS, linear.PAIRS_MIN_FILL)
    calls = [0]
    real = native.gemm_pairs

    def counted(*args, **kwargs):
        calls[0] += 1
        return real(*args, **kwargs)

    try:
        linear.PAIRS_MIN_ROWS, linear.PAIRS_MIN_FILL = 17, 0.0
        native.gemm_pairs = counted
        runner = make_runner(model_dirs[name], "bfloat16", 512, PAGE[name])
        for steps in (traces.whole(seqs), traces.ragged(seqs), traces.mixed(seqs, max_live=4, budget_tokens=512)[0]):
            got = traces.collect(steps, replay(runner, steps))
            err, rid, pos = max_err(got, ref)
            tol = _tol("bfloat16", ref)
            assert err <= tol, f"{name}: max abs error {err:.3e} at {rid}[{pos}] > {tol:.3e}"
            scale = max(float(np.abs(r).max()) for r in ref.values())
            for r in ref:
                rms = float(np.sqrt(((got[r] - ref[r]) ** 2).mean()))
                assert rms <= RMS_TOL_BF16 * scale, f"{name}: rms error {rms:.3e} in {r}"
        assert calls[0] > 0, "no portion ran on the kernel"
        assert all(g.pool.num_used == 0 for g in runner.cache.groups)
    finally:
        native.gemm_pairs = real
        linear.PAIRS_MIN_ROWS, linear.PAIRS_MIN_FILL = saved


@pytest.mark.parametrize("name", ["A", "D"])
@pytest.mark.parametrize("side", ["norms folded into the products", "norms as kernels of their own",
                                  "the library's product", "rotation as a kernel of its own"])
def test_both_sides_of_the_decode_products_match_plain(model_dirs, name, side):
    """Steps of few rows choose between products by themselves: the weight-streaming kernel with the norms
    folded into its epilogues, the same with the norm kernels, the library; and decode steps leave the heads'
    norm, the rotation and the cache write to the attention kernel where it takes them (D), or not.  Each side, forced, gives the plain implementation's logits when the last 32 tokens are
    decoded one by one and when portions are mixed with decoded tokens (A and D have widths that every
    side takes); with the norms folded, fewer kernels are launched."""
    from atom_b200 import native
    from atom_b200.parts import linear

    seqs = _seqs(name)
    ref = plain_logits(model_dirs[name], seqs)
    saved = (linear.FOLD_NORMS, native.ROWS_M, native.ROTATE_IN_DECODE)
    try:
        linear.FOLD_NORMS = side in ("norms folded into the products", "rotation as a kernel of its own")
        native.ROTATE_IN_DECODE = side != "rotation as a kernel of its own"
        if side == "the library's product":
            native.ROWS_M = 0
        runner = make_runner(model_dirs[name], "bfloat16", 512, PAGE[name])
        before = native.launches
        for steps in (traces.tail_by_token(seqs, 32), traces.mixed(seqs, max_live=4, budget_tokens=512)[0]):
            got = traces.collect(steps, replay(runner, steps))
            err, rid, pos = max_err(got, ref)
            tol = _tol("bfloat16", ref)
            assert err <= tol, f"{name}/{side}: max abs error {err:.3e} at {rid}[{pos}] > {tol:.3e}"
            scale = max(float(np.abs(r).max()) for r in ref.values())
            for r in ref:
                rms = float(np.sqrt(((got[r] - ref[r]) ** 2).mean()))
                assert rms <= RMS_TOL_BF16 * scale, f"{name}/{side}: rms error {rms:.3e} in {r}"
        _launches[(name, side)] = native.launches - before
        assert all(g.pool.num_used == 0 for g in runner.cache.groups)
    finally:
        linear.FOLD_NORMS, native.ROWS_M, native.ROTATE_IN_DECODE = saved
    a, b = _launches.get((name, "norms folded into the products")), _launches.get((name, "norms as kernels of their own"))
    if a is not None and b is not None:
        assert a < b, "folding the norms saved no launch"
    c = _launches.get((name, "rotation as a kernel of its own"))
    if name == "D" and a is not None and c is not None:
        assert a < c, "the decode steps of D did not rotate inside the attention kernel"


@pytest.mark.parametrize("name", ["A", "D"])
@pytest.mark.parametrize("live", [9, 13, 16])
def test_nine_to_sixteen_requests_decode_side_by_side(model_dirs, name, live):
    """Steps of 9 to 16 single tokens take the streaming product's second token tile (with the norms in its
    epilogues) where the widths allow it: every request's prompt in one step, then all of them decoded token
    by token in the same steps, against the plain implementation."""
    lengths = [20 + 3 * i for i in range(live)]
    ps = tiny.prompts(name, lengths, seed=11)
    seqs = {f"q{i}": p for i, p in enumerate(ps)}
    ref = plain_logits(model_dirs[name], seqs)
    tail = 6
    steps = []
    for rid, toks in seqs.items():
        n = len(toks) - tail
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks[:n]), "want": list(range(n))}], "end": []})
    for k in range(tail):
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": rid, "tokens": [toks[len(toks) - tail + k]], "want": [0]} for rid, toks in seqs.items()]})
    steps[-1]["end"] = list(seqs)
    runner = make_runner(model_dirs[name], "bfloat16", 64 * live, PAGE[name], max_num_seqs=16)
    got = traces.collect(steps, replay(runner, steps))
    err, rid, pos = max_err(got, ref)
    tol = _tol("bfloat16", ref)
    assert err <= tol, f"{name}/{live}: max abs error {err:.3e} at {rid}[{pos}] > {tol:.3e}"
    scale = max(float(np.abs(r).max()) for r in ref.values())
    for r in ref:
        rms = float(np.sqrt(((got[r] - ref[r]) ** 2).mean()))
        assert rms <= RMS_TOL_BF16 * scale, f"{name}/{live}: rms error {rms:.3e} in {r}"
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


@pytest.mark.parametrize("page", [8, 32, 128])
def test_other_page_sizes_on_the_tma_kernels(model_dirs, page):
    """Head size 128 with pages of 8, 32 and 128 tokens (boxes of a page, or pieces of a larger one): the last
    32 tokens one by one (rotation and cache write inside the decode kernel) and mixed steps, in bfloat16."""
    name = "D"
    seqs = _seqs(name)
    ref = plain_logits(model_dirs[name], seqs)
    runner = make_runner(model_dirs[name], "bfloat16", 2048, page)
    for steps in (traces.tail_by_token(seqs, 32), traces.mixed(seqs, max_live=4, budget_tokens=2048, page=page)[0]):
        got = traces.collect(steps, replay(runner, steps))
        err, rid, pos = max_err(got, ref)
        tol = _tol("bfloat16", ref)
        assert err <= tol, f"page {page}: max abs error {err:.3e} at {rid}[{pos}] > {tol:.3e}"
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


_launches = {}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_reuses_pages(model_dirs, runners, dtype):
    """With a pool this small the later requests must run on pages the earlier ones freed."""
    name = "B"
    seqs = _seqs(name)
    steps, peak = traces.mixed(seqs, max_live=4, budget_tokens=320)
    total = sum(-(-len(t) // 64) * 64 for t in seqs.values())
    assert peak < total, "the trace does not force re-use"
    runner = runners(name, dtype, peak)
    seen, reused = set(), False
    from atom_b200.engine.batch import StepEntry
    for s in steps:
        runner.step([StepEntry(e["id"], e["tokens"], ()) for e in s["entries"]])
        for rid in s["end"]:
            before = set(runner.cache.table(rid, 0))
            runner.finish(rid)
            seen |= {p for p in before if p >= 0}
        now = {p for rc in runner.cache.requests.values() for p in rc.tables[0] if p >= 0}
        reused = reused or bool(now & seen)
    runner.check_status()
    assert reused


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C", "D"])
def test_captured_decode_steps_match_plain(model_dirs, name, dtype):
    """Decode steps replayed from CUDA graphs (batch sizes 1, 2 and 4, the last with padding
    rows when three requests are live) give the logits of the plain implementation."""
    from atom_b200.config import EngineConfig
    from atom_b200.engine.runner import ModelRunner

    seqs = _seqs(name)
    ref = plain_logits(model_dirs[name], seqs)
    cfg = EngineConfig(model=model_dirs[name], dtype=dtype, kv_cache_block_size=PAGE[name],
                       num_kvcache_blocks=64, max_num_seqs=8, enforce_eager=False,
                       cudagraph_capture_sizes=[1, 2, 4], max_model_len=256)
    runner = ModelRunner(cfg)
    for steps in (traces.tail_by_token(seqs, 32), traces.mixed(seqs, max_live=3, tail=40)[0]):
        got = traces.collect(steps, replay(runner, steps))
        err, rid, pos = max_err(got, ref)
        tol = _tol(dtype, ref)
        assert err <= tol, f"{name}/{dtype}: max abs error {err:.3e} at {rid}[{pos}] > {tol:.3e}"
    assert runner.graph_replays > 50 and runner.graph_shapes >= {1, 4}
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_small_steps_of_any_makeup_replay_graphs_and_match_plain(model_dirs, name, dtype):
    """Steps with prompt portions (beside decoded tokens or not) of up to 128 tokens replay a graph
    recorded for their shape rounded up, whose launch plans hold for every batch of that shape: in
    portions of changing size and mixed, with every row's logits wanted, the logits are the plain
    implementation's."""
    from atom_b200.config import EngineConfig
    from atom_b200.engine.runner import ModelRunner

    seqs = _seqs(name)
    ref = plain_logits(model_dirs[name], seqs)
    cfg = EngineConfig(model=model_dirs[name], dtype=dtype, kv_cache_block_size=PAGE[name],
                       num_kvcache_blocks=96, max_num_seqs=8, enforce_eager=False,
                       cudagraph_capture_sizes=[1, 2, 4], max_model_len=256)
    runner = ModelRunner(cfg)
    for steps in (traces.ragged(seqs), traces.mixed(seqs, max_live=4)[0], traces.tail_by_token(seqs, 32)):
        got = traces.collect(steps, replay(runner, steps))
        err, rid, pos = max_err(got, ref)
        tol = _tol(dtype, ref)
        assert err <= tol, f"{name}/{dtype}: max abs error {err:.3e} at {rid}[{pos}] > {tol:.3e}"
    shapes = [k for k in runner.graph_shapes if isinstance(k, tuple)]
    assert len(shapes) >= 2 and runner.graph_replays > 60, (shapes, runner.graph_replays)
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)
    # the same steps with the option off run eagerly
    off = ModelRunner(EngineConfig(model=model_dirs[name], dtype=dtype, kv_cache_block_size=PAGE[name],
                                   num_kvcache_blocks=96, max_num_seqs=8, enforce_eager=False,
                                   cudagraph_capture_sizes=[1, 2, 4], max_model_len=256, cudagraph_mixed_steps=False))
    steps = traces.ragged(seqs)
    replay(off, steps)
    assert not [k for k in off.graph_shapes if isinstance(k, tuple)]
