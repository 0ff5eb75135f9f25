"""What the engine does with a step it cannot run, and with a fault that a kernel reports.  Every
failure here is made on the host (a bad batch, a pool that is too small, a flag set by the test, a
block table that lacks a page which the kernel is written to skip); none faults the device."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu


def _runner(model_dir, dtype="float32", pages=8, page=8, **kw):
    from atom_b200.config import EngineConfig
    from atom_b200.engine.runner import ModelRunner

    kw.setdefault("enforce_eager", True)
    return ModelRunner(EngineConfig(model=model_dir, dtype=dtype, kv_cache_block_size=page,
                                    num_kvcache_blocks=pages, max_num_seqs=4, **kw))


def _snapshot(runner):
    c = runner.cache
    return ({rid: (rc.committed, {g: list(t) for g, t in rc.tables.items()}) for rid, rc in c.requests.items()},
            [g.pool.num_free for g in c.groups], c.state_slots.num_free)


@pytest.mark.parametrize("bad,needle", [
    (lambda E: [E("a", [1, 2], ()), E("a", [3], ())], "twice"),
    (lambda E: [E("n", [], ())], "no tokens"),
    (lambda E: [E("n", [1, 2, 3], (3,))], "wanted place"),
    (lambda E: [E("n", [1, 2, 3], (-1,))], "wanted place"),
    (lambda E: [E("n", [1, 389, 3], ())], "token id"),
    (lambda E: [E("n", [-1], ())], "token id"),
    (lambda E: [E("n", list(range(1, 60)), ())], "max_model_len"),
    (lambda E: [E("a", [4] * 50, ())], "max_model_len"),          # a known request that would outgrow it
])
def test_a_refused_step_leaves_the_cache_as_it_was(model_dirs, bad, needle):
    from atom_b200.engine.batch import StepEntry, StepError

    runner = _runner(model_dirs["B"], max_model_len=48, pages=16)
    first = runner.step([StepEntry("a", [5, 6, 7], (2,))]).cpu()
    before = _snapshot(runner)
    with pytest.raises(StepError) as e:
        runner.step(bad(StepEntry))
    assert needle in str(e.value)
    assert _snapshot(runner) == before
    runner.cache.check()
    # and the engine goes on: the same request continues, with the logits of the plain implementation
    cfg, w = plain.read_config(model_dirs["B"]), plain.read_tensors(model_dirs["B"])
    got = runner.step([StepEntry("a", [8, 9], (0, 1))]).cpu().numpy()
    ref = plain.forward(cfg, w, [5, 6, 7, 8, 9]).numpy()
    assert np.abs(first.numpy()[0] - ref[2]).max() < 1e-4 and np.abs(got - ref[3:5]).max() < 1e-4
    runner.check_status()


def test_device_tokens_are_refused_outside_a_captured_decode_step(model_dirs):
    from atom_b200.engine.batch import StepEntry, StepError

    runner = _runner(model_dirs["B"], enforce_eager=False, cudagraph_capture_sizes=[1, 2], pages=16)
    runner.step([StepEntry("a", [5, 6, 7], ()), StepEntry("b", [1], ())])
    before = _snapshot(runner)
    dev = torch.zeros(2, dtype=torch.int32, device="cuda:0")
    for entries, toks, rows in (
            ([StepEntry("a", [0, 0], (1,)), StepEntry("b", [0], (0,))], dev, None),         # not one token each
            ([StepEntry("a", [0], (0,)), StepEntry("b", [0], (0,))], dev[:1], None),        # one token short
            ([StepEntry("a", [0], (0,)), StepEntry("b", [0], (0,))], dev.long(), None),     # not int32
            ([StepEntry("a", [0], (0,)), StepEntry("b", [0], (0,))], dev, [0, 2])):         # a row beyond the source
        with pytest.raises(StepError):
            runner.step(entries, device_tokens=toks, device_token_rows=rows)
        assert _snapshot(runner) == before


def test_out_of_pages_changes_nothing(model_dirs):
    """A step that does not fit raises OutOfPages before a page is taken or a request admitted."""
    from atom_b200.cache import OutOfPages
    from atom_b200.engine.batch import StepEntry

    runner = _runner(model_dirs["B"], pages=4, page=8)
    runner.step([StepEntry("a", list(range(1, 18)), ())])          # 3 of 4 pages
    before = _snapshot(runner)
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("a", [3], ()), StepEntry("b", list(range(1, 11)), ())])     # b needs 2 pages
    assert _snapshot(runner) == before
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("a", list(range(1, 18)), ())])      # a alone would need 5 pages
    assert _snapshot(runner) == before
    runner.finish("a")
    for i in range(4):
        runner.step([StepEntry(f"s{i}", [1], ())])
    full = _snapshot(runner)
    with pytest.raises(OutOfPages) as e:                           # no request slot left (max_num_seqs 4)
        runner.step([StepEntry("one-more", [1], ())])
    assert "request slots" in str(e.value) and _snapshot(runner) == full
    runner.cache.check()
    for rid in list(runner.cache.requests):
        runner.finish(rid)
    assert runner.cache.num_free_pages(0) == 4 and runner.cache.state_slots.num_free == 4
    runner.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kernel_reports_a_position_without_a_page(dtype):
    """The cache-write kernel is handed a block table that has no page where a token has to be written:
    it skips that write, sets the status word, and writes every other token.  The host's check then
    raises once, and the word is clear again."""
    from atom_b200 import native
    from atom_b200.engine.batch import StepError  # noqa: F401  (the runner turns NativeError into it)

    dev = torch.device("cuda:0")
    nh, nkv, hd, page, T = 4, 2, 32, 8, 12
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=dev).to(dtype)
    kp = torch.zeros(4, nkv, page, hd, device=dev, dtype=dtype)
    vp = torch.zeros_like(kp)
    bt = torch.tensor([[2, -1, 0, 0]], dtype=torch.int32, device=dev)          # positions 8..15 have no page
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    sot = torch.zeros(T, dtype=torch.int32, device=dev)
    native.check_error_flags()
    status = native.status_flag(dev)
    native.qknorm_rope_kvwrite(qkv, nh, nkv, hd, None, None, 1e-6, None, 0, pos, sot, bt, page, kp, vp, status)
    with pytest.raises(native.NativeError) as e:
        native.check_error_flags()
    assert "without a cache page" in str(e.value)
    native.check_error_flags()                                                  # cleared by the raise
    v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
    assert torch.equal(vp[2], v[:8].permute(1, 0, 2).contiguous())              # the tokens that have a page are there
    assert float(vp[[0, 1, 3]].abs().sum()) == 0 and float(kp[[0, 1, 3]].abs().sum()) == 0


def test_engine_raises_when_a_kernel_flag_is_set_and_goes_on(model_dirs):
    """The fault flags travel to the host with every step's tokens: a set flag ends the step that
    reads it with StepError (in the eager path and in the path that reads a step's tokens one call
    later), is cleared by that, and the engine serves the next requests as before."""
    from atom_b200 import LLMEngine, SamplingParams
    from atom_b200.engine.batch import StepError

    name = "B"
    cfg, w = plain.read_config(model_dirs[name]), plain.read_tensors(model_dirs[name])
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    prompt = tiny.prompts(name, [9], seed=4)[0]
    for eager in (True, False):
        eng = LLMEngine(model_dirs[name], dtype="float32", kv_cache_block_size=8, num_kvcache_blocks=32,
                        max_num_seqs=4, enforce_eager=eager, cudagraph_capture_sizes=[1, 2], max_model_len=64)
        for flag, needle in ((0, "bounded wait"), (1, "without a cache page")):
            eng.add_request(prompt, sp)
            eng.step()                                   # the prompt
            eng.runner.flags[flag] = 1
            with pytest.raises(StepError) as e:
                for _ in range(3):
                    eng.step()
            assert needle in str(e.value)
            assert eng.runner.flags.tolist() == [0, 0]
            # the step's requests ended with reason "fault" and gave everything back
            assert eng.is_finished() and all(g.pool.num_used == 0 for g in eng.runner.cache.groups)
            assert [s.finish_reason for s in eng._seqs.values() if s.is_finished][-1] == "fault"
            out = eng.generate([prompt], sp)[0]
            assert out["token_ids"] == plain.generate_greedy(cfg, w, prompt, 6)
        eng.runner.cache.check()
