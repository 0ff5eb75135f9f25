"""The scheduler's decisions on the CPU (no model): budget, portions, decode beside
prefill, first-come-first-served admission, what happens when pages run out, finishing."""
import pytest

from atom_b200.cache import CacheManager
from atom_b200.engine.scheduler import Scheduler
from atom_b200.engine.sequence import Sequence, SequenceStatus
from atom_b200.parts.spec import CacheNeed
from atom_b200.sampling import SamplingParams

FULL = CacheNeed("pages", num_kv_heads=2, head_dim=16)


def make(num_pages=16, page=4, max_seqs=4, budget=64, max_len=64, cap=0, eos=(2,)):
    cache = CacheManager({0: FULL}, page, num_pages, max_seqs)
    return Scheduler(cache, max_seqs, budget, max_len, eos_token_ids=eos, portion_cap=cap), cache


def seq(n, max_tokens=8, sid=None, **kw):
    return Sequence(list(range(3, 3 + n)), SamplingParams(max_tokens=max_tokens, **kw), seq_id=sid)


def run(s, cache, step, tokens=None):
    """Stands in for the model: commits what was scheduled and 'samples' the given tokens."""
    for e in step.entries:
        cache.commit(e.seq.seq_id, e.start + e.num_tokens)
    n = sum(e.samples for e in step.entries)
    fin = s.postprocess(step, tokens if tokens is not None else [7] * n)
    cache.check()
    return fin


def test_prompt_in_portions_under_the_budget():
    s, cache = make(num_pages=64, budget=10, max_len=200)
    a = seq(25, sid=100)
    s.add(a)
    sizes = []
    for _ in range(3):
        st = s.schedule()
        sizes.append([(e.start, e.num_tokens, e.samples) for e in st.entries])
        run(s, cache, st)
    assert sizes == [[(0, 10, False)], [(10, 10, False)], [(20, 5, True)]]
    assert a.num_output_tokens == 1 and a.num_computed == 25
    st = s.schedule()
    assert [(e.start, e.num_tokens, e.samples) for e in st.entries] == [(25, 1, True)]


def test_portion_cap_and_no_alignment():
    s, cache = make(num_pages=64, budget=64, max_len=200, cap=13)
    s.add(seq(30, sid=1))
    st = s.schedule()
    assert [(e.start, e.num_tokens) for e in st.entries] == [(0, 13)]   # 13 is no multiple of the page (4)
    run(s, cache, st)
    st = s.schedule()
    assert [(e.start, e.num_tokens) for e in st.entries] == [(13, 13)]


def test_decode_tokens_ride_beside_prompt_portions():
    s, cache = make(num_pages=64, budget=12, max_len=200)
    a, b = seq(5, sid=1), seq(30, sid=2)
    s.add(a)
    run(s, cache, s.schedule())            # a's prompt, samples its first token
    s.add(b)
    st = s.schedule()
    got = [(e.seq.seq_id, e.start, e.num_tokens, e.samples) for e in st.entries]
    assert got == [(1, 5, 1, True), (2, 0, 11, False)]      # decode first, the rest of the budget to b
    assert st.num_tokens == 12
    run(s, cache, st)
    st = s.schedule()
    got = [(e.seq.seq_id, e.start, e.num_tokens) for e in st.entries]
    assert got == [(1, 6, 1), (2, 11, 11)]


def test_max_num_seqs_and_fifo():
    s, cache = make(num_pages=64, max_seqs=2, budget=64, max_len=200)
    for i in range(3):
        s.add(seq(4, sid=i))
    st = s.schedule()
    assert [e.seq.seq_id for e in st.entries] == [0, 1]
    assert [q.seq_id for q in s.waiting] == [2]


def test_admission_waits_for_pages_first_come_first_served():
    s, cache = make(num_pages=8, page=4, budget=64, max_len=200)
    big, small = seq(20, sid=1), seq(3, sid=2)
    first = seq(14, sid=0)
    s.add(first)
    run(s, cache, s.schedule())            # holds 4 pages
    s.add(big)                             # needs 6 pages: must wait
    s.add(small)                           # would fit, but does not overtake
    st = s.schedule()
    assert [e.seq.seq_id for e in st.entries] == [0]
    assert [q.seq_id for q in s.waiting] == [1, 2]


def test_unschedulable_requests_are_finished_with_a_reason():
    s, cache = make(num_pages=4, page=4, budget=64, max_len=32)
    too_long, too_big, ok = seq(40, sid=1), seq(20, sid=2), seq(5, sid=3)
    for q in (too_long, too_big, ok):
        s.add(q)
    st = s.schedule()
    assert [q.seq_id for q in st.rejected] == [1, 2]
    assert too_long.finish_reason.startswith("unschedulable") and "max_model_len" in too_long.finish_reason
    assert too_big.finish_reason.startswith("unschedulable") and "pages" in too_big.finish_reason
    assert [e.seq.seq_id for e in st.entries] == [3]


def test_pages_run_out_in_decode_newest_is_preempted_and_recomputed():
    s, cache = make(num_pages=4, page=4, budget=64, max_len=64)
    a, b = seq(5, max_tokens=10, sid=1), seq(5, max_tokens=10, sid=2)
    s.add(a)
    s.add(b)
    st = s.schedule()
    assert [e.seq.seq_id for e in st.entries] == [1, 2]     # 2 pages each: the pool is full
    run(s, cache, st)
    for _ in range(3):                     # both decode inside their second page
        st = s.schedule()
        assert not st.preempted and [e.seq.seq_id for e in st.entries] == [1, 2]
        run(s, cache, st)
    assert a.num_tokens == 9 and cache.num_free_pages(0) == 0
    st = s.schedule()                      # a's position 8 needs a third page: b (newest) must go
    assert [q.seq_id for q in st.preempted] == [2]
    assert [e.seq.seq_id for e in st.entries] == [1]
    assert b.status == SequenceStatus.WAITING and b.num_computed == 0 and s.waiting[0] is b
    assert b.num_output_tokens == 4        # what it generated is kept and will be recomputed
    assert s.num_preemptions == 1
    run(s, cache, st)
    # b re-enters only when the pool has room for all it holds; then prompt + generated run as one prompt
    while b.status == SequenceStatus.WAITING:
        st = s.schedule()
        run(s, cache, st)
    e = [e for e in st.entries if e.seq is b][0]
    assert (e.start, e.num_tokens, e.samples) == (0, 9, True)
    assert b.num_output_tokens == 5
    while not s.is_finished():
        run(s, cache, s.schedule())
    assert a.num_output_tokens == 10 and b.num_output_tokens == 10
    assert a.finish_reason == b.finish_reason == "max_tokens"
    assert cache.num_free_pages(0) == 4


def test_newest_in_need_preempts_itself():
    s, cache = make(num_pages=3, page=4, budget=64, max_len=64)
    a, b = seq(2, max_tokens=30, sid=1), seq(7, max_tokens=30, sid=2)
    s.add(a)
    s.add(b)
    run(s, cache, s.schedule())            # a: 1 page, b: 2 pages
    st = s.schedule()
    assert not st.preempted
    run(s, cache, st)                      # a: 4 tokens, b: 9 tokens (8 in the cache)
    st = s.schedule()                      # b's position 8 needs a page, none is free, b is the newest
    assert [q.seq_id for q in st.preempted] == [2]
    assert [e.seq.seq_id for e in st.entries] == [1]
    assert s.waiting[0] is b


def test_stop_rules():
    s, cache = make(num_pages=64, budget=64, max_len=12, eos=(2,), max_seqs=8)
    a = seq(3, max_tokens=3, sid=1)
    b = seq(3, max_tokens=9, sid=2)
    c = seq(3, max_tokens=9, sid=3, ignore_eos=True)
    d = seq(3, max_tokens=9, sid=4, stop_token_ids=[9])
    e = seq(3, max_tokens=50, sid=5, ignore_eos=True)
    for q in (a, b, c, d, e):
        s.add(q)
    fin = run(s, cache, s.schedule(), [5, 2, 2, 9, 5])
    assert {q.seq_id: q.finish_reason for q in fin} == {2: "eos", 4: "stop_9"}
    assert cache.requests.keys() == {1, 3, 5}
    fin = run(s, cache, s.schedule(), [5, 5, 5])
    fin += run(s, cache, s.schedule(), [5, 5, 5])
    assert a.finish_reason == "max_tokens" and a.num_output_tokens == 3
    while not e.is_finished:
        run(s, cache, s.schedule())
    assert e.finish_reason == "max_model_len" and e.num_tokens == 12
    assert c.is_finished and c.finish_reason == "max_tokens"
    assert s.is_finished() and cache.num_free_pages(0) == 64


def test_stop_sequences_and_logprobs():
    """A request ends when its tokens end with one of its stop sequences (checked before EOS, as in
    atom/model_engine/scheduler.py:2298-2316); log-probabilities are kept for the requests that ask."""
    s, cache = make(num_pages=64, budget=64, max_len=40, eos=(2,), max_seqs=8)
    a = Sequence([3, 4, 5], SamplingParams(max_tokens=20, logprobs=True), seq_id=1, stop_token_sequences=[[7, 8, 9], [6]])
    b = Sequence([3, 4, 8], SamplingParams(max_tokens=20), seq_id=2, stop_token_sequences=[[8, 9]])   # may span prompt and output
    c = Sequence([3, 4, 5], SamplingParams(max_tokens=20), seq_id=3, stop_token_sequences=[[9, 2]])
    for q in (a, b, c):
        s.add(q)
    fin = s.postprocess(_commit(cache, s.schedule()), [7, 9, 9], [-0.5, -1.0, -2.0])
    assert [q.seq_id for q in fin] == [2] and b.finish_reason == "stop_sequence" and b.logprobs == []
    fin = s.postprocess(_commit(cache, s.schedule()), [8, 2], [-0.25, -3.0])
    assert [q.seq_id for q in fin] == [3] and c.finish_reason == "stop_sequence"      # not "eos": sequences come first
    fin = s.postprocess(_commit(cache, s.schedule()), [9], [-0.125])
    assert [q.seq_id for q in fin] == [1] and a.finish_reason == "stop_sequence"
    assert a.output_token_ids == [7, 8, 9] and a.logprobs == [-0.5, -0.25, -0.125]
    assert s.is_finished() and cache.num_free_pages(0) == 64


def _commit(cache, step):
    for e in step.entries:
        cache.commit(e.seq.seq_id, e.start + e.num_tokens)
    return step


def test_sampling_params_checks():
    with pytest.raises(ValueError):
        SamplingParams(n=0)
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)
    assert SamplingParams(stop_strings="x").stop_strings == ["x"]


def test_a_request_that_begins_like_an_earlier_one_starts_behind_its_pages():
    cache = CacheManager({0: FULL}, 4, 32, 4, prefix_caching=True)
    s = Scheduler(cache, 4, 64, 64, eos_token_ids=(2,))
    a = Sequence(list(range(10, 23)), SamplingParams(max_tokens=2), seq_id=1)        # 13 tokens: three full pages
    s.add(a)
    while not a.is_finished:
        run(s, cache, s.schedule())
    assert cache.groups[0].pool.num_cached == 3
    b = Sequence(list(range(10, 23)) + [5, 6], SamplingParams(max_tokens=2), seq_id=2)
    c = Sequence(list(range(10, 18)), SamplingParams(max_tokens=2), seq_id=3)         # 8 tokens: one page may be taken
    s.add(b)
    s.add(c)
    st = s.schedule()
    assert [(e.seq.seq_id, e.start, e.num_tokens, e.samples) for e in st.entries] == [(2, 12, 3, True), (3, 4, 4, True)]
    assert b.num_computed == 12 and cache.committed(2) == 12
    run(s, cache, st)
    while not s.is_finished():
        run(s, cache, s.schedule())
    assert cache.prefix_hit_tokens == 16 and cache.groups[0].pool.num_used == 0


def test_abort_frees_pages():
    s, cache = make()
    a = seq(9, sid=1)
    s.add(a)
    run(s, cache, s.schedule())
    s.abort(1)
    assert a.finish_reason == "aborted" and cache.num_free_pages(0) == 16 and s.is_finished()


def test_many_requests_tiny_pool_all_finish():
    import random
    rng = random.Random(0)
    s, cache = make(num_pages=12, page=4, max_seqs=4, budget=16, max_len=40)
    seqs = [seq(rng.randint(1, 20), max_tokens=rng.randint(1, 12), sid=i, ignore_eos=True) for i in range(25)]
    for q in seqs:
        s.add(q)
    steps = 0
    while not s.is_finished():
        st = s.schedule()
        assert st.num_tokens <= 16
        assert len({e.seq.seq_id for e in st.entries}) == len(st.entries)
        run(s, cache, st)
        steps += 1
        assert steps < 2000
    assert all(q.is_finished and q.num_output_tokens == q.params.max_tokens for q in seqs)
    assert cache.num_free_pages(0) == 12 and cache.state_slots.num_free == 4
    assert s.num_preemptions > 0


def test_portions_off_takes_a_prompt_whole_or_not_at_all():
    """enable_chunked_prefill=False (the reference's switch, atom/model_engine/scheduler.py:1765-1767):
    a prompt is scheduled only in a step that has room for all of it; a prompt longer than the token
    budget can never run and is refused with a reason; decoding goes on meanwhile."""
    cache = CacheManager({0: FULL}, 4, 64, 4)
    s = Scheduler(cache, 4, 20, 200, eos_token_ids=(2,), enable_chunked_prefill=False)
    a, b, c, d = seq(12, sid=1), seq(15, sid=2), seq(25, sid=3), seq(6, sid=4)
    for q in (a, b, c, d):
        s.add(q)
    st = s.schedule()
    # a fits (12 of 20); b (15) does not fit beside it and is not cut: it waits, and nothing behind it is taken
    assert [(e.seq.seq_id, e.start, e.num_tokens, e.samples) for e in st.entries] == [(1, 0, 12, True)]
    run(s, cache, st)
    st = s.schedule()
    # a decodes (1), b runs whole (15): 16 of 20; c (25 > 20) is refused with a reason; d (6) no longer fits
    assert [(e.seq.seq_id, e.start, e.num_tokens) for e in st.entries] == [(1, 12, 1), (2, 0, 15)]
    assert [q.seq_id for q in st.rejected] == [3] and "max_num_batched_tokens" in c.finish_reason
    run(s, cache, st)
    st = s.schedule()
    assert [(e.seq.seq_id, e.start, e.num_tokens) for e in st.entries] == [(1, 13, 1), (2, 15, 1), (4, 0, 6)]
    run(s, cache, st)
    assert all(e.samples for e in st.entries)


def test_portions_off_recomputes_a_preempted_request_whole():
    cache = CacheManager({0: FULL}, 4, 6, 4)
    s = Scheduler(cache, 4, 16, 200, eos_token_ids=(2,), enable_chunked_prefill=False)
    a, b = seq(7, sid=1, max_tokens=12), seq(8, sid=2, max_tokens=12)
    s.add(a)
    s.add(b)
    run(s, cache, s.schedule())                     # both prompts: 2 + 2 pages... a grows first
    while not s.num_preemptions:
        run(s, cache, s.schedule())
    assert b.status == SequenceStatus.WAITING and b.num_computed == 0
    n = b.num_tokens
    while b.status == SequenceStatus.WAITING:
        st = s.schedule()
        run(s, cache, st)
    e = next(e for e in st.entries if e.seq is b)
    assert (e.start, e.num_tokens) == (0, n)        # what it had, prompt and generated tokens, in one step


def test_step_labels_for_profiler_traces():
    """The names steps carry in a trace (after atom/model_engine/run_labels.py): kind, requests, tokens,
    portions and single tokens, padding of a captured shape, contexts of eager steps."""
    from atom_b200.engine.runner import step_label
    assert step_label([1, 1, 1], [41, 7, 100], graph_batch=4) == "decode[bs=3/4 tok=3 d=3]"
    assert step_label([1] * 8, [9] * 8, graph_batch=8) == "decode[bs=8 tok=8 d=8]"
    assert step_label([70, 1, 1, 5, 1], [70, 9, 9, 30, 2], graph_shape=(128, 8)) == "mixed[bs=5/8 tok=78/128 p=2 d=3]"
    assert step_label([600, 300], [600, 300]) == "prefill[bs=2 tok=900 p=2 ctx=[600, 300]]"
    assert step_label([1], [12]) == "eager_decode[bs=1 tok=1 d=1 ctx=12]"
    assert step_label([2, 1, 1, 1, 1, 1, 1], [5, 6, 7, 8, 9, 10, 11]) == "prefill[bs=7 tok=8 p=1 d=6 ctx=[5, 6, 7]...+4]"
