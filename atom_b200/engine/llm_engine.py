"""The user-facing engine, with the reference's surface (atom/model_engine/llm_engine.py:36-260):
``LLMEngine(model, **engine_options)``, ``add_request``, ``step``, ``is_finished`` and
``generate(prompts, sampling_params) -> list of dicts`` with the keys text, token_ids,
latency, finish_reason, num_tokens_input, num_tokens_output, ttft, tpot (:752-762).
It is one process: the scheduler, the runner and the sampler are called directly (the
reference puts processes and sockets between them)."""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Sequence as Seq, Union

import torch

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry, StepError
from .runner import ModelRunner
from .scheduler import ScheduledEntry, ScheduledStep, Scheduler
from .sequence import Sequence


def _load_tokenizer(model_dir: str):
    """A tokenizer if the folder has one (the reference uses transformers' AutoTokenizer,
    atom/model_engine/llm_engine.py:45); random-weight folders have none and run on token ids."""
    if not any(os.path.isfile(os.path.join(model_dir, f)) for f in ("tokenizer.json", "tokenizer_config.json")):
        return None
    try:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(model_dir)
    except Exception:  # pragma: no cover - depends on the folder
        return None


class _Pending:
    """A launched step: its schedule, the sampled ids on the device, their pinned host copy
    (in flight) and the event that marks the copy's end."""

    def __init__(self, sched, ids, host, event, lp_host=None, flags_host=None):
        self.sched, self.ids, self.host, self.event = sched, ids, host, event
        self.lp_host = lp_host      # pinned copy of the tokens' log-probabilities, if some request wants them
        self.flags_host = flags_host    # pinned copy of the kernels' fault flags as they stood after the step


class LLMEngine:
    def __init__(self, model: str, model_config=None, **kwargs):
        self.config = EngineConfig(model=model, **kwargs)
        self.runner = ModelRunner(self.config, model_config=model_config)
        self.tokenizer = _load_tokenizer(model) if model and os.path.isdir(model) else None
        eos = list(self.runner.spec.eos_token_ids)
        if self.tokenizer is not None and self.tokenizer.eos_token_id is not None:
            if self.tokenizer.eos_token_id not in eos:
                eos.append(self.tokenizer.eos_token_id)
        self.scheduler = Scheduler(
            self.runner.cache,
            max_num_seqs=self.config.max_num_seqs,
            max_num_batched_tokens=self.config.max_num_batched_tokens,
            max_model_len=self.runner.max_model_len,
            eos_token_ids=eos,
            portion_cap=self.config.long_prefill_token_threshold,
            enable_chunked_prefill=self.config.enable_chunked_prefill,
        )
        self.sampler = Sampler(self.runner.device, self.config.seed)
        self._seqs: Dict[int, Sequence] = {}
        self._next_seq_id = 0     # per engine: a second engine of the process gives the same ids, hence the same default seeds
        self.num_steps = 0
        self.num_prompt_tokens = 0
        self.num_generated_tokens = 0
        self.d2h_bytes = 0      # bytes of sampled token ids read back to the host so far
        # A decode step that has been launched but whose tokens the host has not read yet.  The
        # next decode step is launched before they are read (its tokens stay on the device), so
        # the host's work for a step overlaps the device's work for the one before: the
        # reference's deferred output (atom/model_engine/model_runner.py:204-223, :358-392).
        self._pending: Optional[_Pending] = None
        self.overlap_steps = not self.config.enforce_eager
        self.num_overlapped = 0
        self.last_step_tokens = (0, 0)
        self._pin_ring = None
        self._pin_next = 0
        self._profiler = None
        # every decode graph a batch of this engine can replay, before the first request
        self.runner.capture_graphs(min(self.config.max_num_seqs, self.config.max_num_batched_tokens))

    # ------------------------------------------------------------------ profiling

    def start_profile(self) -> None:
        """Starts a torch profiler (host and device activity) if ``torch_profiler_dir`` is set; the
        trace is written by ``stop_profile``.  (The reference's start_profile / stop_profile,
        atom/model_engine/llm_engine.py:286-295, model_runner.py:1025-1130.)"""
        if self.config.torch_profiler_dir is None or self._profiler is not None:
            return
        from torch.profiler import ProfilerActivity, profile

        os.makedirs(self.config.torch_profiler_dir, exist_ok=True)
        self._profiler = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA])
        self._profiler.__enter__()
        self.runner.profiling = True       # every step becomes a labelled range (runner.step_label)

    def stop_profile(self) -> Optional[str]:
        """Stops the profiler and writes ``<model name>_ts_<time>.pt.trace.json.gz``; returns its path."""
        if self._profiler is None:
            return None
        import gzip
        import shutil

        prof, self._profiler = self._profiler, None
        self.runner.profiling = False
        torch.cuda.synchronize(self.runner.device)
        prof.__exit__(None, None, None)
        name = os.path.basename(self.config.model.rstrip("/")) or "trace"
        name = "".join(c if c.isalnum() or c in "_-." else "_" for c in name)
        stamp = time.strftime("%Y%m%d_%H%M%S") + f"_{int(time.time() % 1 * 1000):03d}"
        path = os.path.join(self.config.torch_profiler_dir, f"{name}_ts_{stamp}.pt.trace.json")
        prof.export_chrome_trace(path)
        with open(path, "rb") as src, gzip.open(path + ".gz", "wb") as dst:
            shutil.copyfileobj(src, dst)
        os.remove(path)
        return path + ".gz"

    # ------------------------------------------------------------------ requests

    def add_request(self, prompt: Union[str, Seq[int]], sampling_params: Optional[SamplingParams] = None) -> int:
        """One request; returns its id.  For ``n > 1`` use ``add_request_fanout``."""
        params = sampling_params or SamplingParams()
        if params.n != 1:
            raise ValueError("add_request makes one request; for SamplingParams.n > 1 call add_request_fanout")
        return self.add_request_fanout(prompt, params)[0]

    def add_request_fanout(self, prompt: Union[str, Seq[int]],
                           sampling_params: Optional[SamplingParams] = None) -> List[int]:
        """Tokenizes once and makes ``sampling_params.n`` sibling requests with the same prompt and
        random streams of their own (atom/model_engine/llm_engine.py:618-720); returns their ids."""
        params = sampling_params or SamplingParams()
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer in the model folder; pass token ids")
            ids = self.tokenizer.encode(prompt)
        else:
            ids = [int(t) for t in prompt]
        if not ids:
            raise ValueError("empty prompt")
        V = self.runner.spec.vocab_size
        if min(ids) < 0 or max(ids) >= V:
            raise ValueError(f"prompt has a token id outside [0, {V})")
        stops: List[List[int]] = []
        if params.stop_strings:
            if self.tokenizer is None:
                raise ValueError("stop_strings need a tokenizer in the model folder; use stop_token_ids")
            for text in params.stop_strings:
                toks = self.tokenizer.encode(text, add_special_tokens=False)
                if toks:
                    stops.append([int(t) for t in toks])
        out = []
        for i in range(params.n):
            seq = Sequence(ids, params, self._next_seq_id, stop_token_sequences=stops, sibling_index=i)
            self._next_seq_id += 1
            self._seqs[seq.seq_id] = seq
            self.scheduler.add(seq)
            out.append(seq.seq_id)
        return out

    def abort(self, seq_id: int) -> None:
        self.scheduler.abort(seq_id)

    def _seed_of(self, seq: Sequence) -> int:
        if seq.params.seed is not None:
            return (seq.params.seed + seq.sibling_index) & 0xFFFFFFFF
        return (self.config.seed * 0x9E3779B1 + seq.seq_id * 0x85EBCA6B + 1) & 0xFFFFFFFF

    # ------------------------------------------------------------------ one step

    def is_finished(self) -> bool:
        return self.scheduler.is_finished() and self._pending is None

    def _sample(self, logits, sampling: List[Sequence], ahead: int = 0) -> torch.Tensor:
        return self.sampler.sample(
            logits, [s.params for s in sampling], [self._seed_of(s) for s in sampling],
            [s.num_output_tokens + ahead for s in sampling])

    def _logprobs(self, logits, ids, sampling: List[Sequence]) -> Optional[torch.Tensor]:
        """Log-probabilities of the sampled tokens (device, float32) if a request of the batch wants them."""
        if not any(s.return_logprobs for s in sampling):
            return None
        return self.sampler.logprobs(logits, ids)

    def _read_later(self, sched: ScheduledStep, ids: torch.Tensor, lps: Optional[torch.Tensor] = None) -> "_Pending":
        """Starts the copy of the sampled ids (and of the kernels' fault flags) to pinned host memory;
        the host waits for it later."""
        n = ids.numel()
        if self._pin_ring is None or self._pin_ring[0].numel() < 2 * n + 2:
            self._pin_ring = [torch.empty(max(2 * n + 2, 128), dtype=torch.int32).pin_memory() for _ in range(4)]
        self._pin_next = (self._pin_next + 1) % 4      # a buffer is read two calls later at most
        buf = self._pin_ring[self._pin_next]
        host = buf[:n]
        host.copy_(ids, non_blocking=True)
        lp_host = None
        if lps is not None:
            lp_host = buf[n:2 * n].view(torch.float32)
            lp_host.copy_(lps, non_blocking=True)
        flags_host = buf[2 * n:2 * n + 2]
        flags_host.copy_(self.runner.flags, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return _Pending(sched, ids, host, ev, lp_host, flags_host)

    def _resolve(self, pending: "_Pending") -> List[Sequence]:
        """Waits for a launched step's tokens, raises if a kernel of the step (or of one before it)
        reported a fault, and does the step's bookkeeping."""
        pending.event.synchronize()
        self.runner.raise_for_flags(pending.flags_host.tolist())
        tokens = pending.host.tolist()
        lps = pending.lp_host.tolist() if pending.lp_host is not None else None
        self.d2h_bytes += 4 * len(tokens) * (2 if lps is not None else 1) + 8
        self.num_generated_tokens += len(tokens)
        return self.scheduler.postprocess(pending.sched, tokens, lps)

    def _abandon(self, *scheds: Optional[ScheduledStep]) -> None:
        """A kernel of a step reported a fault: what the step's requests have in the cache is not to be
        trusted (and a step launched ahead of it has moved them on without the scheduler's knowledge).
        They end with reason "fault" and give everything back; the engine goes on with the others."""
        for sched in scheds:
            for e in (sched.entries if sched is not None else ()):
                if not e.seq.is_finished:
                    self.scheduler.abort(e.seq.seq_id, reason="fault")

    def _look_ahead(self, pending: "_Pending") -> Optional["_Pending"]:
        """Launches the decode step after ``pending`` without knowing its tokens, if nothing but
        one more token per running request can happen: nobody waits, the running requests are
        exactly those of the pending step, and their next positions have pages.  A request that
        ends with the pending token for a reason the host can foresee (token count, length) is
        left out of the step; the others' tokens are gathered on the device."""
        sch = self.scheduler
        seqs = [e.seq for e in pending.sched.entries]
        if sch.waiting or len(seqs) != len(sch.running) or any(a is not b for a, b in zip(seqs, sch.running)):
            return None
        if len(seqs) > sch.max_num_batched_tokens:
            return None
        entries, sched, rows, going = [], ScheduledStep(), [], []
        cache, need = self.runner.cache, {}
        for i, e in enumerate(pending.sched.entries):
            s = e.seq
            if not e.samples or e.num_tokens != 1:
                return None
            if s.num_output_tokens + 1 >= s.params.max_tokens or s.num_tokens + 1 >= sch.max_model_len:
                continue                             # its last token is the pending one
            start = e.start + 1                      # position of the token the pending step produces
            for gi, n in cache.pages_to_extend(s.seq_id, start + 1).items():
                need[gi] = need.get(gi, 0) + n
            entries.append(StepEntry(s.seq_id, [0], (0,)))
            sched.entries.append(ScheduledEntry(s, start, 1, True))
            rows.append(i)
            going.append(s)
        if not entries or not self.runner._graph_size(entries):
            return None
        if any(n > cache.num_free_pages(gi) for gi, n in need.items()):
            return None
        logits = self.runner.step(entries, device_tokens=pending.ids,
                                  device_token_rows=rows if len(rows) < len(seqs) else None)
        ids = self._sample(logits, going, ahead=1)
        self.num_steps += 1
        self.num_overlapped += 1
        self.last_step_tokens = (0, len(entries))
        return self._read_later(sched, ids, self._logprobs(logits, ids, going))

    def step(self) -> List[Sequence]:
        """schedule -> run the batch -> sample -> bookkeeping; returns what finished.

        A pure decode step is left pending (launched, tokens unread); the next call first tries
        to launch the following decode step and only then reads the pending tokens, so a
        request's tokens reach the host one call later than they were computed."""
        if self._pending is not None:
            pending, self._pending = self._pending, None
            ahead = self._look_ahead(pending) if self.overlap_steps else None
            try:
                finished = self._resolve(pending)
            except StepError:
                self._abandon(pending.sched, ahead.sched if ahead is not None else None)
                raise
            if ahead is not None:
                self._pending = ahead
                return finished
            return finished + self._step_now()
        return self._step_now()

    def _step_now(self) -> List[Sequence]:
        sched: ScheduledStep = self.scheduler.schedule()
        finished = list(sched.rejected)
        if not sched.entries:
            return finished
        entries, sampling = [], []
        for e in sched.entries:
            toks = e.seq.token_ids[e.start:e.start + e.num_tokens]
            entries.append(StepEntry(e.seq.seq_id, toks, (e.num_tokens - 1,) if e.samples else ()))
            if e.samples:
                sampling.append(e.seq)
        logits = self.runner.step(entries)
        self.num_steps += 1
        n_decode = sum(1 for e in sched.entries if e.samples and e.num_tokens == 1)
        n_prompt = sum(e.num_tokens for e in sched.entries) - n_decode
        self.num_prompt_tokens += n_prompt
        self.last_step_tokens = (n_prompt, n_decode)      # of the step launched last: prompt tokens, decoded tokens
        if not sampling:
            return finished + self.scheduler.postprocess(sched, [])
        ids = self._sample(logits, sampling)
        lps = self._logprobs(logits, ids, sampling)
        pure_decode = all(e.samples and e.num_tokens == 1 for e in sched.entries)
        if self.overlap_steps and pure_decode and self.runner._graph_size(entries):
            self._pending = self._read_later(sched, ids, lps)
            return finished
        try:
            return finished + self._resolve(self._read_later(sched, ids, lps))
        except StepError:
            self._abandon(sched)
            raise

    # ------------------------------------------------------------------ whole requests

    def generate(self, prompts: Seq[Union[str, Seq[int]]],
                 sampling_params: Union[SamplingParams, Seq[SamplingParams], None] = None) -> List[dict]:
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = [i for p, sp in zip(prompts, sampling_params) for i in self.add_request_fanout(p, sp)]
        while not self.is_finished():
            self.step()
        self.runner.check_status()
        return [self._output(self._seqs.pop(i)) for i in ids]     # n outputs per prompt, in the prompts' order

    def _output(self, seq: Sequence) -> dict:
        out = seq.output_token_ids
        end = seq.finish_time or time.perf_counter()
        ttft = (seq.first_token_time - seq.arrive_time) if seq.first_token_time else 0.0
        tpot = (end - seq.first_token_time) / (len(out) - 1) if seq.first_token_time and len(out) > 1 else 0.0
        return {
            "text": self.tokenizer.decode(out) if self.tokenizer is not None else None,
            "token_ids": out,
            "logprobs": list(seq.logprobs) if seq.return_logprobs else None,
            "latency": end - seq.arrive_time,
            "finish_reason": seq.finish_reason,
            "num_tokens_input": seq.num_prompt_tokens,
            "num_tokens_output": len(out),
            "ttft": ttft,
            "tpot": tpot,
        }

    def stats(self) -> dict:
        """Counters like the reference's collect_metrics (atom/model_engine/engine_utility.py:322-393)."""
        c = self.runner.cache
        return {
            "running": len(self.scheduler.running),
            "waiting": len(self.scheduler.waiting),
            "finished": self.scheduler.num_finished,
            "preemptions": self.scheduler.num_preemptions,
            "steps": self.num_steps,
            "prompt_tokens": self.num_prompt_tokens,
            "generation_tokens": self.num_generated_tokens,
            "kv_pages_total": [g.pool.num_pages for g in c.groups],
            "kv_pages_free": [g.pool.num_free for g in c.groups],
            "prefix_cache_hit_tokens": c.prefix_hit_tokens,
            "prefix_cache_query_tokens": c.prefix_query_tokens,
        }
