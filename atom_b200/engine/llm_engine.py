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
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import ScheduledStep, Scheduler
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
        self.num_steps = 0
        self.num_prompt_tokens = 0
        self.num_generated_tokens = 0
        self.d2h_bytes = 0      # bytes of sampled token ids read back to the host so far

    # ------------------------------------------------------------------ requests

    def add_request(self, prompt: Union[str, Seq[int]], sampling_params: Optional[SamplingParams] = None) -> int:
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
        seq = Sequence(ids, params)
        self._seqs[seq.seq_id] = seq
        self.scheduler.add(seq)
        return seq.seq_id

    def abort(self, seq_id: int) -> None:
        self.scheduler.abort(seq_id)

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

    def _seed_of(self, seq: Sequence) -> int:
        if seq.params.seed is not None:
            return seq.params.seed
        return (self.config.seed * 0x9E3779B1 + seq.seq_id * 0x85EBCA6B + 1) & 0xFFFFFFFF

    # ------------------------------------------------------------------ one step

    def step(self) -> List[Sequence]:
        """schedule -> run the batch -> sample -> bookkeeping; returns what finished."""
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
        tokens: List[int] = []
        if sampling:
            ids = self.sampler.sample(
                logits, [s.params for s in sampling], [self._seed_of(s) for s in sampling],
                [s.num_output_tokens for s in sampling])
            tokens = ids.tolist()
            self.d2h_bytes += 4 * len(tokens)
        self.num_steps += 1
        self.num_prompt_tokens += sum(e.num_tokens for e in sched.entries if not (e.samples and e.num_tokens == 1))
        self.num_generated_tokens += len(tokens)
        finished += self.scheduler.postprocess(sched, tokens)
        return finished

    # ------------------------------------------------------------------ whole requests

    def generate(self, prompts: Seq[Union[str, Seq[int]]],
                 sampling_params: Union[SamplingParams, Seq[SamplingParams], None] = None) -> List[dict]:
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        while not self.is_finished():
            self.step()
        self.runner.check_status()
        return [self._output(self._seqs.pop(i)) for i in ids]

    def _output(self, seq: Sequence) -> dict:
        out = seq.output_token_ids
        end = seq.finish_time or time.perf_counter()
        ttft = (seq.first_token_time - seq.arrive_time) if seq.first_token_time else 0.0
        tpot = (end - seq.first_token_time) / (len(out) - 1) if seq.first_token_time and len(out) > 1 else 0.0
        return {
            "text": self.tokenizer.decode(out) if self.tokenizer is not None else None,
            "token_ids": out,
            "logprobs": None,
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
        }
