"""The model runner: owns the model, its weights, the cache and ONE step function.

``step(entries)`` takes a batch of (request, its next tokens): portions of prompts beside
single decoded tokens, cut anywhere.  It runs only the tokens it is given, as one batch,
against what earlier steps left in the cache, and returns the 32-bit logits at the places
that were asked for.  The scheduler, the generation loop and the trace replay all call
this one function.  (Reference: ModelRunner.forward, atom/model_engine/model_runner.py:3327,
which takes either prompt portions or decoded tokens, never both.)
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import native
from ..cache import NO_PAGE, CacheManager, OutOfPages
from ..cache.storage import CacheStorage
from ..config.engine_config import EngineConfig
from ..config.model_config import ModelConfig, load_model_config
from ..models.model import Model
from ..models.registry import build_model_spec
from ..parts.base import Runtime, Workspace
from ..weights import load_weights, random_weights_on_device
from .batch import StepContext, StepEntry, pack_layout

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class StepError(RuntimeError):
    pass


class ModelRunner:
    def __init__(self, engine_config: EngineConfig, model_config: Optional[ModelConfig] = None,
                 device: str = "cuda:0"):
        if not torch.cuda.is_available():
            raise RuntimeError("atom_b200 runs on a CUDA device only (no CPU path)")
        native.lib()  # build/load the kernels now: fail here, loudly, if they are missing
        self.cfg = engine_config
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = _DTYPES[engine_config.dtype]
        self.model_config = model_config or load_model_config(engine_config.model)
        self.spec = build_model_spec(self.model_config)
        self.model = Model(self.spec)
        self.rt = Runtime(self.dtype, self.device, Workspace(self.device))
        if engine_config.load_dummy:
            tensors = random_weights_on_device(self.model, engine_config.seed, self.dtype, self.device)
        else:
            tensors = load_weights(self.model, engine_config.model, self.dtype, self.device)
        self.model.bind(tensors, self.rt)
        self.weight_bytes = sum(t.numel() * t.element_size() for t in tensors.values())
        self.max_model_len = min(engine_config.max_model_len or self.spec.max_position, self.spec.max_position)
        self.page_size = engine_config.kv_cache_block_size

        needs = self.model.cache_needs()
        probe = CacheManager(needs, self.page_size, 1, 1)
        num_pages = engine_config.num_kvcache_blocks
        if num_pages <= 0:
            num_pages = self._pages_from_free_memory(probe)
        self.cache = CacheManager(needs, self.page_size, num_pages, engine_config.max_num_seqs)
        self.storage = CacheStorage(self.cache, self.dtype, self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._meta_dev = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)
        self._staging = [torch.zeros(1 << 16, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._staging_events: List[Optional[torch.cuda.Event]] = [None] * 4
        self._staging_next = 0
        self.steps_run = 0
        self.h2d_bytes = 0      # bytes of step metadata copied host -> device so far

    # ------------------------------------------------------------------ sizing

    def _pages_from_free_memory(self, probe: CacheManager) -> int:
        """Pages per group from the memory that is left: the reference's rule
        (atom/model_engine/model_runner.py:1591-1611) without its warm-up measurement; the
        activations of the largest step are estimated from the token budget instead."""
        free, total = torch.cuda.mem_get_info(self.device)
        per_page = CacheStorage.bytes_per_page(probe, self.dtype)
        if per_page == 0:
            return 1
        es = 4 if self.dtype == torch.float32 else 2
        # Every matrix product of a layer writes one [tokens, out] buffer; buffers are shared
        # between layers, so the widest layer decides.
        per_layer: Dict[str, int] = {}
        for path, part, _ in self.model.named_parts():
            if path.startswith("layers."):
                key = path.split(".")[1]
                per_layer[key] = per_layer.get(key, 0) + sum(
                    ps.shape[0] for ps in part.params().values() if ps.role == "matrix")
        widest = max(per_layer.values(), default=0) + 4 * self.spec.hidden_size
        act = self.cfg.max_num_batched_tokens * (widest * es * 3 // 2 + self.spec.hidden_size * 8)
        logits = min(self.cfg.max_num_seqs, self.cfg.max_num_batched_tokens) * self.spec.vocab_size * 4 * 2
        budget = total * self.cfg.gpu_memory_utilization - (total - free) - act - logits - 0.02 * total
        n = int(budget // per_page)
        if n < 1:
            raise RuntimeError("no device memory left for the cache")
        return n

    # ------------------------------------------------------------------ the step

    def _reserve(self, entries: Sequence[StepEntry]) -> List[int]:
        """Admits new requests and takes the pages this step needs; all or nothing."""
        cache = self.cache
        need_total: Dict[int, int] = {}
        new_slots = 0
        targets = []
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.rid!r} brings no tokens")
            known = e.rid in cache.requests
            start = cache.committed(e.rid) if known else 0
            target = start + len(e.tokens)
            if target > self.max_model_len:
                raise StepError(f"request {e.rid!r}: {target} tokens exceed max_model_len {self.max_model_len}")
            if not known:
                new_slots += 1
            for gi, n in cache.pages_to_extend(e.rid if known else None, target).items():
                need_total[gi] = need_total.get(gi, 0) + n
            targets.append(target)
        if new_slots > cache.state_slots.num_free:
            raise OutOfPages(f"{new_slots} new requests, {cache.state_slots.num_free} request slots free")
        for gi, n in need_total.items():
            if n > cache.num_free_pages(gi):
                raise OutOfPages(f"step needs {n} pages of group {gi}, {cache.num_free_pages(gi)} free")
        for e, target in zip(entries, targets):
            if e.rid not in cache.requests:
                cache.admit(e.rid)
            cache.extend(e.rid, target)
        return targets

    def build_context(self, entries: Sequence[StepEntry], targets: List[int]) -> StepContext:
        cache = self.cache
        S = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        q_starts = [t - n for t, n in zip(targets, q_lens)]
        T = sum(q_lens)
        V = self.spec.vocab_size
        cu = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu[1:])
        rows: List[int] = []
        for i, e in enumerate(entries):
            for w in e.want:
                if not 0 <= w < q_lens[i]:
                    raise StepError(f"request {e.rid!r}: wanted place {w} outside its {q_lens[i]} tokens")
                rows.append(int(cu[i]) + int(w))
        R = len(rows)
        widths = [max(1, max(len(cache.table(e.rid, g.index)) for e in entries)) for g in cache.groups]
        layout, total = pack_layout(T, S, R, widths)
        if total > self._meta_dev.numel():
            n = 1 << (total - 1).bit_length()
            if self.rt.workspace.frozen:
                raise StepError("step metadata outgrew its buffer while a graph holds it")
            self._meta_dev = torch.zeros(n, dtype=torch.int32, device=self.device)
            self._staging = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(4)]
            self._staging_events = [None] * 4
        k = self._staging_next
        self._staging_next = (k + 1) % len(self._staging)
        if self._staging_events[k] is not None:
            self._staging_events[k].synchronize()
        host = self._staging[k].numpy()

        def sec(name):
            o, n = layout[name]
            return host[o:o + n]

        tok = sec("token_ids")
        pos = sec("positions")
        sot = sec("seq_of_token")
        for i, e in enumerate(entries):
            a, b = cu[i], cu[i + 1]
            tok[a:b] = np.asarray(e.tokens, dtype=np.int64)
            pos[a:b] = np.arange(q_starts[i], targets[i], dtype=np.int32)
            sot[a:b] = i
        if T and (tok.min() < 0 or tok.max() >= V):
            raise StepError(f"token id outside [0, {V})")
        sec("cu_q")[:] = cu
        sec("ctx_len")[:] = targets
        slots = [cache.requests[e.rid].state_slot for e in entries]
        sec("state_slots")[:] = slots
        lr = sec("logits_rows")
        lr[:] = 0
        lr[:R] = rows
        for g, w in zip(cache.groups, widths):
            bt = sec(f"bt{g.index}").reshape(S, w)
            bt[:] = NO_PAGE
            for i, e in enumerate(entries):
                t = cache.table(e.rid, g.index)
                bt[i, :len(t)] = t
        dev = self._meta_dev
        dev[:total].copy_(self._staging[k][:total], non_blocking=True)
        self.h2d_bytes += 4 * total
        ev = torch.cuda.Event()
        ev.record()
        self._staging_events[k] = ev

        def dsec(name):
            o, n = layout[name]
            return dev[o:o + n]

        return StepContext(
            num_tokens=T, num_seqs=S, num_logits_rows=R,
            token_ids=dsec("token_ids"), positions=dsec("positions"), seq_of_token=dsec("seq_of_token"),
            cu_q=dsec("cu_q"), ctx_len=dsec("ctx_len"), state_slots=dsec("state_slots"),
            logits_rows=dsec("logits_rows")[:R] if R else dsec("logits_rows")[:0],
            block_tables={g.index: dsec(f"bt{g.index}").view(S, w) for g, w in zip(cache.groups, widths)},
            status=self.status, q_lens=q_lens, q_starts=q_starts, host_state_slots=slots,
            max_q_len=max(q_lens), max_ctx_len=max(targets),
        )

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs one batch; returns logits [R, vocab] float32 on the device, rows in the order
        of the entries and of their ``want`` lists.  The cache then holds the new tokens."""
        if not entries:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        targets = self._reserve(entries)
        ctx = self.build_context(entries, targets)
        logits = self.model.forward(ctx, self.storage)
        for e, t in zip(entries, targets):
            self.cache.commit(e.rid, t)
        self.steps_run += 1
        return logits

    def finish(self, rid: Hashable) -> None:
        """The request is over (or preempted): its pages and its state slot go back."""
        if rid in self.cache.requests:
            self.cache.release(rid)

    def check_status(self) -> None:
        """Raises if a kernel met a position without a page (synchronises the device)."""
        self._status_host.copy_(self.status)
        torch.cuda.current_stream().synchronize()
        if int(self._status_host[0]) != 0:
            raise StepError("a kernel found a token position without a cache page")
