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

import torch

from .. import native
from ..cache import CacheManager, OutOfPages
from ..cache.storage import CacheStorage
from ..config.engine_config import EngineConfig
from ..config.model_config import ModelConfig, load_model_config
from ..models.model import Model
from ..models.registry import build_model_spec
from ..parts.base import Runtime, Workspace
from ..weights import load_weights, random_weights_on_device
from .batch import StepBuilder, StepEntry, StepError

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class _DecodeGraph:
    num_launches = 0
    graph = None
    workspace = None
    logits = None


# Steps that are not pure decode steps replay a graph too when they are small enough to be bound by
# the host's launches (a few hundred per step, 3-4 ms): one graph per (tokens, requests) rounded up to
# these.  Where the device becomes the bound, rows of padding cost more than the launches, and that
# point lies the lower the larger the model is.  Measured with 8 decoded tokens beside a portion
# (graph against eager): Qwen3-0.6B sizes 16 tokens 3.37 -> 1.85 ms, 400 tokens 3.07 -> 2.46 ms, even at
# 800; 1.7B sizes 200 tokens 3.14 -> 2.63 ms, even at 350; 8B sizes 16 tokens 5.09 -> 4.88 ms, 100
# tokens 5.31 -> 5.09 ms, 408 tokens (in a shape of 448) 7.26 -> 7.8 ms.  Hence the limit below:
# about 600e9 / parameters tokens, at least 128.
_MIXED_TOKENS = (16, 32, 48, 64, 80, 96, 128, 160, 192, 224, 256, 320, 384, 448, 512, 640, 768, 896, 1024)
_MIXED_SEQS = (8, 32, 64)


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
        self.cache = CacheManager(needs, self.page_size, num_pages, engine_config.max_num_seqs,
                                  prefix_caching=engine_config.enable_prefix_caching)
        self.storage = CacheStorage(self.cache, self.dtype, self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.builder = StepBuilder(self.cache, self.device, self.spec.vocab_size, self.status)
        self.steps_run = 0
        # Decode steps (one token per request) of these batch sizes replay a captured CUDA graph.
        self.graphs_enabled = not engine_config.enforce_eager and self.model.graph_safe
        self._graph_sizes = sorted(set(int(b) for b in engine_config.cudagraph_capture_sizes if int(b) > 0))
        self._graphs: Dict[object, "_DecodeGraph"] = {}     # batch size, or (tokens, requests), -> graph
        self.mixed_graphs = self.graphs_enabled and engine_config.cudagraph_mixed_steps
        params = self.weight_bytes / (4 if self.dtype == torch.float32 else 2)
        limit = 128 if self.dtype == torch.float32 else max(128.0, 600e9 / max(params, 1.0))
        self._mixed_tokens = tuple(t for t in _MIXED_TOKENS if t <= limit) or _MIXED_TOKENS[:1]
        self._table_width = max(1, -(-self.max_model_len // self.page_size))
        self.graph_replays = 0

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

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None,
             device_token_rows: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Runs one batch; returns logits [R, vocab] float32 on the device, rows in the order
        of the entries and of their ``want`` lists.  The cache then holds the new tokens.

        device_tokens: for a batch of single-token requests whose tokens are still on the device
        (the sampler's output of the step before, int32, in the entries' order; or, with
        ``device_token_rows``, entry i's token at ``device_tokens[device_token_rows[i]]``, for a
        step that some requests of the step before have left): they replace the entries' token
        values, which are then placeholders.  The host never has to see them before this step
        is launched."""
        if not entries:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        targets = self._reserve(entries)
        size = self._graph_size(entries)
        shape = None if size or device_tokens is not None else self._mixed_shape(entries)
        if device_tokens is not None:
            rows = None if device_token_rows is None else [int(r) for r in device_token_rows]
            n_src = device_tokens.numel()
            if not size or device_tokens.dtype != torch.int32 or (
                    n_src != len(entries) if rows is None
                    else len(rows) != len(entries) or any(not 0 <= r < n_src for r in rows)):
                raise StepError("device_tokens needs a captured decode step and one int32 token per entry")
            logits = self._step_graph(entries, targets, size, device_tokens, rows)
        elif size:
            logits = self._step_graph(entries, targets, size)
        elif shape:
            logits = self._step_mixed_graph(entries, targets, shape)
        else:
            ctx = self.builder.build(entries, targets)
            logits = self.model.forward(ctx, self.storage)
        for e, t in zip(entries, targets):
            self.cache.commit(e.rid, t)
        self.steps_run += 1
        return logits

    @property
    def h2d_bytes(self) -> int:
        """Bytes of step metadata copied host -> device so far."""
        return self.builder.h2d_bytes

    # ------------------------------------------------------------------ captured decode steps

    def _graph_size(self, entries: Sequence[StepEntry]) -> int:
        """The captured batch size a step replays, 0 if it runs eagerly: every request brings
        exactly one token, and the batch fits the largest captured size."""
        if not self.graphs_enabled or not self._graph_sizes:
            return 0
        n = len(entries)
        if n > self._graph_sizes[-1] or any(len(e.tokens) != 1 for e in entries):
            return 0
        for b in self._graph_sizes:
            if b >= n:
                return b
        return 0

    def _mixed_shape(self, entries: Sequence[StepEntry]):
        """(tokens, requests) of the fixed shape that a step of prompt portions (beside decoded tokens or
        not) replays, None if it runs eagerly: small enough, and no more wanted rows than requests."""
        if not self.mixed_graphs:
            return None
        T = sum(len(e.tokens) for e in entries)
        S = max(len(entries), sum(len(e.want) for e in entries))
        if T > self._mixed_tokens[-1] or S > _MIXED_SEQS[-1]:
            return None
        return (next(t for t in self._mixed_tokens if t >= T), next(n for n in _MIXED_SEQS if n >= S))

    def _capture_mixed(self, shape) -> "_DecodeGraph":
        """As ``_capture``, for a step of ``shape`` = (tokens, requests) of any makeup: launch plans are
        made for every batch that fits the shape, and for the longest request the engine takes."""
        tokens, seqs = shape
        g = _DecodeGraph()
        g.workspace = Workspace(self.device)
        g.logits = torch.empty((seqs, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        saved = self.rt.workspace
        self.rt.workspace = g.workspace
        try:
            def run():
                ctx = self.builder.fixed_context_mixed(tokens, seqs, self._table_width, self.max_model_len)
                ctx.logits_out = g.logits
                self.model.forward(ctx, self.storage)

            self.builder.build_fixed_mixed([], [], tokens, seqs, self._table_width)   # all padding
            run()
            torch.cuda.current_stream().synchronize()
            g.graph = torch.cuda.CUDAGraph()
            before = native.launches
            with torch.cuda.graph(g.graph):
                run()
            g.num_launches = native.launches - before
            g.workspace.frozen = True
        finally:
            self.rt.workspace = saved
        return g

    def _step_mixed_graph(self, entries: Sequence[StepEntry], targets: List[int], shape) -> torch.Tensor:
        g = self._graphs.get(shape)
        if g is None:
            g = self._graphs[shape] = self._capture_mixed(shape)
        self.builder.build_fixed_mixed(entries, targets, shape[0], shape[1], self._table_width)
        g.graph.replay()
        native.add_launches(g.num_launches)
        self.graph_replays += 1
        return g.logits[: sum(len(e.want) for e in entries)]       # valid until the next step of this shape

    def capture_graphs(self, max_batch: int) -> list:
        """Captures, ahead of the first request, the decode graphs that batches of up to
        ``max_batch`` requests replay (the reference captures all of its sizes at start,
        atom/model_engine/model_runner.py capture_cudagraph); without this call a size is
        captured when a step first needs it.  Returns the sizes captured now."""
        done = []
        if not self.graphs_enabled:
            return done
        for b in self._graph_sizes:
            if b not in self._graphs:
                self._graphs[b] = self._capture(b)
                done.append(b)
            if b >= max_batch:
                break
        if self.mixed_graphs:      # (a capture in the middle of serving would stall a step by ~0.1 s)
            for n in _MIXED_SEQS:
                for t in self._mixed_tokens:
                    if (t, n) not in self._graphs:
                        self._graphs[(t, n)] = self._capture_mixed((t, n))
                        done.append((t, n))
                if n >= max_batch:
                    break
        return done

    def _capture(self, size: int) -> "_DecodeGraph":
        """Runs a decode step of ``size`` padding rows once eagerly (loads kernels, sizes the
        buffers), then records the same launches into a graph.  The graph has its own
        activation buffers and logits, so steps of other shapes cannot move them."""
        g = _DecodeGraph()
        g.workspace = Workspace(self.device)
        g.logits = torch.empty((size, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        saved = self.rt.workspace
        self.rt.workspace = g.workspace
        try:
            def run():
                # launch plans are made for the longest request the engine takes
                ctx = self.builder.fixed_context(size, self._table_width, self.max_model_len)
                ctx.logits_out = g.logits
                self.model.forward(ctx, self.storage)

            self.builder.build_fixed([], [], size, self._table_width)   # all rows padding
            run()
            torch.cuda.current_stream().synchronize()
            g.graph = torch.cuda.CUDAGraph()
            before = native.launches
            with torch.cuda.graph(g.graph):
                run()
            g.num_launches = native.launches - before     # own kernels recorded in the graph
            g.workspace.frozen = True
        finally:
            self.rt.workspace = saved
        return g

    def _step_graph(self, entries: Sequence[StepEntry], targets: List[int], size: int,
                    device_tokens: Optional[torch.Tensor] = None,
                    device_token_rows: Optional[List[int]] = None) -> torch.Tensor:
        g = self._graphs.get(size)
        if g is None:
            g = self._graphs[size] = self._capture(size)
        ctx = self.builder.build_fixed(entries, targets, size, self._table_width, device_token_rows)
        if device_tokens is not None:          # on the stream, after the arrays' copy
            if device_token_rows is not None:
                device_tokens = device_tokens.index_select(0, ctx.token_ids[: len(entries)])
            ctx.token_ids[: len(entries)].copy_(device_tokens)
        g.graph.replay()
        native.add_launches(g.num_launches)
        self.graph_replays += 1
        rows = []
        for i, e in enumerate(entries):
            for w in e.want:
                if w != 0:
                    raise StepError(f"request {e.rid!r}: wanted place {w} outside its 1 token")
                rows.append(i)
        if rows == list(range(len(entries))):
            return g.logits[: len(entries)]       # valid until the next step of this size
        if not rows:
            return g.logits[:0]
        return g.logits[torch.tensor(rows, device=self.device)]

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
        native.check_error_flags()
