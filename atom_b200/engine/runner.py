"""The model runner: owns the model, its weights, the cache and ONE step function.

``step(entries)`` takes a batch of (request, its next tokens): portions of prompts beside
single decoded tokens, cut anywhere.  It runs only the tokens it is given, as one batch,
against what earlier steps left in the cache, and returns the 32-bit logits at the places
that were asked for.  The scheduler, the generation loop and the trace replay all call
this one function.  (Reference: ModelRunner.forward, atom/model_engine/model_runner.py:3327,
which takes either prompt portions or decoded tokens, never both.)
"""
from __future__ import annotations

import contextlib

from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
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


def step_label(q_lens: Sequence[int], ctx_lens: Sequence[int], graph_batch: Optional[int] = None,
               graph_shape=None) -> str:
    """The name of a step's range in a profiler trace, after the reference's labels
    (atom/model_engine/run_labels.py:38-110): the kind, then ``key=value`` fields in brackets.

      decode[bs=3/4 tok=3 d=3]            single-token requests replayed from the graph of batch 4
      mixed[bs=5 tok=77/128 p=2 d=3]      portions beside decoded tokens, replayed from the graph of 128 tokens
      prefill[bs=2 tok=900 p=2 ctx=[600, 300]]   a step with portions that runs eagerly
      eager_decode[bs=3 tok=3 d=3 ctx=[41, 7, 100]]

    bs: requests (``/n``: the captured batch it is padded to); tok: tokens of the step; p / d: requests with a
    portion of several tokens / with one token; ctx: the requests' lengths after the step (the first three and a
    count when there are more than five)."""
    bs, tok = len(q_lens), sum(q_lens)
    p = sum(1 for n in q_lens if n > 1)
    d = bs - p
    fields = []
    if graph_batch:
        kind = "decode"
        fields.append(f"bs={bs}/{graph_batch}" if graph_batch > bs else f"bs={bs}")
        fields.append(f"tok={tok}")
    elif graph_shape:
        kind = "mixed"
        fields.append(f"bs={bs}/{graph_shape[1]}" if graph_shape[1] > bs else f"bs={bs}")
        fields.append(f"tok={tok}/{graph_shape[0]}" if graph_shape[0] > tok else f"tok={tok}")
    else:
        kind = "prefill" if p else "eager_decode"
        fields += [f"bs={bs}", f"tok={tok}"]
    if p:
        fields.append(f"p={p}")
    if d:
        fields.append(f"d={d}")
    if not graph_batch and not graph_shape:
        ctx = [int(c) for c in ctx_lens]
        if len(ctx) == 1:
            fields.append(f"ctx={ctx[0]}")
        elif len(ctx) <= 5:
            fields.append(f"ctx={ctx}")
        else:
            fields.append(f"ctx={ctx[:3]}...+{len(ctx) - 3}")
    return f"{kind}[{' '.join(fields)}]"


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

        # Decode steps (one token per request) of these batch sizes replay a captured CUDA graph.
        self.graphs_enabled = not engine_config.enforce_eager and self.model.graph_safe
        self._graph_sizes = sorted(set(int(b) for b in engine_config.cudagraph_capture_sizes if int(b) > 0))
        self._graphs: Dict[object, "_DecodeGraph"] = {}     # (batch size | (tokens, requests), plan signature) -> graph
        self._graph_keys: Dict[object, object] = {}         # (shape, context class) -> key into _graphs
        self.mixed_graphs = self.graphs_enabled and engine_config.cudagraph_mixed_steps
        params = self.weight_bytes / (4 if self.dtype == torch.float32 else 2)
        limit = 128 if self.dtype == torch.float32 else max(128.0, 600e9 / max(params, 1.0))
        self._mixed_tokens = tuple(t for t in _MIXED_TOKENS if t <= limit) or _MIXED_TOKENS[:1]
        self._table_width = max(1, -(-self.max_model_len // self.page_size))
        self.graph_replays = 0
        self.profiling = False     # set by whoever starts a profiler: steps then carry labels in the trace
        # All graphs share one workspace and one logits buffer: steps run one after another.
        self._graph_ws = Workspace(self.device, keep_outgrown=True)
        self._graph_logits: Optional[torch.Tensor] = None
        self.memory: Dict[str, int] = {"weights": self.weight_bytes}

        needs = self.model.cache_needs()
        self.flags = native.device_flags(self.device)
        self.status = native.status_flag(self.device)
        num_pages = engine_config.num_kvcache_blocks
        if num_pages <= 0:
            num_pages = self._pages_from_free_memory(needs)
        self.cache = CacheManager(needs, self.page_size, num_pages, engine_config.max_num_seqs,
                                  prefix_caching=engine_config.enable_prefix_caching)
        self.storage = CacheStorage(self.cache, self.dtype, self.device)
        self.memory["cache"] = self.storage.bytes()
        self.builder = StepBuilder(self.cache, self.device, self.spec.vocab_size, self.status)
        self.steps_run = 0

    # ------------------------------------------------------------------ sizing

    def _largest_step(self) -> List[int]:
        """Token counts of the requests of the largest step the scheduler can make."""
        budget = min(self.cfg.max_num_batched_tokens, self.cfg.max_num_seqs * self.max_model_len)
        lens = []
        while budget > 0 and len(lens) < self.cfg.max_num_seqs:
            n = min(budget, self.max_model_len)
            lens.append(n)
            budget -= n
        return lens

    def _graph_memory_bound(self, eager_ws_bytes: int, largest_tokens: int) -> int:
        """Device memory that the graphs captured after the cache is made will take: their shared logits
        and workspace, the fixed-shape step arrays, and the graph objects themselves."""
        if not self.graphs_enabled:
            return 0
        max_batch = min(self.cfg.max_num_seqs, self.cfg.max_num_batched_tokens)
        sizes = [b for b in self._graph_sizes if b < max_batch] + [next((b for b in self._graph_sizes if b >= max_batch), 0)]
        rows = max(sizes + ([_MIXED_SEQS[-1]] if self.mixed_graphs else []))
        tokens = max(sizes + ([self._mixed_tokens[-1]] if self.mixed_graphs else []))
        logits = rows * self.spec.vocab_size * 4
        workspace = int(eager_ws_bytes * min(1.0, 1.25 * tokens / max(largest_tokens, 1))) + (64 << 20)
        groups = max(1, len({n.group_key() for n in self.model.cache_needs().values() if n.kind == "pages"}))
        shapes = [(b, b) for b in sizes if b]
        if self.mixed_graphs:
            shapes += [(t, n) for n in _MIXED_SEQS for t in self._mixed_tokens]
        arrays = sum(4 * (3 * t + 4 * n + 16 + groups * n * self._table_width) for t, n in shapes)
        # a captured step of a few hundred kernels was measured at 3-5 MB of device memory; a shape has
        # one graph per context class whose launch plans differ (about two on average)
        objects = (128 << 20) + len(shapes) * 2 * 5 * (1 << 20)
        return logits + workspace + arrays + objects

    def _pages_from_free_memory(self, needs) -> int:
        """Pages per group from the memory that is left after a warm-up step of the largest size the
        scheduler can make (the reference measures the same way, after a warm-up prefill, and takes
        an estimate for its graphs off: atom/model_engine/model_runner.py:1584-1611).  The warm-up
        runs against a cache of its own, just large enough, which is given back; the activation
        buffers it sized stay, so later steps allocate nothing."""
        lens = self._largest_step()
        pages = sum(-(-n // self.page_size) for n in lens) + 1
        probe = CacheManager(needs, self.page_size, pages, len(lens))
        per_page = CacheStorage.bytes_per_page(probe, self.dtype)
        if per_page == 0:
            return 1
        storage = CacheStorage(probe, self.dtype, self.device)
        builder = StepBuilder(probe, self.device, self.spec.vocab_size, self.status)
        entries = [StepEntry(("warm-up", i), [0] * n, (n - 1,)) for i, n in enumerate(lens)]
        for e in entries:
            probe.admit(e.rid)
            probe.extend(e.rid, len(e.tokens))
        with torch.no_grad():
            self.model.forward(builder.build(entries, [len(e.tokens) for e in entries]), storage)
        torch.cuda.synchronize(self.device)
        self.check_status()
        ws_bytes = self.rt.workspace.bytes()
        del storage, builder, probe
        torch.cuda.empty_cache()
        free, total = torch.cuda.mem_get_info(self.device)
        reserve = self._graph_memory_bound(ws_bytes, sum(lens))
        self.memory.update(activations=ws_bytes, graph_reserve=reserve, in_use_before_cache=total - free)
        budget = total * self.cfg.gpu_memory_utilization - (total - free) - reserve
        n = int(budget // per_page)
        if n < 1:
            raise RuntimeError("no device memory left for the cache")
        return n

    # ------------------------------------------------------------------ the step

    def _validate(self, entries: Sequence[StepEntry]) -> None:
        """Everything about a step that can be refused is refused here, before a page is taken: a
        step that raises StepError leaves the cache as it was."""
        seen = set()
        V = self.spec.vocab_size
        for e in entries:
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.rid!r} brings no tokens")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.rid!r}: wanted place {w} outside its {n} tokens")
            toks = np.asarray(e.tokens, dtype=np.int64)
            if toks.ndim != 1 or toks.min() < 0 or toks.max() >= V:
                raise StepError(f"request {e.rid!r}: token id outside [0, {V})")
            e.tokens = toks       # (the arrays are built from this copy)

    def _reserve(self, entries: Sequence[StepEntry]) -> List[int]:
        """Admits new requests and takes the pages this step needs; all or nothing."""
        cache = self.cache
        need_total: Dict[int, int] = {}
        new_slots = 0
        targets = []
        for e in entries:
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
        self._validate(entries)
        size = self._graph_size(entries)
        if size and any(tuple(e.want) not in ((), (0,)) for e in entries):
            size = 0          # (a row wanted twice: the general path takes any list)
        if device_tokens is not None:
            rows = None if device_token_rows is None else [int(r) for r in device_token_rows]
            n_src = device_tokens.numel()
            if not size or device_tokens.dtype != torch.int32 or (
                    n_src != len(entries) if rows is None
                    else len(rows) != len(entries) or any(not 0 <= r < n_src for r in rows)):
                raise StepError("device_tokens needs a captured decode step and one int32 token per entry")
        targets = self._reserve(entries)
        shape = None if size or device_tokens is not None else self._mixed_shape(entries)
        with self._labelled(entries, targets, size, shape):
            if device_tokens is not None:
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

    def _labelled(self, entries, targets, size, shape):
        """While a profiler records (``profiling``), every step is a range of its own in the trace, named by
        ``step_label``; otherwise nothing."""
        if not self.profiling:
            return contextlib.nullcontext()
        return torch.profiler.record_function(step_label(
            [len(e.tokens) for e in entries], targets, graph_batch=size or None, graph_shape=shape))

    @property
    def h2d_bytes(self) -> int:
        """Bytes of step metadata copied host -> device so far."""
        return self.builder.h2d_bytes

    # ------------------------------------------------------------------ captured steps

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

    def _context_class(self, longest: int) -> int:
        """Launch plans of a captured step are made for a longest context; steps replay the graph of
        the class their own longest context falls into: 256, 1024, 4096, ... up to max_model_len."""
        c = 256
        while c < longest:
            c *= 4
        return min(c, max(self.max_model_len, 1))

    @property
    def graph_shapes(self) -> set:
        """Shapes (batch sizes and (tokens, requests) pairs) that have a captured graph."""
        return {k[0] for k in self._graphs}

    def _fixed_context(self, shape, ctx_class: int):
        if isinstance(shape, tuple):
            return self.builder.fixed_context_mixed(shape[0], shape[1], self._table_width, ctx_class)
        return self.builder.fixed_context(shape, self._table_width, ctx_class)

    def _graph_for(self, shape, longest: int) -> "_DecodeGraph":
        """The graph of ``shape`` (a batch size, or (tokens, requests)) for steps whose longest context is
        ``longest``, captured now if no step has needed it yet.  Context classes whose launch plans come
        out equal share one graph."""
        cls = self._context_class(longest)
        key = self._graph_keys.get((shape, cls))
        if key is None:
            key = self._graph_keys[(shape, cls)] = (shape, self.model.plan_signature(self._fixed_context(shape, cls)))
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = self._capture(shape, cls)
        return g

    def _capture(self, shape, ctx_class: int) -> "_DecodeGraph":
        """Runs a step of ``shape`` made of padding alone once eagerly (loads kernels, sizes the
        buffers), then records the same launches into a graph.  Graphs write their activations to a
        workspace and their logits to a buffer that all graphs of this runner share."""
        mixed = isinstance(shape, tuple)
        rows = shape[1] if mixed else shape
        g = _DecodeGraph()
        if self._graph_logits is None or self._graph_logits.shape[0] < rows:
            max_batch = min(self.cfg.max_num_seqs, self.cfg.max_num_batched_tokens)
            most = max([b for b in self._graph_sizes if b <= max(rows, max_batch)] + [rows] +
                       ([_MIXED_SEQS[-1]] if self.mixed_graphs else []))
            self._graph_logits = torch.empty((most, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        g.logits = self._graph_logits
        saved = self.rt.workspace
        self.rt.workspace = self._graph_ws
        try:
            def run():
                ctx = self._fixed_context(shape, ctx_class)
                ctx.logits_out = g.logits
                self.model.forward(ctx, self.storage)

            if mixed:
                self.builder.build_fixed_mixed([], [], shape[0], shape[1], self._table_width)   # all padding
            else:
                self.builder.build_fixed([], [], shape, self._table_width)
            run()
            torch.cuda.current_stream().synchronize()
            g.graph = torch.cuda.CUDAGraph()
            before = native.launches
            with torch.cuda.graph(g.graph):
                run()
            g.num_launches = native.launches - before     # own kernels recorded in the graph
        finally:
            self.rt.workspace = saved
        return g

    def capture_graphs(self, max_batch: int) -> list:
        """Captures, ahead of the first request, the graphs that steps of up to ``max_batch`` requests
        replay (the reference captures all of its sizes at start, atom/model_engine/model_runner.py
        capture_cudagraph), for every context class up to max_model_len; without this call a graph is
        captured when a step first needs it (which stalls that step by ~0.1 s).  The largest shapes
        come first, so that the shared buffers are sized once.  Returns the keys captured now."""
        done = []
        if not self.graphs_enabled:
            return done
        free0 = torch.cuda.mem_get_info(self.device)[0]
        shapes: list = []
        for b in self._graph_sizes:
            shapes.append(b)
            if b >= max_batch:
                break
        if self.mixed_graphs:
            for n in _MIXED_SEQS:
                shapes += [(t, n) for t in self._mixed_tokens]
                if n >= max_batch:
                    break
        classes, c = [], 256
        while True:
            classes.append(self._context_class(c))
            if c >= self.max_model_len:
                break
            c *= 4
        shapes.sort(key=lambda sh: (sh[0] if isinstance(sh, tuple) else sh), reverse=True)
        for sh in shapes:
            for c in sorted(set(classes), reverse=True):
                n = len(self._graphs)
                self._graph_for(sh, c)
                if len(self._graphs) > n:
                    done.append((sh, c))
        torch.cuda.synchronize(self.device)
        self.memory["graphs"] = free0 - torch.cuda.mem_get_info(self.device)[0]
        return done

    def _step_mixed_graph(self, entries: Sequence[StepEntry], targets: List[int], shape) -> torch.Tensor:
        g = self._graph_for(shape, max(targets))
        self.builder.build_fixed_mixed(entries, targets, shape[0], shape[1], self._table_width)
        g.graph.replay()
        native.add_launches(g.num_launches)
        self.graph_replays += 1
        return g.logits[: sum(len(e.want) for e in entries)]       # valid until the next captured step

    def _step_graph(self, entries: Sequence[StepEntry], targets: List[int], size: int,
                    device_tokens: Optional[torch.Tensor] = None,
                    device_token_rows: Optional[List[int]] = None) -> torch.Tensor:
        g = self._graph_for(size, max(targets))
        ctx = self.builder.build_fixed(entries, targets, size, self._table_width, device_token_rows)
        if device_tokens is not None:          # on the stream, after the arrays' copy
            if device_token_rows is not None:
                device_tokens = device_tokens.index_select(0, ctx.token_ids[: len(entries)])
            ctx.token_ids[: len(entries)].copy_(device_tokens)
        g.graph.replay()
        native.add_launches(g.num_launches)
        self.graph_replays += 1
        rows = [i for i, e in enumerate(entries) if len(e.want)]
        if rows == list(range(len(entries))):
            return g.logits[: len(entries)]       # valid until the next captured step
        if not rows:
            return g.logits[:0]
        return g.logits[torch.tensor(rows, device=self.device)]

    def finish(self, rid: Hashable) -> None:
        """The request is over (or preempted): its pages and its state slot go back."""
        if rid in self.cache.requests:
            self.cache.release(rid)

    def check_status(self) -> None:
        """Raises if a kernel met a position without a page or gave up a bounded wait since the
        last check (synchronises the device)."""
        try:
            native.check_error_flags()
        except native.NativeError as e:
            raise StepError(str(e)) from e

    def raise_for_flags(self, values: Sequence[int]) -> None:
        """``values``: a host copy of ``self.flags`` taken after a step.  Raises, and clears the device
        flags, if one is set: the step's results (and the cache) are not to be trusted."""
        if any(values):
            self.flags.zero_()
            raise StepError("; ".join(m for m, x in zip(native.FLAG_MESSAGES, values) if x))
