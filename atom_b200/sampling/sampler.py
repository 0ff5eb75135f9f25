"""Turns logits into token ids on the device: greedy, temperature (the exponential race of
atom/model_ops/sampler.py:104-132) and top-k / top-p (:134-295), one kernel for all rows."""
from __future__ import annotations

import ctypes
from typing import Sequence

import numpy as np
import torch

from .. import native
from .params import SamplingParams

_vp, _i = ctypes.c_void_p, ctypes.c_int
native.declare("atom_sample", [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp])
native.declare("atom_sample_simple", [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp])
native.declare("atom_token_logprob", [_vp, _vp, _vp, _i, _i, _vp])


class Sampler:
    def __init__(self, device, default_seed: int = 0):
        self.device = torch.device(device)
        self.default_seed = default_seed
        self._probs = None
        self._part = None
        self._pinned = None
        self._events = [None] * 4
        self._next = 0
        self.h2d_bytes = 0

    def _staging(self, R: int):
        """A pinned host array [5, R] from a ring: written again only after its copy is done."""
        if self._pinned is None or self._pinned[0].numel() < 5 * R:
            n = max(5 * R, 5 * 64)
            self._pinned = [torch.zeros(n, dtype=torch.float32).pin_memory() for _ in range(4)]
            self._events = [None] * 4
        k = self._next
        self._next = (k + 1) % 4
        if self._events[k] is not None:
            self._events[k].synchronize()
        return self._pinned[k].numpy()[: 5 * R].reshape(5, R), k

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               indices: Sequence[int]) -> torch.Tensor:
        """logits [R, V] float32 on the device.  seeds[r] is the request's random stream,
        indices[r] counts the tokens the request has generated so far.  Returns int32 [R]."""
        R, V = logits.shape
        assert logits.dtype == torch.float32 and logits.is_contiguous() and len(params) == R
        host, k = self._staging(R)
        hi = host.view(np.uint32)
        any_filter = False
        for r, p in enumerate(params):
            host[0, r] = p.temperature
            hi[1, r] = seeds[r] & 0xFFFFFFFF
            hi[2, r] = indices[r] & 0xFFFFFFFF
            host.view(np.int32)[3, r] = p.top_k
            host[4, r] = p.top_p
            any_filter = any_filter or (p.filters and not p.greedy)
        dev = torch.empty((5, R), dtype=torch.float32, device=self.device)
        dev.copy_(self._pinned[k][: 5 * R].view(5, R), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[k] = ev
        self.h2d_bytes += host.nbytes
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        if not any_filter:
            # one argmax per row: many blocks scan pieces of the vocabulary at once
            chunks = max(1, min(64, (2 * native.sm_count()) // R, -(-V // 1024)))
            if self._part is None or self._part.numel() < R * chunks * 2:
                self._part = torch.empty(max(R * chunks * 2, 4096), dtype=torch.float32, device=self.device)
            code = native.lib().atom_sample_simple(
                out.data_ptr(), logits.data_ptr(), dev[0].data_ptr(), dev[1].data_ptr(), dev[2].data_ptr(),
                self._part.data_ptr(), chunks, R, V, torch.cuda.current_stream().cuda_stream)
            native._check(code, "sample_simple")
            native.add_launches(1)          # (the chunks' kernel and the one that picks among them)
            return out
        probs = None
        if any_filter:
            if self._probs is None or self._probs.numel() < R * V:
                self._probs = torch.empty(R * V, dtype=torch.float32, device=self.device)
            probs = self._probs
        code = native.lib().atom_sample(
            out.data_ptr(), logits.data_ptr(), dev[0].data_ptr(), dev[1].data_ptr(), dev[2].data_ptr(),
            dev[3].data_ptr() if any_filter else None, dev[4].data_ptr() if any_filter else None,
            probs.data_ptr() if probs is not None else None, R, V,
            torch.cuda.current_stream().cuda_stream)
        native._check(code, "sample")
        return out

    def logprobs(self, logits: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """float32 [R]: log-probability of ids[r] under softmax(logits[r]) (the raw distribution, before
        temperature and filters: what the reference reports, atom/model_engine/model_runner.py:3233-3240)."""
        R, V = logits.shape
        assert logits.dtype == torch.float32 and logits.is_contiguous() and ids.dtype == torch.int32 and ids.numel() == R
        out = torch.empty(R, dtype=torch.float32, device=self.device)
        native._check(native.lib().atom_token_logprob(out.data_ptr(), logits.data_ptr(), ids.data_ptr(), R, V,
                                                      native._stream()), "token_logprob")
        return out
