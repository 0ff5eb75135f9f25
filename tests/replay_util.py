"""Replays a trace through the engine's runner in-process (what bin/trace_run does, minus
the files) and computes the plain implementation's logits for the same requests."""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np

import plain_qwen3 as plain


def make_runner(model_dir: str, dtype: str, max_tokens: int, page: int = 16, max_num_seqs: int = 16):
    from atom_b200.config import EngineConfig
    from atom_b200.engine.runner import ModelRunner

    cfg = EngineConfig(model=model_dir, dtype=dtype, kv_cache_block_size=page,
                       num_kvcache_blocks=max(1, -(-max_tokens // page)), max_num_seqs=max_num_seqs,
                       enforce_eager=True)
    return ModelRunner(cfg)


def replay(runner, steps: List[dict]) -> Dict[int, np.ndarray]:
    from atom_b200.engine.batch import StepEntry

    out = {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in s["entries"]]
        logits = runner.step(entries)
        runner.check_status()
        if logits.shape[0]:
            out[s["step"]] = logits.float().cpu().numpy()
        for rid in s.get("end", []):
            runner.finish(rid)
        runner.cache.check()
    return out


_plain_cache: Dict = {}


def plain_logits(model_dir: str, seqs: Dict[str, Sequence[int]]) -> Dict[str, np.ndarray]:
    key = model_dir
    if key not in _plain_cache:
        _plain_cache[key] = (plain.read_config(model_dir), plain.read_tensors(model_dir), {})
    cfg, w, memo = _plain_cache[key]
    out = {}
    for rid, toks in seqs.items():
        k = tuple(toks)
        if k not in memo:
            memo[k] = plain.forward(cfg, w, toks).numpy()
        out[rid] = memo[k]
    return out


def max_err(got: Dict[str, np.ndarray], ref: Dict[str, np.ndarray]):
    """(largest absolute error, request, position) over all requests."""
    worst = (0.0, None, -1)
    for rid, r in ref.items():
        g = got[rid]
        assert g.shape == r.shape, f"{rid}: got {g.shape}, want {r.shape}"
        assert np.isfinite(g).all(), f"{rid}: non-finite logits"
        e = np.abs(g.astype(np.float64) - r).max(axis=1)
        i = int(e.argmax())
        if e[i] > worst[0]:
            worst = (float(e[i]), rid, i)
    return worst
