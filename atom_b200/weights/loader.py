"""Reads a model's parameters from safetensors by tensor name.

What to read comes from the ModelSpec: every part lists its parameters and the spec maps
each to one checkpoint tensor or to several stacked along dim 0 (q/k/v, gate/up; the row
layout of atom/model_ops/linear.py:1830-1863 and :1252-1285).  Types: matrices are kept in
the compute type (bfloat16, or float32 in the 32-bit mode); a vector stored in 32-bit stays
32-bit; integer tables become int32.  Anything that does not fit is reported in ONE error
that lists missing tensors, unexpected tensors and wrong shapes together (the reference only
warns, atom/model_loader/loading_core.py:411-468).  A tensor that the spec names as a duplicate
of another (the output matrix of a tied model) may be present if it equals that other tensor.
After the tensors are bound, every part's ``after_load`` runs once (the reference's
process_weights_after_loading, atom/model_loader/loader.py:354-360).
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Dict, List, Tuple

import torch

from ..models.model import Model
from ..parts.spec import ParamSpec


class WeightError(RuntimeError):
    """The checkpoint does not match the model; lists every mismatch."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong
        lines = [f"{where}: checkpoint does not match the model"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


class WeightFileError(RuntimeError):
    """A checkpoint file cannot be read at all (cut off, or not safetensors)."""


def expected_tensors(model: Model) -> Dict[str, Tuple[str, str, int, Tuple[int, ...], ParamSpec]]:
    """checkpoint tensor name -> (parameter key, param name, offset along the parameter's stack_dim,
    expected shape, spec)."""
    out: Dict[str, Tuple[str, str, int, Tuple[int, ...], ParamSpec]] = {}
    for path, part, pspec in model.named_parts():
        for name, ps in part.params().items():
            srcs = pspec.sources.get(name)
            if srcs is None:
                raise ValueError(f"{path}.{name}: the architecture names no checkpoint tensor for it")
            d = ps.stack_dim
            if not 0 <= d < len(ps.shape):
                raise ValueError(f"{path}.{name}: stack_dim {d} for a tensor of shape {ps.shape}")
            rows = ps.rows if ps.rows is not None else (ps.shape[d],)
            if len(rows) != len(srcs) or sum(rows) != ps.shape[d]:
                raise ValueError(f"{path}.{name}: {len(srcs)} source tensors for the split {rows} of axis {d}")
            off = 0
            for src, r in zip(srcs, rows):
                out[src] = (f"{path}.{name}", name, off, tuple(ps.shape[:d]) + (r,) + tuple(ps.shape[d + 1:]), ps)
                off += r
    return out


def _checkpoint_files(model_dir: str) -> List[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        # Every shard the index names must exist (atom/model_loader/loading_core.py:53-88).
        with open(index) as f:
            names = sorted(set(json.load(f).get("weight_map", {}).values()))
        files = [os.path.join(model_dir, n) for n in names]
        gone = [f for f in files if not os.path.isfile(f)]
        if gone:
            raise FileNotFoundError(f"{model_dir}: shards named by the index are missing: {gone}")
        return files
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"{model_dir}: no .safetensors file")
    return files


def _target_dtype(ps: ParamSpec, stored: List[torch.dtype], compute: torch.dtype) -> torch.dtype:
    if ps.role == "table":
        return torch.int32
    if ps.role == "vector":
        if compute == torch.float32 or all(d == torch.float32 for d in stored):
            return torch.float32
        return torch.bfloat16
    return compute


def load_weights(model: Model, model_dir: str, compute: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """Returns '<part path>.<param>' -> tensor on ``device``; raises WeightError on any mismatch."""
    from safetensors import safe_open

    want = expected_tensors(model)
    ignored = [re.compile(p) for p in model.spec.ignored_tensors]
    handles, where = [], {}
    for f in _checkpoint_files(model_dir):
        try:
            h = safe_open(f, framework="pt", device="cpu")
        except Exception as e:       # a cut-off or foreign file: say which one
            raise WeightFileError(f"{f}: not a readable safetensors file ({e})") from e
        handles.append(h)
        for k in h.keys():
            where[k] = h
    missing = sorted(n for n in want if n not in where)
    duplicates = {n: other for n, other in model.spec.duplicate_tensors if n not in want}
    unexpected = sorted(
        n for n in where if n not in want and n not in duplicates and not any(p.match(n) for p in ignored)
    )
    wrong, stored_dtypes = [], {}
    for n, other in duplicates.items():
        if n in where and other in where:
            a, b = where[n].get_tensor(n), where[other].get_tensor(other)
            if a.shape != b.shape or a.dtype != b.dtype or not torch.equal(a, b):
                wrong.append(f"{n}: the model uses {other} in its place, but the file's {n} differs from it")
    for n, (key, _, _, shape, _) in want.items():
        if n in where:
            sl = where[n].get_slice(n)
            got = tuple(sl.get_shape())
            if got != tuple(shape):
                wrong.append(f"{n}: file has {list(got)}, model needs {list(shape)}")
            stored_dtypes.setdefault(key, []).append(_st_dtype(sl.get_dtype()))
    if missing or unexpected or wrong:
        raise WeightError(model_dir, missing, unexpected, sorted(wrong))

    out: Dict[str, torch.Tensor] = {}
    specs = {}
    for n, (key, _, off, shape, ps) in want.items():
        specs[key] = ps
    for key, ps in specs.items():
        dt = _target_dtype(ps, stored_dtypes[key], compute)
        out[key] = torch.empty(ps.shape, dtype=dt, device=device)
    for n, (key, _, off, shape, ps) in want.items():
        t = where[n].get_tensor(n)
        dst = out[key]
        d = ps.stack_dim
        dst.narrow(d, off, shape[d]).copy_(t.to(dst.dtype) if t.dtype != dst.dtype else t)
    return out


def _st_dtype(name: str) -> torch.dtype:
    return {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
            "I32": torch.int32, "I64": torch.int64}.get(name, torch.float32)
