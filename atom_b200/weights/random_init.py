"""Random weights: a model folder written from a configuration and a seed, and a fast
on-device fill for benchmarks.

Distributions: matrices and embeddings N(0, 0.02^2), norm weights U(0.8, 1.2), biases 0.
The folder writer draws every checkpoint tensor in the spec's order from one CPU generator
in 32-bit and stores bfloat16, so the 32-bit and the bfloat16 engine read the same values.
(The reference's dummy weights are unseeded xavier/ones, atom/model_loader/loader.py:178-227.)
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..config.model_config import ModelConfig, save_model_config
from ..models.model import Model
from ..models.registry import build_model_spec
from .loader import expected_tensors

_STD = 0.02
_NORM_LO, _NORM_HI = 0.8, 1.2


def _draw(shape, init: str, gen: torch.Generator, device="cpu") -> torch.Tensor:
    if init == "normal":
        return torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * _STD
    if init == "norm":
        return torch.rand(shape, generator=gen, dtype=torch.float32, device=device) * (_NORM_HI - _NORM_LO) + _NORM_LO
    if init == "zeros":
        return torch.zeros(shape, dtype=torch.float32, device=device)
    raise ValueError(f"unknown init '{init}'")


def write_random_model(model_dir: str, config: ModelConfig, seed: int, dtype: torch.dtype = torch.bfloat16) -> None:
    """Writes ``config.json`` and ``model.safetensors`` with seeded random weights."""
    from safetensors.torch import save_file

    model = Model(build_model_spec(config))
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    tensors: Dict[str, torch.Tensor] = {}
    for name, (_, _, _, shape, ps) in expected_tensors(model).items():
        tensors[name] = _draw(shape, ps.init, gen).to(dtype).contiguous()
    os.makedirs(model_dir, exist_ok=True)
    save_model_config(config, model_dir)
    save_file(tensors, os.path.join(model_dir, "model.safetensors"), metadata={"format": "pt"})


def random_weights_on_device(model: Model, seed: int, compute: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """Fills every parameter on the device from a device generator (same distributions as the
    folder writer, other values): for models too large to write to disk first."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for path, part, _ in model.named_parts():
        for name, ps in part.params().items():
            dt = torch.int32 if ps.role == "table" else (
                torch.float32 if compute == torch.float32 else torch.bfloat16)
            t = torch.empty(ps.shape, dtype=dt, device=device)
            # Draw in slabs to bound the 32-bit temporary for very large matrices.
            rows = ps.shape[0]
            slab = max(1, (64 << 20) // max(1, t[0].numel() if t.dim() > 1 else 1))
            for r0 in range(0, rows, slab):
                r1 = min(rows, r0 + slab)
                t[r0:r1].copy_(_draw((r1 - r0,) + tuple(ps.shape[1:]), ps.init, gen, device))
            out[f"{path}.{name}"] = t
    return out


def main(argv=None) -> int:
    """``python -m atom_b200.weights --config DIR_OR_JSON --seed N --out DIR``: a model
    folder with the architecture and sizes of the given config.json and seeded random weights."""
    import argparse
    import shutil
    import tempfile

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--config", required=True, help="a config.json, or a folder that holds one")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", required=True)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="storage type of the tensors")
    args = ap.parse_args(argv)
    from ..config.model_config import load_model_config

    src = args.config
    if os.path.isfile(src):        # load_model_config reads <folder>/config.json
        tmp = tempfile.mkdtemp()
        try:
            shutil.copy(src, os.path.join(tmp, "config.json"))
            config = load_model_config(tmp)
        finally:
            shutil.rmtree(tmp, ignore_errors=True)
    else:
        config = load_model_config(src)
    write_random_model(args.out, config, args.seed, torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    print(f"wrote {args.out}: {config.architecture}, seed {args.seed}")
    return 0

