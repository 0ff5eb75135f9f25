"""The plain implementation against outputs of the reference's own code (the functions of its
model code that run on a CPU; made by tests/golden/make_golden.py)."""
import json
import os

import torch

import plain_qwen3 as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rope_silu.json")


def test_rope_matches_reference_function():
    g = json.load(open(GOLDEN))["rope"]
    x = torch.tensor(g["x"], dtype=torch.float32)
    cos, sin = plain.rope_cos_sin(torch.tensor(g["positions"]), x.shape[-1], g["theta"])
    got = plain.apply_rope(x, cos, sin)
    assert torch.allclose(got, torch.tensor(g["out"]), rtol=0, atol=1e-6)


def test_silu_and_mul_matches_reference_function():
    g = json.load(open(GOLDEN))["silu_and_mul"]
    got = plain.silu_and_mul(torch.tensor(g["x"], dtype=torch.float32))
    assert torch.allclose(got, torch.tensor(g["out"]), rtol=1e-6, atol=1e-6)


def test_rms_norm_matches_reference_function():
    g = json.load(open(GOLDEN))["rms_norm"]
    got = plain.rms_norm(torch.tensor(g["x"], dtype=torch.float32), torch.tensor(g["weight"]), g["eps"])
    assert torch.allclose(got, torch.tensor(g["out"]), rtol=1e-6, atol=1e-6)
