"""Makes tests/golden/rope_silu.json: outputs of the functions of ROCm/ATOM's model code
that are plain torch and can run on a CPU, for fixed seeded inputs.

    python tests/golden/make_golden.py /path/to/ROCm-ATOM-checkout

The reference's model modules import the AMD-only ``aiter`` package at module level, so they
cannot be imported here (the stub in the reference's tests/aiter_stub.py answers every
``aiter`` name with a mock, so a model imported against it computes nothing).  This script
reads the function definitions out of the reference's source files with ``ast`` and executes
them unchanged in a namespace that holds only torch:
    apply_rotary_emb            atom/model_ops/rotary_embedding.py:14-24
    SiluAndMul.forward_native   atom/model_ops/activation.py:78-82
    rms_norm_ref                atom/model_ops/fla_ops/layernorm_guard.py:44-73  (the reference's
                                plain RMSNorm; without gate, bias or groups it is the formula of the
                                aiter kernel that atom/model_ops/layernorm.py:57-63 calls)
Everything else of the plain implementation (tests/plain_qwen3.py) rests on the reference's
formulas; tests/test_golden.py compares the plain implementation with this file.
"""
import ast
import json
import os
import sys

import torch
import torch.nn.functional as F


def _function_source(path, name, cls=None):
    with open(path) as f:
        src = f.read()
    tree = ast.parse(src)
    nodes = tree.body
    if cls is not None:
        nodes = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == cls).body
    fn = next(n for n in nodes if isinstance(n, ast.FunctionDef) and n.name == name)
    return ast.get_source_segment(src, fn), fn.lineno, fn.end_lineno


def main(ref_root):
    ns = {"torch": torch, "F": F, "Optional": __import__("typing").Optional}
    rope_src, a, b = _function_source(os.path.join(ref_root, "atom/model_ops/rotary_embedding.py"), "apply_rotary_emb")
    exec(rope_src, ns)
    silu_src, c, d = _function_source(os.path.join(ref_root, "atom/model_ops/activation.py"), "forward_native",
                                      cls="SiluAndMul")
    exec("import textwrap\n", ns)
    import textwrap
    exec(textwrap.dedent(silu_src), ns)

    norm_src, e, f = _function_source(os.path.join(ref_root, "atom/model_ops/fla_ops/layernorm_guard.py"), "rms_norm_ref")
    exec(norm_src, ns)

    g = torch.Generator().manual_seed(1234)
    T, heads, hd, theta = 5, 3, 16, 10000.0
    x = torch.randn((T, heads, hd), generator=g, dtype=torch.float32)
    positions = torch.tensor([0, 1, 7, 100, 1000])
    # the table as the reference forms it (atom/model_ops/rotary_embedding.py:58-80)
    inv_freq = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float) / hd))
    freqs = torch.einsum("i,j -> ij", positions.to(torch.float), inv_freq)
    rope_out = ns["apply_rotary_emb"](x, freqs.cos(), freqs.sin())
    gu = torch.randn((4, 12), generator=g, dtype=torch.float32) * 3
    silu_out = ns["forward_native"](None, gu)
    nx = torch.randn((6, 40), generator=g, dtype=torch.float32) * 2.5
    nweight = 1.0 + 0.3 * torch.randn((40,), generator=g, dtype=torch.float32)
    neps = 3e-5
    norm_out = ns["rms_norm_ref"](nx, nweight, None, eps=neps)
    out = {
        "source": {"apply_rotary_emb": f"atom/model_ops/rotary_embedding.py:{a}-{b}",
                   "SiluAndMul.forward_native": f"atom/model_ops/activation.py:{c}-{d}",
                   "rms_norm_ref": f"atom/model_ops/fla_ops/layernorm_guard.py:{e}-{f}"},
        "rms_norm": {"x": nx.tolist(), "weight": nweight.tolist(), "eps": neps, "out": norm_out.tolist()},
        "rope": {"x": x.tolist(), "positions": positions.tolist(), "theta": theta, "out": rope_out.tolist()},
        "silu_and_mul": {"x": gu.tolist(), "out": silu_out.tolist()},
    }
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rope_silu.json")
    with open(path, "w") as f:
        json.dump(out, f)
    print("wrote", path)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/ROCm-ATOM-checkout")
    main(sys.argv[1])
