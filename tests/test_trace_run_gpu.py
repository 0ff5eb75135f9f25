"""bin/trace_run as a user runs it: a child process that reads steps from standard input,
writes <step>.f32 files and prints ``done <step>``; its logits against the plain
implementation, for a trace that mixes portions with decoded tokens and re-uses pages."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import tiny
import traces
from replay_util import max_err, plain_logits

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_dirs, tmp_path, dtype):
    name = "B"
    ps = tiny.prompts(name, [3, 29, 64, 100, 131], seed=3)
    seqs = {f"r{i}": p for i, p in enumerate(ps)}
    steps, peak = traces.mixed(seqs, max_live=4, budget_tokens=320)
    total = sum(-(-len(t) // 64) * 64 for t in seqs.values())
    assert peak < total            # pages must be used again
    out = tmp_path / f"out_{dtype}"
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs[name],
                        "--dtype", dtype, "--out", str(out), "--max-tokens", str(peak)],
                       input=text, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    done = [int(l.split()[1]) for l in p.stdout.splitlines() if l.startswith("done ")]
    assert done == [s["step"] for s in steps]
    V = tiny.CONFIGS[name]["vocab_size"]
    outputs = {}
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        f = out / f"{s['step']}.f32"
        if n == 0:
            assert not f.exists()
            continue
        a = np.fromfile(f, dtype="<f4")
        assert a.size == n * V
        outputs[s["step"]] = a.reshape(n, V)
    got = traces.collect(steps, outputs)
    ref = plain_logits(model_dirs[name], seqs)
    err, rid, pos = max_err(got, ref)
    scale = max(float(np.abs(r).max()) for r in ref.values())
    tol = 1e-4 * max(1.0, scale) if dtype == "float32" else 8e-2 * scale
    assert err <= tol, f"{dtype}: max abs error {err:.3e} at {rid}[{pos}]"
