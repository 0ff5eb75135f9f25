"""The kernels of one decode step on a time line, taken with the engine's own profiler hook.

    python -m atom_b200.benchmarks.timeline [--batch 8] [--context 4096] [--layers 36]

Builds an engine with random weights at Qwen3-8B's sizes (or the sizes given), fills ``batch``
requests to the context length, runs decode steps from the captured CUDA graph and records a
few of them with ``LLMEngine.start_profile`` / ``stop_profile``.  For every kernel of one step
it prints when it began, how long it ran and its *exposed* time: how much later it ended than
everything before it.  With programmatic dependent launch a kernel begins (and loads what does
not depend on its predecessor) while the one in front still runs, so durations overlap and
only the exposed times add up to the step.
"""
from __future__ import annotations

import argparse
import gzip
import json
import re
import tempfile

import numpy as np
import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--intermediate", type=int, default=12288)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--per-layer", action="store_true", help="print one layer's kernels and the per-layer sums only")
    args = ap.parse_args(argv)

    from atom_b200 import LLMEngine, SamplingParams
    from atom_b200.config import config_from_dict
    from atom_b200.engine.batch import StepEntry

    cfg = config_from_dict({
        "architectures": ["Qwen3ForCausalLM"], "hidden_size": args.hidden, "num_hidden_layers": args.layers,
        "num_attention_heads": args.heads, "num_key_value_heads": args.kv_heads, "head_dim": args.head_dim,
        "intermediate_size": args.intermediate, "vocab_size": args.vocab, "rms_norm_eps": 1e-6,
        "rope_theta": 1000000.0, "max_position_embeddings": max(40960, args.context + 8), "hidden_act": "silu",
        "tie_word_embeddings": False, "attention_bias": False, "torch_dtype": "bfloat16"})
    B, ctx = args.batch, args.context
    out_dir = tempfile.mkdtemp()
    eng = LLMEngine("", model_config=cfg, dtype="bfloat16", load_dummy="random", seed=4, kv_cache_block_size=args.page,
                    num_kvcache_blocks=B * (ctx // args.page + 2) + 16, max_num_seqs=max(64, B),
                    max_num_batched_tokens=8192, max_model_len=ctx + 8, torch_profiler_dir=out_dir)
    runner, rng = eng.runner, np.random.default_rng(1)
    ids = [f"d{i}" for i in range(B)]
    for rid in ids:
        toks = rng.integers(0, args.vocab, size=ctx - 40).tolist()
        for s in range(0, len(toks), 4096):
            runner.step([StepEntry(rid, toks[s:s + 4096], ())])
    sp = SamplingParams(temperature=0.0, max_tokens=1 << 30, ignore_eos=True)

    def one(i):
        logits = runner.step([StepEntry(rid, [int(rng.integers(0, args.vocab))], (0,)) for rid in ids])
        eng.sampler.sample(logits, [sp] * B, [0] * B, [i] * B)

    for i in range(6):
        one(i)
    torch.cuda.synchronize()
    eng.start_profile()
    for i in range(6, 11):
        one(i)
    torch.cuda.synchronize()
    path = eng.stop_profile()
    with gzip.open(path) as f:
        events = [e for e in json.load(f)["traceEvents"] if e.get("cat") == "kernel"]
    events.sort(key=lambda e: e["ts"])

    def short(name):
        return re.sub(r"\(.*", "", name).replace("atom::", "").replace("void ", "")[:52]

    firsts = [i for i, e in enumerate(events) if "embedding" in e["name"]]
    if len(firsts) < 4:
        print("the profiler recorded no complete step")
        return 1
    step = events[firsts[2]:firsts[3]]
    t0, end = step[0]["ts"], step[0]["ts"]
    rows, exposed_by_kernel = [], {}
    for e in step:
        fin = e["ts"] + e["dur"]
        exposed = max(0.0, fin - end)
        end = max(end, fin)
        rows.append((short(e["name"]), e["ts"] - t0, e["dur"], exposed))
        exposed_by_kernel[short(e["name"])] = exposed_by_kernel.get(short(e["name"]), 0.0) + exposed
    span = events[firsts[3]]["ts"] - t0
    print(f"decode step, batch {B}, context {ctx}, {args.layers} layers: {span:.1f} us from the first kernel of the "
          f"step to the first of the next")
    shown = rows if not args.per_layer else rows[:2] + rows[2:2 + 9]
    print(f"{'kernel':52s} {'begin':>9s} {'ran':>8s} {'exposed':>8s}   (us)")
    for name, begin, dur, exposed in shown:
        print(f"{name:52s} {begin:9.1f} {dur:8.1f} {exposed:8.1f}")
    print("\nexposed time by kernel over the step (us), and per layer:")
    for name, v in sorted(exposed_by_kernel.items(), key=lambda kv: -kv[1]):
        print(f"{name:52s} {v:9.1f} {v / max(1, args.layers):8.2f}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
