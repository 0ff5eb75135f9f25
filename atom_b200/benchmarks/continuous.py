"""Continuous batching through the engine's own entry point: many requests arrive at once and
the scheduler works them off under a token budget per step.

    python -m atom_b200.benchmarks.continuous [--model 4b] [--requests 128] [--budget 2048]
        [--prompt-len 16 2048] [--output-len 16 512] [--temperature 1.0] [--num-kvcache-blocks N]

The model has the layer sizes named by ``--model`` with seeded random weights in bfloat16; prompt
and output lengths are uniform in the given ranges and token ids uniform over the vocabulary
(seed 6), as the reference's load generator draws them (atom/benchmarks/benchmark_serving.py:172-232),
but offline: every request is added before the first step.  Requests end at their drawn output
length (``ignore_eos``).  With ``--num-kvcache-blocks`` the pool can be made so small that requests
are preempted and computed again.

Printed as one JSON line: generated and processed tokens per second over the whole run (wall clock
around ``LLMEngine.step()`` calls, sampled ids read back to the host), the number of steps of each
kind (prompt portions only, decoded tokens only, both), a histogram of step times, time to the
first token and time per output token over the requests, preemptions, and how much of each step's
time the device had to take at least (the step's weight and cache bytes at the measured copy
bandwidth, its flops at the measured matrix throughput).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import time

import numpy as np
import torch

from .sizes import SIZES


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1400.0, "fallback"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="4b", choices=sorted(SIZES))
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--requests", type=int, default=128)
    ap.add_argument("--budget", type=int, default=2048, help="max_num_batched_tokens: tokens per step")
    ap.add_argument("--prompt-len", type=int, nargs=2, default=(16, 2048))
    ap.add_argument("--output-len", type=int, nargs=2, default=(16, 512))
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--max-num-seqs", type=int, default=512)
    ap.add_argument("--num-kvcache-blocks", type=int, default=-1, help="pages of the pool (-1: what memory allows)")
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--seed", type=int, default=6)
    ap.add_argument("--enable_prefix_caching", action="store_true")
    args = ap.parse_args(argv)

    from atom_b200 import LLMEngine, SamplingParams
    from atom_b200.config import config_from_dict

    cfg_d, weight_seed = SIZES[args.model]
    cfg_d = dict(cfg_d)
    if args.layers > 0:
        cfg_d["num_hidden_layers"] = args.layers
    mcfg = config_from_dict(cfg_d)
    V, L = cfg_d["vocab_size"], cfg_d["num_hidden_layers"]
    H, nh, nkv, hd, I = (cfg_d[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                            "head_dim", "intermediate_size"))
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * I * H
    weight_bytes = 2 * (L * per_layer + V * H)
    kv_per_token = 2 * L * nkv * hd * 2
    hbm_gbs, tflops, peaks_from = _peaks()

    rng = np.random.default_rng(args.seed)
    p_len = rng.integers(args.prompt_len[0], args.prompt_len[1] + 1, size=args.requests)
    o_len = rng.integers(args.output_len[0], args.output_len[1] + 1, size=args.requests)
    prompts = [rng.integers(0, V, size=int(n)).tolist() for n in p_len]

    eng = LLMEngine("", model_config=mcfg, dtype="bfloat16", load_dummy="random", seed=weight_seed,
                    kv_cache_block_size=args.page, num_kvcache_blocks=args.num_kvcache_blocks,
                    max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.budget,
                    max_model_len=int(args.prompt_len[1] + args.output_len[1] + 8),
                    enable_prefix_caching=args.enable_prefix_caching)

    def run(prompts, o_len):
        ids = []
        for p, n in zip(prompts, o_len):
            ids.append(eng.add_request(p, SamplingParams(temperature=args.temperature, max_tokens=int(n),
                                                         ignore_eos=True)))
        steps = []
        torch.cuda.synchronize()
        t_begin = time.perf_counter()
        while not eng.is_finished():
            n0 = eng.num_steps
            live = sum(s.num_computed for s in eng.scheduler.running)
            t0 = time.perf_counter()
            eng.step()
            t1 = time.perf_counter()
            ptok, dtok = eng.last_step_tokens if eng.num_steps > n0 else (0, 0)
            steps.append((t1 - t0, ptok, dtok, live))
        torch.cuda.synchronize()
        total = time.perf_counter() - t_begin
        eng.runner.check_status()
        outs = [eng._output(eng._seqs.pop(i)) for i in ids]
        return steps, total, outs

    # warm-up: a few short requests through every kind of step (compiles, captures graphs, touches the pool)
    run([p[:64] for p in prompts[:4]], [4] * 4)
    pre0 = eng.scheduler.num_preemptions
    steps, total, outs = run(prompts, o_len)

    gen = sum(o["num_tokens_output"] for o in outs)
    processed = sum(s[1] + s[2] for s in steps)
    kinds = {"prompt_only": 0, "decode_only": 0, "mixed": 0, "bookkeeping_only": 0}
    floor = 0.0
    for dt, ptok, dtok, live in steps:
        kinds["mixed" if ptok and dtok else "prompt_only" if ptok else "decode_only" if dtok else "bookkeeping_only"] += 1
        if ptok + dtok:
            bytes_ = weight_bytes + live * kv_per_token
            flops = 2.0 * (ptok + dtok) * (L * per_layer) + 2.0 * max(dtok, 1) * V * H
            floor += max(bytes_ / (hbm_gbs * 1e9), flops / (tflops * 1e12))
    ms = sorted(s[0] * 1e3 for s in steps)
    edges = [1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 64]
    hist, lo = {}, 0.0
    for e in edges + [float("inf")]:
        n = sum(1 for x in ms if lo <= x < e)
        if n:
            hist[f"{lo:g}-{e:g} ms"] = n
        lo = e

    def q(xs, f):
        xs = sorted(xs)
        return xs[min(len(xs) - 1, int(f * len(xs)))]

    ttft = [o["ttft"] for o in outs]
    tpot = [o["tpot"] for o in outs if o["num_tokens_output"] > 1]
    out = {
        "metric": f"continuous batching, generated tokens/s (Qwen3-{args.model.upper()} sizes, bf16, 1 B200)",
        "value": round(gen / total, 1), "unit": "tokens/s",
        "processed_tokens_per_s": round(processed / total, 1),
        "seconds": round(total, 3), "requests": args.requests,
        "prompt_tokens": int(sum(p_len)), "generated_tokens": int(gen),
        "prompt_tokens_computed": int(sum(s[1] for s in steps)),
        "steps": len(steps), "step_kinds": kinds, "step_ms_histogram": hist,
        "step_ms": {"median": round(statistics.median(ms), 3), "p90": round(q(ms, 0.9), 3), "max": round(ms[-1], 3)},
        "ttft_s": {"median": round(statistics.median(ttft), 3), "max": round(max(ttft), 3)},
        "tpot_ms": {"median": round(statistics.median(tpot) * 1e3, 3), "p90": round(q(tpot, 0.9) * 1e3, 3)},
        "preemptions": eng.scheduler.num_preemptions - pre0,
        "overlapped_steps": eng.num_overlapped,
        "device_floor_s": round(floor, 3), "floor_frac": round(floor / total, 4), "peaks": peaks_from,
        "config": {"layers": L, "hidden": H, "heads": nh, "kv_heads": nkv, "head_dim": hd, "intermediate": I,
                   "vocab": V, "page_size": args.page, "budget": args.budget, "temperature": args.temperature,
                   "pages": eng.stats()["kv_pages_total"][0], "prefix_caching": args.enable_prefix_caching},
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
