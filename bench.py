#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context C]

The model has the layer sizes of Qwen3-8B (36 layers, hidden 4096, 32 heads, 8 kv heads,
head size 128, feed-forward 12288, vocabulary 151936, untied output matrix) with seeded
random weights in bfloat16; token ids are uniform over the vocabulary.  A "step" is one
decode step of the whole batch.  Printed, as ONE JSON line:

  value      decoded tokens per second at batch B (default 8) with contexts that end at C
             (default 4096) tokens, timed on the device around K runner steps + sampling;
  e2e        the same through ``LLMEngine.step()``: host scheduling, the step's integer
             arrays copied from pinned host memory, sampled ids read back to the host;
  prefill    one prompt of 2,048 tokens through one step (logits of its last token);
  roofline   bytes the decode step has to read (every weight once, the cache of the live
             requests) / its time, against the measured copy bandwidth;
  points     decode at batch 1 and 64; prefill of 512, 8,192 and 32,768 tokens and decode at contexts
             of 1k, 16k and 32k tokens, each with its share of the peak (``_frac``).

The engine is set up as a user gets it: ``max_model_len`` is the model's max_position_embeddings
(40,960 for these sizes) and the cache pool is sized by the engine from the memory that is left.

Every weight matrix of the model (tens of GB) is read in every step, far more than the
126 MB L2 holds, so consecutive timed steps do not find their inputs in L2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from atom_b200.benchmarks.sizes import SIZES  # noqa: E402  (needs ROOT on the path)

PREFILL_TOKENS = 2048
PAGE = 16


def load_peaks():
    """Measured peaks written beside this file by the machine's owner, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi while the bench runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples = []          # (time, sm, max, power, [reasons])
        self.windows = []          # (t0, t1) of timed regions
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm, mx = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            try:
                power = float(parts[2])
            except ValueError:
                power = 0.0
            reasons = [n for n, v in zip(names, parts[3:7]) if v.lower().startswith("active")]
            self.samples.append((time.time(), sm, mx, power, reasons))

    def window(self, t0, t1):
        self.windows.append((t0, t1))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        inside = [s for s in self.samples if any(a - 0.1 <= s[0] <= b + 0.1 for a, b in self.windows)]
        use = inside or self.samples
        reasons = sorted({r for s in use for r in s[4]})
        return {"sm_mhz": statistics.median(s[1] for s in use), "sm_max_mhz": max(s[2] for s in use),
                "reasons": reasons, "samples": len(use), "power_w_max": max(s[3] for s in use)}


def model_numbers(cfg, n_layers):
    """Bytes of weights a decode step reads, cache bytes per token, and flops of a step."""
    H, nh, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    I, V = cfg["intermediate_size"], cfg["vocab_size"]
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I          # matrix elements
    vectors = 2 * H + 2 * hd
    weight_bytes = 2 * (n_layers * (per_layer + vectors) + V * H + H)
    kv_bytes_per_token = 2 * n_layers * nkv * hd * 2

    def flops(tokens, ctx_pairs, logits_rows):
        # ctx_pairs: number of (query, key) pairs the attention computes per head
        return (2.0 * tokens * n_layers * per_layer + 4.0 * n_layers * nh * hd * ctx_pairs
                + 2.0 * logits_rows * V * H)

    return weight_bytes, kv_bytes_per_token, flops


def reference_arm() -> dict:
    """The unmodified reference, installed without its dependencies under baseline/_ref.  Its
    engine imports the AMD-only ``aiter`` kernel package at module level, which exists in no
    wheel here and has no NVIDIA build, so the arm reports why it cannot run."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "atom")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip --no-deps --target baseline/_ref)"}
    sys.path.insert(0, ref)
    try:
        import importlib

        importlib.import_module("atom.model_engine.model_runner")
    except Exception as e:      # the expected outcome on this platform
        why = f"{type(e).__name__}: {e}".splitlines()[0][:160]
        return {"impl": "reference", "unavailable":
                f"ROCm/ATOM's engine cannot be imported here ({why}); every kernel it calls lives in the AMD-only aiter package"}
    finally:
        sys.path.remove(ref)
    return {"impl": "reference", "unavailable":
            "ROCm/ATOM imported, but its kernels (aiter: ROCm ASM/CK/Triton) have no NVIDIA build to run"}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--model", default="8b", choices=sorted(SIZES), help="layer sizes: Qwen3-8B (default), -4B or -32B")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--no-sweep", action="store_true",
                    help="skip the further points: prefill of 512 / 8,192 / 32,768 tokens, decode at contexts 1k / 16k / 32k")
    ap.add_argument("--max-model-len", type=int, default=0,
                    help="longest request the engine takes (default: the model's max_position_embeddings)")
    ap.add_argument("--num-kvcache-blocks", type=int, default=-1,
                    help="cache pages (default -1: sized by the engine from the memory that is left)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--only-measured-graphs", action="store_true",
                    help="capture only the decode graphs of the measured batch sizes and none for small mixed steps "
                         "(a short start-up, for runs under a profiler)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps(reference_arm()))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print("bench.py: this engine runs on one GPU; --gpus > 1 is not supported")
        return 2
    K, W = max(1, args.steps), max(3, args.warmup)

    import numpy as np
    import torch

    from atom_b200 import LLMEngine, SamplingParams, native
    from atom_b200.config import config_from_dict
    from atom_b200.engine.batch import StepEntry

    peaks = load_peaks()
    cfg_d, weight_seed = SIZES[args.model]
    cfg_d = dict(cfg_d)
    full_layers = cfg_d["num_hidden_layers"]
    n_layers = args.layers if args.layers > 0 else full_layers
    cfg_d["num_hidden_layers"] = n_layers
    mcfg = config_from_dict(cfg_d)
    V = cfg_d["vocab_size"]
    weight_bytes, kv_per_token, flops = model_numbers(cfg_d, n_layers)

    batches = [args.batch] + ([] if args.no_points else [b for b in (1, 64) if b != args.batch])
    ctx_end = args.context
    ctx_start = ctx_end - (W + K)
    assert ctx_start >= 1, "context too short for warm-up + steps"
    max_b = max(batches)
    max_model_len = args.max_model_len or cfg_d["max_position_embeddings"]
    sweep_prefill = [] if args.no_sweep else [n for n in (512, 8192, 32768) if n <= max_model_len]
    sweep_ctx = [] if args.no_sweep else [c for c in (1024, 16384, 32768) if c <= max_model_len and c != ctx_end]
    assert max(ctx_end, PREFILL_TOKENS) <= max_model_len, "--context beyond --max-model-len"

    clocks = ClockSampler(0)
    t_setup = time.time()
    # The engine as a user gets it: requests as long as the model allows, the cache sized from the memory
    # that is left after a warm-up step, graphs for every batch size captured at start.
    eng = LLMEngine("", model_config=mcfg, dtype="bfloat16", load_dummy="random", seed=weight_seed,
                    kv_cache_block_size=PAGE, num_kvcache_blocks=args.num_kvcache_blocks,
                    max_num_seqs=max(64, max_b), max_num_batched_tokens=max([8192] + sweep_prefill),
                    max_model_len=max_model_len,
                    **(dict(cudagraph_capture_sizes=sorted(batches), cudagraph_mixed_steps=False)
                       if args.only_measured_graphs else {}))
    runner = eng.runner
    rng = np.random.default_rng(8)
    sp_greedy = SamplingParams(temperature=0.0, max_tokens=1 << 30, ignore_eos=True)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    def prefill_run(n_tokens, warm=3, reps=5):
        """Median device time of one step that runs a prompt of n_tokens whole (logits of its last token)."""
        prompt = rng.integers(0, V, size=n_tokens).tolist()
        times = []
        for i in range(warm + reps):
            torch.cuda.synchronize()
            a, b = ev(), ev()
            t0 = time.time()
            a.record()
            runner.step([StepEntry("p", prompt, (n_tokens - 1,))])
            b.record()
            torch.cuda.synchronize()
            if i >= warm:
                times.append(a.elapsed_time(b))
                clocks.window(t0, time.time())
            runner.finish("p")
        ms = statistics.median(times)
        fl = flops(n_tokens, n_tokens * (n_tokens + 1) / 2, 1)
        return ms, fl / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)

    prefill_ms, pf_frac = prefill_run(PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / (prefill_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3), "frac": round(pf_frac, 4)}

    # ---------------------------------------------------------------- decode, timed on the device
    def fill(b, start):
        """b requests whose caches hold ``start`` tokens, by running their prompts."""
        ids = [f"d{i}" for i in range(b)]
        for rid in ids:
            toks = rng.integers(0, V, size=start).tolist()
            for s in range(0, start, 4096):
                runner.step([StepEntry(rid, toks[s:s + 4096], ())])
        return ids

    def decode_run(b, start=None):
        ids = fill(b, ctx_start if start is None else start)
        toks = rng.integers(0, V, size=(W + K, b))
        params, seeds = [sp_greedy] * b, [0] * b
        launches0 = 0

        def one(i):
            logits = runner.step([StepEntry(rid, [int(toks[i, j])], (0,)) for j, rid in enumerate(ids)])
            eng.sampler.sample(logits, params, seeds, [i] * b)

        for i in range(W):
            one(i)
        torch.cuda.synchronize()
        launches0 = native.launches
        a, e = ev(), ev()
        t0 = time.time()
        a.record()
        for i in range(W, W + K):
            one(i)
        e.record()
        torch.cuda.synchronize()
        clocks.window(t0, time.time())
        ms = a.elapsed_time(e) / K
        n_launch = native.launches - launches0
        runner.check_status()
        for rid in ids:
            runner.finish(rid)
        return ms, n_launch

    results = {args.batch: decode_run(args.batch)}
    ms_main, launches = results[args.batch]

    # ---------------------------------------------------------------- end to end through LLMEngine
    e2e = None
    if not args.no_e2e:
        b = args.batch
        sp = SamplingParams(temperature=0.0, max_tokens=W + K + 1, ignore_eos=True)
        for _ in range(b):
            eng.add_request(rng.integers(0, V, size=ctx_start).tolist(), sp)
        while any(s.num_uncomputed > 1 or s.num_output_tokens == 0 for s in eng.scheduler.running) \
                or eng.scheduler.waiting:
            eng.step()           # prompts, in portions, until every request decodes
        done = min(s.num_output_tokens for s in eng.scheduler.running)
        for _ in range(max(0, W - done)):
            eng.step()
        left = min(sp.max_tokens - s.num_output_tokens for s in eng.scheduler.running)
        n = min(K, left - 1)
        h2d0, d2h0 = runner.h2d_bytes + eng.sampler.h2d_bytes, eng.d2h_bytes
        torch.cuda.synchronize()
        t0 = time.time()
        for _ in range(n):
            eng.step()
        torch.cuda.synchronize()
        t1 = time.time()
        clocks.window(t0, t1)
        e2e = {"value": round(b * n / (t1 - t0), 1), "unit": "tokens/s", "steps": n,
               "ms_per_step": round((t1 - t0) * 1e3 / n, 3),
               "h2d_bytes_per_step": (runner.h2d_bytes + eng.sampler.h2d_bytes - h2d0) // n,
               "d2h_bytes_per_step": (eng.d2h_bytes - d2h0) // n}
        while not eng.is_finished():
            eng.step()

    for b in batches[1:]:
        results[b] = decode_run(b)
    value = args.batch / (ms_main * 1e-3)
    ctx_mid = ctx_end - K / 2.0
    step_bytes = weight_bytes + args.batch * ctx_mid * kv_per_token
    achieved = step_bytes / (ms_main * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks["source"]}
    points = {f"decode_b{b}": round(b / (results[b][0] * 1e-3), 1) for b in batches if b != args.batch}
    # further points: other prompt lengths (tokens/s and share of the burst peak), other contexts at the
    # main batch (tokens/s and share of copy bandwidth)
    for n in sweep_prefill:
        ms, frac = prefill_run(n, warm=2, reps=3)
        points[f"prefill_{n}"] = round(n / (ms * 1e-3), 1)
        points[f"prefill_{n}_frac"] = round(frac, 4)
    for c in sweep_ctx:
        ms, _ = decode_run(args.batch, c - (W + K))
        points[f"decode_b{args.batch}_ctx{c}"] = round(args.batch / (ms * 1e-3), 1)
        bytes_c = weight_bytes + args.batch * (c - K / 2.0) * kv_per_token
        points[f"decode_b{args.batch}_ctx{c}_frac"] = round(bytes_c / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)

    clocks.stop()
    out = {
        "metric": f"decode tokens/s (Qwen3-{args.model.upper()} sizes, bf16, 1 B200)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_main, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "model": f"Qwen3-{args.model.upper()} sizes, random weights (seed {weight_seed})", "layers": n_layers, "layers_of_model": full_layers,
            "hidden": cfg_d["hidden_size"], "heads": cfg_d["num_attention_heads"],
            "kv_heads": cfg_d["num_key_value_heads"], "head_dim": cfg_d["head_dim"],
            "intermediate": cfg_d["intermediate_size"], "vocab": V, "global_batch": args.batch,
            "seq_len": ctx_end, "page_size": PAGE, "kv_cache": "bf16", "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (all weights read every step)",
            "cuda_graphs": bool(getattr(runner, "graphs_enabled", False)),
            "max_model_len": runner.max_model_len, "kv_pages": runner.cache.groups[0].pool.num_pages,
        },
        "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points,
        "clocks": clocks.summary(), "weight_gb": round(weight_bytes / 1e9, 2),
        "setup_s": round(time.time() - t_setup, 1),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
