"""Timings of single kernels at the sizes of a model's layers, outside the engine.

    python -m atom_b200.benchmarks.kernels gemm      [--rows 1,8] [--shape qkv|o|gate_up|down|lm_head]
    python -m atom_b200.benchmarks.kernels attention [--mode decode|prefill] [--batch 1,8,64] [--context 4096]
    python -m atom_b200.benchmarks.kernels elementwise [--tokens 8,2048]

With up to 16 rows the gemm mode times the library beside the weight-streaming product, with more rows
(--rows 2048) beside the tcgen05 product with two CTAs to a tile, the two sides in turn.
Sizes default to Qwen3-8B's (hidden 4096, 32 heads, 8 kv heads, head size 128, feed-forward
12288, vocabulary 151936).  Every timing replays a CUDA graph of several launches over
different copies of the operands (together larger than L2), so neither host launch
overhead nor cache hits flatter the numbers; the bandwidth printed is the bytes of the
weights (or of the cache) divided by the time of one launch.
(The reference's benchmarks drive a server, atom/benchmarks/benchmark_serving.py; kernels
are timed here directly because this engine's kernels are its own.)
"""
from __future__ import annotations

import argparse

import numpy as np
import torch

from .. import native

DEV = "cuda:0"


def _time_graph(fns, reps: int = 6) -> float:
    """Microseconds per launch: the launches captured in one graph, replayed ``reps`` times."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (reps * len(fns))


def bench_gemm(args) -> None:
    H, I, V = args.hidden, args.intermediate, args.vocab
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    shapes = {"qkv": (qkv, H), "o": (H, args.heads * args.head_dim), "gate_up": (2 * I, H), "down": (H, I),
              "lm_head": (V, H)}
    for name, (N, K) in shapes.items():
        if args.shape and name != args.shape:
            continue
        copies = max(1, int(400e6 // (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device=DEV).bfloat16() for _ in range(copies)]
        for M in args.rows:
            x = torch.randn(M, K, device=DEV).bfloat16()
            o1 = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
            gb = N * K * 2 / 1e9
            line = f"{name:8s} rows={M:3d}"
            t = _time_graph([(lambda w=w: native.gemm_bf16(o1, x, w)) for w in ws])
            line += f"  library {t:7.1f} us ({gb / t * 1e6:6.0f} GB/s)"
            if M <= 16 and native.gemm_rows_supports(M, N, K, K):
                t = _time_graph([(lambda w=w: native.gemm_rows(x, w, o1)) for w in ws])
                line += f"  streaming {t:7.1f} us ({gb / t * 1e6:6.0f} GB/s)"
                if name == "gate_up":
                    o2 = torch.empty(M, N // 2, device=DEV, dtype=torch.bfloat16)
                    t = _time_graph([(lambda w=w: native.gemm_rows(x, w, o2, gated=True)) for w in ws])
                    line += f"  +silu*mul {t:7.1f} us ({gb / t * 1e6:6.0f} GB/s)"
            if M > 16 and native.gemm_pairs_supports(M, N, K, K, N):
                # many rows: the tcgen05 kernel against the library, turn and turn about (a B200 under its power
                # cap slows down within a second of work, so the two sides share the warm and the cold moments)
                gated = name == "gate_up"
                o2 = torch.empty(M, N // 2 if gated else N, device=DEV, dtype=torch.bfloat16)
                own = [(lambda w=w: native.gemm_pairs(x, w, o2, gated=gated)) for w in ws]
                lib_ = [(lambda w=w: native.gemm_bf16(o1, x, w)) for w in ws]
                if gated:
                    lib_ = [f for w in ws for f in ((lambda w=w: native.gemm_bf16(o1, x, w)), (lambda: native.silu_mul(o2, o1)))]
                to, tl = [], []
                for _ in range(3):
                    to.append(_time_graph(own, reps=2))
                    tl.append(_time_graph(lib_, reps=2) * (2 if gated else 1))
                fl = 2.0 * M * N * K
                line = (f"{name:8s} rows={M:5d}  library{' + silu*mul' if gated else ''} {np.median(tl):7.1f} us  "
                        f"two CTAs to a tile{' with silu*mul' if gated else ''} {np.median(to):7.1f} us "
                        f"({fl / np.median(to) / 1e6:5.0f} TFLOP/s)  fill {native.gemm_pairs_waves(M, N // 2 if gated else N, gated):.2f}")
            print(line, flush=True)
    native.check_error_flags()


def bench_attention(args) -> None:
    nh, nkv, hd, page, ctx = args.heads, args.kv_heads, args.head_dim, args.page, args.context
    for B in args.batch:
        q_lens = [1] * B if args.mode == "decode" else [ctx] * B
        T, S = sum(q_lens), B
        P = -(-ctx // page)
        copies = 4 if args.mode == "decode" else 1
        caches = [(torch.randn(S * P, nkv, page, hd, device=DEV).bfloat16(),
                   torch.randn(S * P, nkv, page, hd, device=DEV).bfloat16()) for _ in range(copies)]
        bt = torch.randperm(S * P, device=DEV).to(torch.int32).view(S, P).contiguous()
        q = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
        out = torch.empty(T, nh * hd, device=DEV, dtype=torch.bfloat16)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32, device=DEV)
        cl = torch.tensor([ctx] * B, dtype=torch.int32, device=DEV)
        sot = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(torch.int32).to(DEV)
        long_rows = native.LONG_ROWS if (args.tc and native.flash_has_tc(hd)) else 0
        plan = native.flash_plan(q_lens, nh // nkv, nkv, ctx, long_rows=long_rows)
        scratch = torch.empty(max(1, native.flash_scratch_elems(T, nh, hd, plan[2])), dtype=torch.float32, device=DEV)

        rotate = args.mode == "decode" and args.rotate and native.flash_rotating_supports(hd, page, S * P, nh, nkv, hd)
        if rotate:      # as the engine's decode steps run it: norm, rotation and cache write inside the kernel
            table = torch.randn(ctx + 1, hd, device=DEV)
            rows = torch.full((T,), ctx - 1, dtype=torch.int32, device=DEV)
            nw = torch.ones(hd, device=DEV, dtype=torch.bfloat16)
            status = torch.zeros(1, dtype=torch.int32, device=DEV)

        def run(k, v):
            if rotate:
                native.flash_attention_rotating(out, q, k, v, bt, cu, cl, sot, T, S, nh, nkv, hd, hd ** -0.5, 0, plan[2],
                                                scratch, table, hd, rows, nw, nw, 1e-6, True, status)
            else:
                native.flash_attention(out, q, q.shape[1], k, v, bt, cu, cl, sot, T, S, nh, nkv, hd, hd ** -0.5, 0,
                                       plan, scratch)

        t = _time_graph([(lambda kv=kv: run(*kv)) for kv in caches] * (1 if copies > 1 else 4))
        if args.mode == "decode":
            gb = B * ctx * nkv * hd * 2 * 2 / 1e9
            print(f"decode  batch={B:3d} context={ctx} splits={plan[2]:2d}{' rotating' if rotate else ''}: {t:8.1f} us  "
                  f"{gb / t * 1e6:7.0f} GB/s of cache", flush=True)
        else:
            fl = 4.0 * nh * hd * ctx * (ctx + 1) / 2 * B
            kind = "tcgen05" if len(plan) > 3 and plan[3] else "mma.sync"
            print(f"prefill batch={B:3d} tokens={ctx} ({kind}): {t:8.1f} us  {fl / t / 1e6:7.1f} TFLOP/s", flush=True)


def bench_elementwise(args) -> None:
    """Residual add + RMSNorm, per-head norm + rotation + cache write, SiLU * mul: bytes moved / time."""
    H, I, nh, nkv, hd, page = args.hidden, args.intermediate, args.heads, args.kv_heads, args.head_dim, args.page
    bf = torch.bfloat16
    for T in args.tokens:
        copies = 4
        P = -(-T // page)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        w, qw, kw = torch.ones(H, device=DEV, dtype=bf), torch.ones(hd, device=DEV, dtype=bf), torch.ones(hd, device=DEV, dtype=bf)
        cos_sin = torch.randn(T + 1, hd, device=DEV)
        pos = torch.arange(T, dtype=torch.int32, device=DEV)
        sot = torch.zeros(T, dtype=torch.int32, device=DEV)
        bt = torch.randperm(P, device=DEV).to(torch.int32).view(1, P).contiguous()
        sets = []
        for _ in range(copies):
            sets.append(dict(res=torch.randn(T, H, device=DEV), delta=torch.randn(T, H, device=DEV).to(bf),
                             out=torch.empty(T, H, device=DEV, dtype=bf),
                             qkv=torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).to(bf),
                             kp=torch.zeros(P, nkv, page, hd, device=DEV, dtype=bf),
                             vp=torch.zeros(P, nkv, page, hd, device=DEV, dtype=bf),
                             gu=torch.randn(T, 2 * I, device=DEV).to(bf), act=torch.empty(T, I, device=DEV, dtype=bf)))
        t = _time_graph([(lambda d=d: native.add_rmsnorm(d["out"], d["res"], d["delta"], w, 1e-6)) for d in sets])
        by = T * H * (2 + 4 + 4 + 2)
        print(f"add_rmsnorm         tokens={T:5d}: {t:7.1f} us  {by / t / 1e3:6.0f} GB/s", flush=True)
        t = _time_graph([(lambda d=d: native.qknorm_rope_kvwrite(d["qkv"], nh, nkv, hd, qw, kw, 1e-6, cos_sin, hd, pos, sot,
                                                                 bt, page, d["kp"], d["vp"], status)) for d in sets])
        by = T * hd * 2 * ((nh + 2 * nkv) + nh + 2 * nkv)
        print(f"qknorm_rope_kvwrite tokens={T:5d}: {t:7.1f} us  {by / t / 1e3:6.0f} GB/s", flush=True)
        t = _time_graph([(lambda d=d: native.silu_mul(d["act"], d["gu"])) for d in sets])
        by = T * I * 2 * 3
        print(f"silu_mul            tokens={T:5d}: {t:7.1f} us  {by / t / 1e3:6.0f} GB/s", flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    ints = lambda s: [int(x) for x in s.split(",")]
    for name in ("gemm", "attention", "elementwise"):
        p = sub.add_parser(name)
        p.add_argument("--hidden", type=int, default=4096)
        p.add_argument("--heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=128)
        p.add_argument("--intermediate", type=int, default=12288)
        p.add_argument("--vocab", type=int, default=151936)
        if name == "gemm":
            p.add_argument("--rows", type=ints, default=[1, 8])
            p.add_argument("--shape", default=None)
        elif name == "elementwise":
            p.add_argument("--tokens", type=ints, default=[8, 2048])
            p.add_argument("--page", type=int, default=16)
        else:
            p.add_argument("--mode", choices=["decode", "prefill"], default="decode")
            p.add_argument("--batch", type=ints, default=[1, 8, 64])
            p.add_argument("--context", type=int, default=4096)
            p.add_argument("--page", type=int, default=16)
            p.add_argument("--tc", type=int, default=1, help="0: keep long portions off the tcgen05 kernel")
            p.add_argument("--rotate", type=int, default=1,
                           help="decode: 1 (default) the kernel normalises, rotates and stores the new tokens itself; 0: it finds them ready")
    args = ap.parse_args(argv)
    native.lib()
    {"gemm": bench_gemm, "attention": bench_attention, "elementwise": bench_elementwise}[args.what](args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
