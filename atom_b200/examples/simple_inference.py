"""Offline generation from the command line, after atom/examples/simple_inference.py:15-95:

    python -m atom_b200.examples.simple_inference --model DIR [engine options]
           [--temperature 0.6] [--max-tokens 300] [--prompt TEXT ... | --prompt-token-ids "1,2,3" ...]

Prints ``Prompt:`` / ``Completion:`` for every request.  Without a tokenizer in the model
folder (random-weight folders) prompts are given as token ids and completions printed as ids.
"""
from __future__ import annotations

import argparse

from atom_b200 import SamplingParams
from atom_b200.engine.arg_utils import EngineArgs


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(formatter_class=argparse.RawTextHelpFormatter, description="simple inference")
    EngineArgs.add_cli_args(parser)
    parser.add_argument("--temperature", type=float, default=0.6, help="temperature for sampling")
    parser.add_argument("--max-tokens", type=int, default=300, help="max sampled tokens per prompt")
    parser.add_argument("--top-k", type=int, default=-1)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--prompt", action="append", default=None, help="a text prompt (repeatable)")
    parser.add_argument("--prompt-token-ids", action="append", default=None,
                        help='a prompt as comma-separated token ids (repeatable)')
    args = parser.parse_args(argv)

    llm = EngineArgs.from_cli_args(args).create_engine()
    prompts = []
    for p in args.prompt_token_ids or []:
        prompts.append([int(t) for t in p.replace(" ", "").split(",") if t])
    for p in args.prompt or []:
        prompts.append(p)
    if not prompts:
        if llm.tokenizer is not None:
            prompts = ["introduce yourself", "list all prime numbers within 100", "1+2+3=?"]
        else:
            V = llm.runner.spec.vocab_size
            prompts = [[1 % V, 2 % V, 3 % V], [(7 * i + 5) % V for i in range(19)]]
    sp = SamplingParams(temperature=args.temperature, max_tokens=args.max_tokens, top_k=args.top_k,
                        top_p=args.top_p, ignore_eos=args.ignore_eos)
    llm.start_profile()          # does nothing without --torch-profiler-dir
    outputs = llm.generate(prompts, sp)
    trace = llm.stop_profile()
    if trace:
        print(f"profiler trace: {trace}")
    for prompt, out in zip(prompts, outputs):
        print("\n")
        print(f"Prompt: {prompt!r}")
        print(f"Completion: {(out['text'] if out['text'] is not None else out['token_ids'])!r}")
        print(f"  finish_reason={out['finish_reason']} input={out['num_tokens_input']} "
              f"output={out['num_tokens_output']} ttft={out['ttft']*1e3:.1f} ms tpot={out['tpot']*1e3:.2f} ms")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
