"""Command-line options of the engine, with the reference's spellings and meanings where it
has them (atom/model_engine/arg_utils.py:90-542): --model :93, --enforce-eager :145,
--kv_cache_dtype :163, --block-size :180, --max-model-len :183, --cudagraph-capture-sizes :189,
--load_dummy :209, --max-num-batched-tokens :331, --long-prefill-token-threshold :337,
--enable_chunked_prefill :373, --max-num-seqs :380, --gpu-memory-utilization :386,
--torch-profiler-dir :233, --enable_prefix_caching :150 (off by default here).
Added: --dtype, --seed, --num-kvcache-blocks.  Options for several GPUs, servers,
quantization and speculative decoding are not taken."""
from __future__ import annotations

import argparse
import json
from dataclasses import dataclass
from typing import List, Optional


@dataclass
class EngineArgs:
    model: str = ""
    dtype: str = "bfloat16"
    enforce_eager: bool = False
    kv_cache_dtype: str = "bf16"
    block_size: int = 16
    max_model_len: Optional[int] = None
    cudagraph_mixed_steps: bool = True
    cudagraph_capture_sizes: str = "[1,2,4,8,16,24,32,48,64,96,128,192,256,384,512]"
    load_dummy: Optional[str] = None
    max_num_batched_tokens: int = 16384
    long_prefill_token_threshold: int = 0
    enable_chunked_prefill: bool = True
    enable_prefix_caching: bool = False
    max_num_seqs: int = 512
    gpu_memory_utilization: float = 0.9
    num_kvcache_blocks: int = -1
    seed: int = 0
    torch_profiler_dir: Optional[str] = None

    @staticmethod
    def add_cli_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
        parser.add_argument("--model", type=str, required=True, help="Model folder (config.json, model.safetensors).")
        parser.add_argument("--dtype", choices=["bfloat16", "float32", "bf16", "fp32"], default="bfloat16",
                            help="Compute type; float32 is true 32-bit everywhere.")
        parser.add_argument("--enforce-eager", action="store_true", help="Enforce eager mode execution.")
        parser.add_argument("--kv_cache_dtype", choices=["bf16"], type=str, default="bf16",
                            help="KV cache type (follows --dtype in the float32 mode).")
        parser.add_argument("--block-size", type=int, default=16, help="KV cache block size.")
        parser.add_argument("--max-model-len", type=int, default=None,
                            help="Maximum model context length, the default is max_position_embeddings.")
        parser.add_argument("--cudagraph-capture-sizes", type=str, default="[1,2,4,8,16,24,32,48,64,96,128,192,256,384,512]",
                            help="Sizes to capture cudagraph. Example: [1,2,4,8,16]")
        parser.add_argument("--cudagraph-mixed-steps", action=argparse.BooleanOptionalAction, default=True,
                            help="Replay graphs for small steps that hold prompt portions too (not only for decode steps).")
        parser.add_argument("--load_dummy", nargs="?", const="random", default=None, choices=["random"],
                            help="Use seeded random weights instead of reading the checkpoint.")
        parser.add_argument("--max-num-batched-tokens", type=int, default=16384,
                            help="Maximum number of tokens in one step.")
        parser.add_argument("--long-prefill-token-threshold", type=int, default=0,
                            help="Cap on the tokens of one prompt scheduled in one step (0: none).")
        parser.add_argument("--enable_chunked_prefill", action=argparse.BooleanOptionalAction, default=True,
                            help="Cut prompts into portions under the token budget.")
        parser.add_argument("--enable_prefix_caching", action=argparse.BooleanOptionalAction, default=False,
                            help="Requests that begin like earlier ones reuse their cache pages.")
        parser.add_argument("--max-num-seqs", type=int, default=512, help="Maximum number of running requests.")
        parser.add_argument("--gpu-memory-utilization", type=float, default=0.9,
                            help="Share of device memory the engine may use.")
        parser.add_argument("--num-kvcache-blocks", type=int, default=-1,
                            help="Pages of the KV cache (-1: size from free memory).")
        parser.add_argument("--seed", type=int, default=0, help="Seed of random weights and of sampling.")
        parser.add_argument("--torch-profiler-dir", type=str, default=None,
                            help="Directory to save torch profiler traces")
        return parser

    @classmethod
    def from_cli_args(cls, args: argparse.Namespace) -> "EngineArgs":
        names = cls.__dataclass_fields__.keys()
        return cls(**{n: getattr(args, n) for n in names if hasattr(args, n)})

    def _engine_kwargs(self) -> dict:
        sizes: List[int] = json.loads(self.cudagraph_capture_sizes) if isinstance(
            self.cudagraph_capture_sizes, str) else list(self.cudagraph_capture_sizes)
        return dict(
            dtype=self.dtype, enforce_eager=self.enforce_eager, kv_cache_block_size=self.block_size,
            max_model_len=self.max_model_len, cudagraph_capture_sizes=sizes, cudagraph_mixed_steps=self.cudagraph_mixed_steps, load_dummy=self.load_dummy,
            max_num_batched_tokens=self.max_num_batched_tokens,
            long_prefill_token_threshold=self.long_prefill_token_threshold,
            enable_chunked_prefill=self.enable_chunked_prefill, enable_prefix_caching=self.enable_prefix_caching,
            max_num_seqs=self.max_num_seqs,
            gpu_memory_utilization=self.gpu_memory_utilization, num_kvcache_blocks=self.num_kvcache_blocks,
            seed=self.seed, torch_profiler_dir=self.torch_profiler_dir,
        )

    def create_engine(self):
        from .llm_engine import LLMEngine

        return LLMEngine(self.model, **self._engine_kwargs())
