"""Engine options.  Names and defaults follow the reference's ``Config`` dataclass where it
has the option (atom/config.py:1428-1466): max_num_batched_tokens 16384 (:1428),
max_num_seqs 512 (:1437), max_model_len None (:1438), gpu_memory_utilization 0.9 (:1439),
enforce_eager False (:1445), kv_cache_block_size 16 (:1452), num_kvcache_blocks -1 (:1453),
long_prefill_token_threshold 0 (:1429), load_dummy (:1466)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class EngineConfig:
    model: str = ""                       # folder with config.json and model.safetensors
    dtype: str = "bfloat16"               # "bfloat16" or "float32" (true 32-bit everywhere)
    max_num_batched_tokens: int = 16384   # token budget of one step
    max_num_seqs: int = 512               # most requests running at a time
    max_model_len: Optional[int] = None   # longest request; default max_position_embeddings
    gpu_memory_utilization: float = 0.9   # share of device memory the engine may use
    kv_cache_block_size: int = 16         # tokens per page
    num_kvcache_blocks: int = -1          # pages per cache group; -1: size from free memory
    enforce_eager: bool = False           # never replay decode steps from CUDA graphs
    # decode batch sizes whose steps replay a graph (captured at first use; a batch is padded to the next size)
    cudagraph_capture_sizes: List[int] = field(
        default_factory=lambda: [1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512])
    cudagraph_mixed_steps: bool = True    # small steps with prompt portions replay graphs too (up to 128 tokens in all, more for small models)
    long_prefill_token_threshold: int = 0  # cap on one request's portion per step (0: none)
    enable_chunked_prefill: bool = True
    enable_prefix_caching: bool = False   # requests that begin like earlier ones take their pages (the reference's default is on)
    load_dummy: Optional[str] = None      # "random": seeded random weights instead of the file
    seed: int = 0
    torch_profiler_dir: Optional[str] = None   # where start_profile / stop_profile write their traces

    def __post_init__(self) -> None:
        aliases = {"bf16": "bfloat16", "fp32": "float32"}
        self.dtype = aliases.get(self.dtype, self.dtype)
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        if self.kv_cache_block_size <= 0:
            raise ValueError("kv_cache_block_size must be positive")
        if self.max_num_batched_tokens <= 0 or self.max_num_seqs <= 0:
            raise ValueError("max_num_batched_tokens and max_num_seqs must be positive")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
