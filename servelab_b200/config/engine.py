"""Engine-side configuration (not part of any model's config.json).

Names and defaults follow the reference's ``CacheConfig`` and
``SchedulerConfig`` (servelab/config.py:75-95): block_size 16, num_blocks None
(sized from free device memory times gpu_memory_utilization 0.85),
max_num_seqs 64, max_num_batched_tokens 2048, chunked_prefill True, policy
"fcfs" (or "priority"), recompute preemption.  Knobs of features outside this
engine (prefix cache, cache quantisation, swap/offload) and knobs the reference
defines but never reads (servelab/config.py:95,98-107) are absent.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class CacheConfig:
    block_size: int = 16                   # tokens per page
    num_blocks: Optional[int] = None       # pages per cache group; None => from memory
    gpu_memory_utilization: float = 0.85   # fraction of free device memory for the cache
    reserve_blocks: int = 0                # pages held back from admission only
    poison_cache: bool = False             # debugging: unwritten slots hold a huge value, so a
                                           # kernel that reads one changes the logits visibly

    def __post_init__(self):
        if self.block_size < 1:
            raise ValueError("block_size must be >= 1")
        if self.num_blocks is not None and self.num_blocks < 1:
            raise ValueError("num_blocks must be >= 1 (or None)")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048
    chunked_prefill: bool = True
    policy: str = "fcfs"                   # fcfs | priority

    def __post_init__(self):
        if self.max_num_seqs < 1 or self.max_num_batched_tokens < 1:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be >= 1")
        if self.policy not in ("fcfs", "priority"):
            raise ValueError(f"unknown scheduler policy: {self.policy}")


@dataclass
class EngineConfig:
    cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    dtype: str = "bfloat16"                # bfloat16 | float32
    seed: int = 1234                       # sampler seed (servelab/engine/engine.py:48)
    cuda_graphs: bool = True               # replay decode-only steps as CUDA graphs

    def __post_init__(self):
        if self.dtype in ("bf16",):
            self.dtype = "bfloat16"
        if self.dtype in ("fp32",):
            self.dtype = "float32"
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be bfloat16 or float32, got {self.dtype}")
