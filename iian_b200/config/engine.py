"""Engine, scheduler and cache configuration.

Field names and defaults are the reference's: ``EngineConfig`` (include/iian/engine.h:26-51),
``SchedulerConfig`` (include/iian/scheduler.h:16-23), ``KVCacheConfig``
(include/iian/kv_cache.h:26-34).  Fields for device splits, speculative decoding, quantized
caches and attention-path selection have no counterpart here.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 32                    # requests running at the same time
    max_num_batched_tokens: int = 1024        # token budget of one step
    max_model_len: int = 0                    # per-request limit, prompt + output
    long_prefill_token_threshold: int = 0     # 0 = off; caps one request's portion of a prompt
    enable_chunked_prefill: bool = True
    policy: str = "fcfs"                      # "fcfs" | "priority"

    def validate(self) -> None:
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be >= 1")
        if self.max_num_batched_tokens < 1:
            raise ValueError("max_num_batched_tokens must be >= 1")
        if self.policy not in ("fcfs", "priority"):
            raise ValueError(f"unknown scheduling policy '{self.policy}' (fcfs | priority)")


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"                   # "bfloat16" | "float32"
    max_model_len: int = 0                    # 0 -> min(model's max position, 8192)  (src/iian/engine.cpp:105)
    kv_cache_tokens: int = 0                  # 0 -> max_model_len * min(max_num_seqs, 4)  (src/iian/engine.cpp:134-154)
    kv_cache_gb: float = 0.0                  # optional cap on the cache's size
    block_size: int = 16
    enable_prefix_caching: bool = True
    warmup: bool = True
    seed: int = 0
    cuda_graphs: bool = True                  # replay decode-only steps from captured graphs
    device: int = 0
    sched: SchedulerConfig = field(default_factory=SchedulerConfig)

    def validate(self) -> None:
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got '{self.dtype}'")
        if self.block_size < 1:
            raise ValueError("block_size must be >= 1")
        self.sched.validate()
