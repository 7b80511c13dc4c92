"""Engine options, with the reference's names, defaults and checks (config.py:5-29)."""
from __future__ import annotations

import os
from dataclasses import dataclass

from .model_config import ConfigError, ModelConfig
from .registry import load_model_config

_DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass
class EngineConfig:
    model: str
    kvcache_block_size: int = 16
    model_config: ModelConfig | None = None
    num_kvcache_blocks: int = -1          # -1: sized from free device memory
    max_num_seqs: int = 512
    max_num_batched_tokens: int = 16384
    eos: int = -1
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.9
    enable_chunked_prefill: bool = True
    long_prefill_token_threshold: int = 0
    scheduling_policy: str = "fcfs"
    # Not in the reference (its model is fixed to bfloat16, engine/model_runner.py:31):
    dtype: str = "bfloat16"
    enable_prefix_caching: bool = True
    seed: int = 0
    use_cuda_graphs: bool = True
    random_weights: bool = False        # the folder holds config.json only: weights are drawn on the device from ``seed``
    overlap_steps: bool = True          # launch the likely next decode step before reading the current one's tokens

    def __post_init__(self):
        self.model = os.path.expanduser(self.model)
        if not os.path.isdir(self.model):
            raise ConfigError(f"model folder {self.model!r} does not exist")
        if self.dtype not in _DTYPES:
            raise ConfigError(f"dtype must be one of {sorted(_DTYPES)}, got {self.dtype!r}")
        self.dtype = _DTYPES[self.dtype]
        if self.max_num_batched_tokens < self.max_num_seqs:
            raise ConfigError("max_num_batched_tokens must be at least max_num_seqs")
        if self.scheduling_policy not in ("fcfs", "priority"):
            raise ConfigError("scheduling_policy must be 'fcfs' or 'priority'")
        if self.long_prefill_token_threshold < 0:
            raise ConfigError("long_prefill_token_threshold must not be negative")
        if self.kvcache_block_size < 1:
            raise ConfigError("kvcache_block_size must be positive")
        if self.model_config is None:
            self.model_config = load_model_config(self.model)
        self.max_model_len = min(self.max_model_len, self.model_config.max_position_embeddings)
        if not self.enable_chunked_prefill and self.max_num_batched_tokens < self.max_model_len:
            raise ConfigError("without chunked prefill max_num_batched_tokens must cover max_model_len")
        if not 0 < self.gpu_memory_utilization <= 1:
            raise ConfigError("gpu_memory_utilization must be in (0, 1]")
        if self.eos == -1:
            self.eos = self.model_config.eos_token_id
