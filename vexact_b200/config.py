"""The configuration fields the hot-path boundary reads.

The reference keeps a whole configuration tree (vexact/config.py); the forward path touches only a
few of its fields.  These dataclasses carry exactly those, under the reference's names, so that an
object of the reference's own `VeXactConfig` can be passed wherever one of these is expected:
    PPInfo           vexact/config.py:25     pp_size, pp_rank, is_first_rank, is_last_rank
    CacheConfig      vexact/config.py:70     page_size (default 256), max_cache_blocks (default 1024)
    ParallelConfig   vexact/config.py:203    pipeline_parallel_size, torch_distributed_addr / _port
    SchedulerConfig  vexact/config.py:232    max_num_seqs, max_num_batched_tokens (defaults 2048)
    ModelConfig      vexact/config.py:92     hf_config, max_model_len, attn_impl, enforce_eager, use_fp32_logits
"""
from __future__ import annotations

import socket
from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass
class PPInfo:
    pp_size: int
    pp_rank: int
    is_first_rank: bool = field(init=False)
    is_last_rank: bool = field(init=False)

    def __post_init__(self):
        self.is_first_rank = self.pp_rank == 0
        self.is_last_rank = self.pp_rank == self.pp_size - 1


@dataclass(frozen=True)
class CacheConfig:
    page_size: int = 256
    max_cache_blocks: int = 1024

    def __post_init__(self):
        if self.page_size <= 0:
            raise ValueError(f"page_size must be positive, got {self.page_size}")
        if self.max_cache_blocks <= 0:
            raise ValueError(f"max_cache_blocks must be positive, got {self.max_cache_blocks}")


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@dataclass(frozen=True)
class ParallelConfig:
    pipeline_parallel_size: int = 1
    torch_distributed_addr: str = "127.0.0.1"
    torch_distributed_port: Optional[str] = None
    world_size: int = field(init=False)

    def __post_init__(self):
        if self.pipeline_parallel_size <= 0:
            raise ValueError(f"pipeline_parallel_size must be positive, got {self.pipeline_parallel_size}")
        object.__setattr__(self, "world_size", self.pipeline_parallel_size)
        if self.torch_distributed_port is None:
            object.__setattr__(self, "torch_distributed_port", str(_free_port()))


@dataclass(frozen=True)
class SchedulerConfig:
    max_num_seqs: int = 2048
    max_num_batched_tokens: int = 2048


@dataclass
class ModelConfig:
    hf_config: Any = None
    max_model_len: int = 4096
    attn_impl: str = "fa-invariant"
    enable_batch_invariant: bool = True
    enforce_eager: bool = False
    use_fp32_logits: bool = False

    def __post_init__(self):
        valid_attn_impls = ["fa-invariant", "fa-invariant-cute", "triton-invariant", "flex"]   # config.py:138
        if self.attn_impl not in valid_attn_impls:
            raise ValueError(f"attn_impl must be one of {valid_attn_impls}, got '{self.attn_impl}'")


@dataclass
class EngineConfig:
    """The slice of `VeXactConfig` (vexact/config.py:299) that `Inferencer.__init__` reads."""

    model: ModelConfig = field(default_factory=ModelConfig)
    cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
