"""Static graph-input buffers and the per-step data carriers.

Mirror of vexact/core/runtime_data.py: `TensorBuffer` (:23, a pinned host tensor paired with its
device twin), `InputBuffers` (:68, the address-stable tensors a captured CUDA graph reads),
`GenerationContext` (:120) and `InferencerOutput` (:134).  Shapes, dtypes and fill values are the
reference's; the graph-replay contract (padding rows carry slot -1, padded requests are zero-length)
depends on them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, NamedTuple, Optional, Union

import torch
from torch import Tensor


class TensorBuffer(NamedTuple):
    """A pinned CPU tensor and the GPU tensor it is copied into."""

    cpu: Tensor
    gpu: Tensor

    @classmethod
    def create(cls, *size: int, dtype: torch.dtype, device, fill_value: Optional[Union[int, float]] = None):
        dev = torch.device(device)
        cpu = torch.empty(size, dtype=dtype, pin_memory=dev.type == "cuda", device="cpu")
        gpu = (torch.full(size, fill_value, dtype=dtype, device=dev) if fill_value is not None
               else torch.empty(size, dtype=dtype, device=dev))
        return cls(cpu=cpu, gpu=gpu)

    def to_device(self, size: Optional[Union[slice, tuple]] = None, non_blocking: bool = True) -> Tensor:
        if size is None:
            self.gpu.copy_(self.cpu, non_blocking=non_blocking)
            return self.gpu
        view = self.gpu[size]
        view.copy_(self.cpu[size], non_blocking=non_blocking)
        return view


class InputBuffers:
    """Pre-allocated inputs of the captured forward: token-level and sequence-level metadata."""

    def __init__(self, device, max_num_seqs: int, max_num_batched_tokens: int, max_blocks_per_req: int,
                 hidden_size: int):
        self.device = torch.device(device)
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_blocks_per_req = max_blocks_per_req
        mk = TensorBuffer.create
        self.slot_mapping = mk(max_num_batched_tokens, dtype=torch.int32, device=device)
        self.context_lens = mk(max_num_seqs, dtype=torch.int32, device=device)
        self.query_start_loc = mk(max_num_seqs + 1, dtype=torch.int32, device=device)
        self.block_tables = mk(max_num_seqs, max_blocks_per_req, dtype=torch.int32, device=device, fill_value=-1)
        # the batch is always packed, so the batch dimension is 1
        self.input_ids = mk(1, max_num_batched_tokens, dtype=torch.long, device=device, fill_value=0)
        self.intermediate_tensors = mk(1, max_num_batched_tokens, hidden_size, dtype=torch.bfloat16, device=device,
                                       fill_value=0)
        self.position_ids = mk(1, max_num_batched_tokens, dtype=torch.long, device=device, fill_value=0)

    def get_kv_context_tensors(self, num_seqs: int, num_tokens: int):
        """(block_tables, context_lens, slot_mapping, query_start_loc) views for a packed batch."""
        return (self.block_tables.gpu[:num_seqs, :], self.context_lens.gpu[:num_seqs],
                self.slot_mapping.gpu[:num_tokens], self.query_start_loc.gpu[: num_seqs + 1])


@dataclass
class GenerationContext:
    """What one pipeline stage hands the next (and what the first stage builds from the requests)."""

    batch_input_ids: Optional[Tensor]        # [1, T] int64 (first stage)
    intermediate_tensors: Optional[Tensor]   # [1, T, H] bf16 (later stages)
    query_start_loc: Tensor                  # [S + 1] int32
    batch_position_ids: Tensor               # [1, T] int64
    block_tables: Tensor                     # [S, W] int32
    context_lens: Tensor                     # [S] int32
    slot_mapping: Tensor                     # [T] int32
    max_seqlen_q: Optional[int]
    generation_configs: list = field(default_factory=list)   # one sampling config per request
    tokens_generated: Any = None             # list[int] in the reference; a tensor after a hop here


@dataclass
class InferencerOutput:
    token_ids: Tensor   # [S] int64
    logits: Tensor      # [S, V] or empty
    logprobs: Tensor    # [S] fp32 or empty
