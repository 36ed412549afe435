"""CUDA-graph capture and replay of the stage forward, one graph per power-of-two token bucket.

Mirror of vexact/inferencer/cudagraph_utils.py: `BatchExecutionDescriptor` (:30), `CudaGraphManager`
(:45) with `build_capture_sizes` (:85), `capture_graphs` (:96), `dispatch` (:102), `capture` (:109) and
`replay` (:179).  A graph is captured over the static `InputBuffers`; at capture time no token may
write the KV cache (slot_mapping = -1 everywhere) and the bucket's tokens are dealt evenly to the
bucket's sequences; a replay serves any batch with no more tokens and no more sequences than the
bucket, with the padding described in `Inferencer._prepare_input_buffers_from_gen_ctx`.

`model` is any callable with the reference's forward keywords (`input_ids`, `intermediate_tensors`,
`position_ids`, plus `forward_kwargs`): an HF module running on this library's operators, or the
native stage (`StageModel`).  Every kernel of this library launches on the current stream and
allocates nothing, which is what makes the capture legal.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch

from .kv_cache_context import KVCacheStore, set_kv_cache_context
from .runtime_data import InputBuffers


@dataclass(frozen=True)
class BatchExecutionDescriptor:
    """Shape a graph was captured for: the padded token bucket and the padded sequence count.

    `decode` marks the extra graph this library captures per bucket for pure decode steps (one token
    per sequence, num_seqs == num_tokens): the attention launch inside it is sized for one query per
    sequence instead of for `num_tokens` queries, which is what a decode batch needs to run at HBM
    speed.  The reference has one graph per bucket and sizes every attention grid for the bucket."""

    num_tokens: int
    num_seqs: int
    decode: bool = False


class CudaGraphManager:
    def __init__(self, model: Callable, device, input_buffers: InputBuffers, cache_config, cache_store: KVCacheStore,
                 max_size: int, pool: Any = None, forward_kwargs: Optional[dict] = None):
        self.model = model
        self.device = torch.device(device)
        self.cache_config = cache_config
        self.cache_store = cache_store
        self.capture_sizes = self.build_capture_sizes(max_size)
        self.pool = pool if pool is not None else torch.cuda.graph_pool_handle()
        self.graphs: dict[BatchExecutionDescriptor, torch.cuda.CUDAGraph] = {}
        self.outputs: dict[BatchExecutionDescriptor, Any] = {}
        self.forward_kwargs = forward_kwargs or {}
        self.input_buffers = input_buffers
        self._descriptors = [BatchExecutionDescriptor(num_tokens=n, num_seqs=min(n, input_buffers.max_num_seqs))
                             for n in self.capture_sizes]
        self._decode_descriptors = [BatchExecutionDescriptor(num_tokens=n, num_seqs=n, decode=True)
                                    for n in self.capture_sizes if n <= input_buffers.max_num_seqs]

    @staticmethod
    def build_capture_sizes(max_size: Optional[int]) -> list[int]:
        """1, 2, 4, ... up to the first power of two that is >= max_size."""
        if max_size is None or max_size <= 0:
            raise ValueError(f"max_size must be positive or None, got {max_size}")
        sizes, n = [], 1
        while n < max_size:
            sizes.append(n)
            n *= 2
        sizes.append(n)
        return sizes

    def capture_graphs(self) -> None:
        if not self.capture_sizes:
            raise RuntimeError("CudaGraphManger capture sizes are not set.")
        for desc in self._descriptors + self._decode_descriptors:
            self.capture(desc)

    def dispatch(self, num_seqs: int, total_tokens: int,
                 max_seqlen_q: Optional[int] = None) -> Optional[BatchExecutionDescriptor]:
        """The smallest captured shape that covers the batch, or None.  A step whose every sequence feeds
        one token (`max_seqlen_q == 1`) gets the bucket's decode graph when there is one."""
        if max_seqlen_q == 1 and total_tokens == num_seqs:
            for desc in self._decode_descriptors:
                if desc.num_seqs >= num_seqs and (desc in self.graphs or not self.graphs):
                    return desc
        for desc in self._descriptors:
            if desc.num_seqs >= num_seqs and desc.num_tokens >= total_tokens:
                return desc
        return None

    @torch.inference_mode()
    def capture(self, desc: BatchExecutionDescriptor) -> BatchExecutionDescriptor:
        num_seqs, tokens = desc.num_seqs, desc.num_tokens
        buf = self.input_buffers
        if num_seqs <= 0 or tokens <= 0:
            raise ValueError(f"num_seqs and capture_tokens must be positive, got {num_seqs=}, capture_tokens={tokens}")
        if num_seqs > tokens:
            raise ValueError(f"num_seqs cannot exceed capture_tokens, got {num_seqs=}, capture_tokens={tokens}")
        if num_seqs > buf.max_num_seqs:
            raise ValueError(f"num_seqs exceeds input buffer capacity: {num_seqs} > {buf.max_num_seqs}")
        if tokens > buf.max_num_batched_tokens:
            raise ValueError(f"capture_tokens exceeds input buffer capacity: {tokens} > {buf.max_num_batched_tokens}")
        if desc in self.graphs:
            return desc
        static_inputs = {
            "input_ids": buf.input_ids.gpu[:, :tokens],
            "intermediate_tensors": buf.intermediate_tensors.gpu[:, :tokens, :],
            "position_ids": buf.position_ids.gpu[:, :tokens],
        }
        block_tables, context_lens, slot_mapping, query_start_loc = buf.get_kv_context_tensors(num_seqs, tokens)
        for t in static_inputs.values():
            t.zero_()
        block_tables.zero_()
        slot_mapping.fill_(-1)                     # nothing may be written to the KV cache while capturing
        if desc.decode and num_seqs != tokens:
            raise ValueError("a decode graph has one token per sequence")
        per_seq = torch.full((num_seqs,), tokens // num_seqs, device=self.device, dtype=torch.int32)
        per_seq[: tokens % num_seqs] += 1
        query_start_loc[0].zero_()
        query_start_loc[1:].copy_(per_seq.cumsum(0))
        context_lens.copy_(per_seq)
        set_kv_cache_context(is_paged_attn=True, key_cache=self.cache_store.key_cache,
                             value_cache=self.cache_store.value_cache, block_tables=block_tables,
                             context_lens=context_lens, slot_mapping=slot_mapping, query_start_loc=query_start_loc,
                             max_seqlen_q=1 if desc.decode else tokens)
        # warm-up outside the capture (lazy one-time set-up: attributes, tensor-map encoder lookup)
        self.model(**static_inputs, **self.forward_kwargs)
        graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(graph, self.pool):
            outputs = self.model(**static_inputs, **self.forward_kwargs)
        self.graphs[desc] = graph
        self.outputs[desc] = outputs
        return desc

    @torch.inference_mode()
    def replay(self, graph_key: BatchExecutionDescriptor) -> Any:
        """Replay a captured graph; the caller has refreshed the static buffers."""
        if graph_key not in self.graphs:
            raise KeyError(f"No captured graph for id {graph_key}. Captured: {list(self.graphs)}")
        self.graphs[graph_key].replay()
        return self.outputs[graph_key]
