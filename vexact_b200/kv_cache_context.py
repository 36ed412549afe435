"""KV-cache context, host block allocator, cache tensors and the paged store.

Mirror of vexact/batch_invariant_ops/kv_cache_context.py: `KVCacheContext` (:49),
`set_kv_cache_context` / `get_kv_cache_context` (:107 / :131), `KVCacheManager`
(:141, lowest free block ids first), `KVCacheStore` (:220) and `store_kvcache`
(:294), the last one backed by the fused K+V CUDA kernel.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Iterable, Optional

import torch

from . import _lib

_context_storage = threading.local()


@dataclass
class KVCacheContext:
    """Per-step attention metadata, read by the attention function from thread-local storage."""

    is_paged_attn: bool = False
    key_cache: Optional[dict] = None        # layer -> [blocks, page, kv_heads, k_dim]
    value_cache: Optional[dict] = None      # layer -> [blocks, page, kv_heads, v_dim]
    block_tables: Optional[torch.Tensor] = None   # [num_seqs, max_blocks_per_seq] int32
    slot_mapping: Optional[torch.Tensor] = None   # [total_tokens] int32, -1 = do not store
    context_lens: Optional[torch.Tensor] = None   # [num_seqs] int32: past + new tokens
    query_start_loc: Optional[torch.Tensor] = None  # [num_seqs + 1] int32
    max_seqlen_q: Optional[int] = None

    def __post_init__(self):
        if self.is_paged_attn:
            assert self.key_cache is not None, "key_cache required for paged attention"
            assert self.value_cache is not None, "value_cache required for paged attention"
            assert self.block_tables is not None, "block_tables required for paged attention"
            assert self.context_lens is not None, "context_lens required for paged attention"
        else:
            assert self.query_start_loc is not None, "query_start_loc required for packed attention"
            assert self.context_lens is not None, "context_lens required for packed attention"


def set_kv_cache_context(
    is_paged_attn: bool = False,
    key_cache=None,
    value_cache=None,
    block_tables: Optional[torch.Tensor] = None,
    context_lens: Optional[torch.Tensor] = None,
    slot_mapping: Optional[torch.Tensor] = None,
    query_start_loc: Optional[torch.Tensor] = None,
    max_seqlen_q: Optional[int] = None,
):
    _context_storage.kv_cache_context = KVCacheContext(
        is_paged_attn=is_paged_attn,
        key_cache=key_cache,
        value_cache=value_cache,
        block_tables=block_tables,
        context_lens=context_lens,
        slot_mapping=slot_mapping,
        query_start_loc=query_start_loc,
        max_seqlen_q=max_seqlen_q,
    )


def get_kv_cache_context() -> Optional[KVCacheContext]:
    return getattr(_context_storage, "kv_cache_context", None)


def has_kv_cache_context() -> bool:
    return hasattr(_context_storage, "kv_cache_context")


def clear_kv_cache_context() -> None:
    if hasattr(_context_storage, "kv_cache_context"):
        del _context_storage.kv_cache_context


@dataclass(frozen=True)
class KVCacheInfo:
    """What a KV cache is built from (kv_cache_context.py:36-46)."""

    layer_idxs: Iterable[int]
    num_kv_heads: int
    head_dim: int
    page_size: int
    max_blocks: int
    device: torch.device
    dtype: torch.dtype = torch.bfloat16


class KVCacheManager:
    """Host-side block allocator (integers only); hands out the lowest free block ids first.

    Same interface as the reference class (kv_cache_context.py:141-218): built from a cache
    config with `max_cache_blocks` and `page_size`; `allocate_blocks(total_tokens,
    num_current_blocks)` returns the newly allocated ids, [] if coverage is already
    sufficient, or None when the pool cannot satisfy the request.
    """

    def __init__(self, cache_config):
        self.cache_config = cache_config
        self.allocated_blocks: set[int] = set()
        self.free_blocks_set = set(range(cache_config.max_cache_blocks))

    def _num_blocks_needed(self, num_tokens: int) -> int:
        page = self.cache_config.page_size
        return (num_tokens + page - 1) // page

    def allocate_blocks(self, total_tokens: int, num_current_blocks: int = 0):
        delta = self._num_blocks_needed(total_tokens) - num_current_blocks
        if delta <= 0:
            return []
        if len(self.free_blocks_set) < delta:
            return None
        out = []
        for _ in range(delta):
            b = min(self.free_blocks_set)
            self.free_blocks_set.remove(b)
            self.allocated_blocks.add(b)
            out.append(b)
        return out

    def num_free_blocks(self) -> int:
        return len(self.free_blocks_set)

    def num_allocated_blocks(self) -> int:
        return len(self.allocated_blocks)

    def free_blocks(self, block_ids) -> None:
        for b in block_ids:
            if b in self.allocated_blocks:
                self.allocated_blocks.remove(b)
                self.free_blocks_set.add(b)


class KVCacheStore:
    """Owns the per-layer K / V cache tensors, [max_cache_blocks, page_size, kv_heads, dim].

    Same constructor as the reference class (kv_cache_context.py:223): `(hf_config, cache_config,
    device)`; key dim = `qk_head_dim` when the config has one (MLA: 192) else `head_dim`, value dim =
    `v_head_dim` when present.  The reference allocates every layer on every pipeline rank; pass
    `layer_ids` (the rank's own layers, e.g. `range(*get_pp_indices(...))`) to allocate only those.
    """

    def __init__(self, hf_config, cache_config, device, layer_ids=None):
        self.hf_config = hf_config
        self.cache_config = cache_config
        self.device = torch.device(device)
        self.page_size = cache_config.page_size
        self.max_blocks = cache_config.max_cache_blocks
        num_kv_heads = hf_config.num_key_value_heads
        head_dim = getattr(hf_config, "head_dim", None) or hf_config.hidden_size // hf_config.num_attention_heads
        k_dim = getattr(hf_config, "qk_head_dim", None) or head_dim
        v_dim = getattr(hf_config, "v_head_dim", None) or k_dim
        dtype = getattr(hf_config, "dtype", None) or vars(hf_config).get("torch_dtype") or torch.bfloat16
        if not isinstance(dtype, torch.dtype):
            dtype = getattr(torch, str(dtype).replace("torch.", ""), torch.bfloat16)
        layers = range(hf_config.num_hidden_layers) if layer_ids is None else layer_ids
        self.key_cache: dict[int, torch.Tensor] = {}
        self.value_cache: dict[int, torch.Tensor] = {}
        for li in layers:
            self.key_cache[li] = torch.zeros((self.max_blocks, self.page_size, num_kv_heads, k_dim),
                                             device=self.device, dtype=dtype)
            self.value_cache[li] = torch.zeros((self.max_blocks, self.page_size, num_kv_heads, v_dim),
                                               device=self.device, dtype=dtype)


def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping: torch.Tensor) -> None:
    """key (N, heads, k_dim), value (N, heads, v_dim) -> paged caches at slot_mapping; -1 skips."""
    assert slot_mapping.numel() == key.shape[0]
    N, heads, k_dim = key.shape
    v_dim = value.shape[-1]
    for name, t, d in (("key", key, k_dim), ("value", value, v_dim)):
        if not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor")
        assert t.stride(-1) == 1
        assert t.stride(1) == d
    assert k_cache.stride(1) == heads * k_dim, (
        f"Cache stride mismatch: expected stride(1)={heads * k_dim}, got {k_cache.stride(1)}")
    assert v_cache.stride(1) == heads * v_dim
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    if slot_mapping.dtype != torch.int32:
        slot_mapping = slot_mapping.to(torch.int32)
    num_slots = k_cache.shape[0] * k_cache.shape[1]
    _lib.check(
        _lib.load().b200_kv_store(key.data_ptr(), value.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                  slot_mapping.data_ptr(), N, heads, k_dim, v_dim, key.stride(0), value.stride(0),
                                  num_slots, _lib.current_stream()),
        "b200_kv_store",
    )
