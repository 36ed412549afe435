"""Paged causal attention behind the reference's two entry points.

* `flash_attn_varlen_func`: the FlashAttention-compatible varlen interface of
  vexact/batch_invariant_ops/triton_invariant_attention.py:905: the paged rollout path
  (`page_table` / `block_table` and `seqused_k` / `cache_seqlens` aliases, forward only) and the
  packed training-side path (no page table; forward and backward).
* `flash_attention_forward`: the HF `ALL_ATTENTION_FUNCTIONS` adapter of
  triton_invariant_attention.py:982 and flash_attention.py:26, which reads the
  thread-local KV-cache context, stores K/V and calls the paged kernel.
* `flex_attention_forward`: the adapter behind the reference's fourth key, `flex`
  (flex_attention.py:280): the same paged call, plus the packed (non-paged) form
  for one sequence.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import _lib
from .kv_cache_context import get_kv_cache_context, store_kvcache

ATTENTION_KEYS = ("fa-invariant", "fa-invariant-cute", "triton-invariant")
FLEX_KEY = "flex"
VALID_ATTN_IMPLS = ATTENTION_KEYS + (FLEX_KEY,)   # vexact/config.py:138


def _require_cuda_int32(name: str, t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != torch.int32:
        raise ValueError(f"{name} must be int32, got {t.dtype}")


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_seqlens_q: torch.Tensor,
                    seqused_k: torch.Tensor, page_table: torch.Tensor, softmax_scale: float,
                    max_seqlen_q: int, seq_order: Optional[torch.Tensor] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q (total_q, heads, dk) against caches (blocks, page, kv_heads, d); returns (total_q, heads, dv)
    (written into `out` when given; rows of q that belong to no sequence are left as they are).

    seq_order (int32 [num_seqs], optional): a permutation of the sequences, longest context first,
    that balances the persistent kernel's CTAs on ragged batches; it never changes a result."""
    for name, t in (("q", q), ("k", k_cache), ("v", v_cache)):
        if not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor")
    _require_cuda_int32("page_table", page_table)
    _require_cuda_int32("cu_seqlens_q", cu_seqlens_q)
    _require_cuda_int32("seqused_k", seqused_k)
    if k_cache.ndim != 4 or v_cache.ndim != 4:
        raise ValueError("paged flash_attn_varlen_func expects k/v with shape (num_blocks, page_size, heads, dim)")
    if q.ndim != 3:
        raise ValueError("paged flash_attn_varlen_func expects q with shape (total_q, heads, dim)")
    if q.shape[-1] != k_cache.shape[-1]:
        raise ValueError(f"q and k head_dim must match, got {q.shape[-1]} and {k_cache.shape[-1]}")
    if q.shape[1] % k_cache.shape[2] != 0:
        raise ValueError(f"query heads ({q.shape[1]}) must be divisible by KV heads ({k_cache.shape[2]})")
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise NotImplementedError("paged attention is implemented for bf16")
    if q.stride(-1) != 1:
        q = q.contiguous()
    if k_cache.stride(-1) != 1 or v_cache.stride(-1) != 1 or page_table.stride(-1) != 1:
        raise ValueError("caches and page_table must be contiguous in their last dimension")
    if not cu_seqlens_q.is_contiguous():
        cu_seqlens_q = cu_seqlens_q.contiguous()
    if not seqused_k.is_contiguous():
        seqused_k = seqused_k.contiguous()
    shape_out = (q.shape[0], q.shape[1], v_cache.shape[-1])
    if out is None:
        out = torch.empty(shape_out, device=q.device, dtype=q.dtype)
    elif tuple(out.shape) != shape_out or out.dtype != q.dtype or out.device != q.device or out.stride(-1) != 1:
        raise ValueError(f"out must be a {q.dtype} tensor of shape {shape_out} on {q.device}")
    num_seqs = seqused_k.numel()
    if seq_order is not None:
        _require_cuda_int32("seq_order", seq_order)
        if seq_order.numel() != num_seqs or not seq_order.is_contiguous():
            raise ValueError("seq_order must be a contiguous permutation of the sequences")
    _lib.check(
        _lib.load().b200_paged_attn_fwd_ordered(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), cu_seqlens_q.data_ptr(),
            seqused_k.data_ptr(), page_table.data_ptr(), num_seqs, int(max_seqlen_q), q.shape[1],
            k_cache.shape[2], q.shape[-1], v_cache.shape[-1], k_cache.shape[0], k_cache.shape[1],
            page_table.shape[1], page_table.stride(0), q.stride(0), q.stride(1), out.stride(0), out.stride(1),
            k_cache.stride(0), k_cache.stride(1), k_cache.stride(2), v_cache.stride(0), v_cache.stride(1),
            v_cache.stride(2), float(softmax_scale), seq_order.data_ptr() if seq_order is not None else None,
            q.shape[0], _lib.current_stream()),
        "b200_paged_attn_fwd_ordered",
    )
    return out


def flash_attn_varlen_func(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: Optional[torch.Tensor] = None,
    max_seqlen_q: Optional[int] = None,
    max_seqlen_k: Optional[int] = None,
    dropout_p: float = 0.0,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    window_size: Optional[tuple] = None,
    softcap: Optional[float] = None,
    alibi_slopes: Optional[torch.Tensor] = None,
    deterministic: bool = False,
    return_attn_probs: bool = False,
    block_table: Optional[torch.Tensor] = None,
    page_table: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    cache_seqlens: Optional[torch.Tensor] = None,
    **kwargs,
):
    """FlashAttention-style varlen call; returns (out, None).

    With `page_table` / `block_table`: the paged rollout path.  Without: the packed path the training side
    uses (forward: triton_invariant_attention.py:48-192): K / V are laid into a temporary paged cache
    and run through the same kernel, so a token gets the same bits from the packed call as from the rollout's
    paged prefill.  Gradients of q, k and v come from `b200_varlen_attn_backward` (:194-431 there)."""
    del alibi_slopes, deterministic, return_attn_probs, kwargs
    if dropout_p != 0.0:
        raise NotImplementedError("dropout is not supported")
    if softcap not in (None, 0.0):
        raise NotImplementedError("softcap is not supported")
    if window_size not in (None, (-1, -1)):
        raise NotImplementedError("sliding-window attention is not supported")
    if page_table is not None and block_table is not None:
        raise ValueError("pass only one of page_table or block_table")
    table = page_table if page_table is not None else block_table
    if table is None:
        if cu_seqlens_q is None:
            raise ValueError("cu_seqlens_q is required when page_table/block_table is not provided")
        if cu_seqlens_k is None:
            raise ValueError("cu_seqlens_k is required when page_table/block_table is not provided")
        if max_seqlen_k is None:
            raise ValueError("max_seqlen_k is required when page_table/block_table is not provided")
        if max_seqlen_q is None:
            raise ValueError("max_seqlen_q is required when page_table/block_table is not provided")
        if not causal:
            raise NotImplementedError("the packed path supports causal=True only")
        scale = softmax_scale if softmax_scale is not None else q.shape[-1] ** -0.5
        return _PackedVarlenForward.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, float(scale), int(max_seqlen_q),
                                          int(max_seqlen_k)), None
    lens = seqused_k if seqused_k is not None else cache_seqlens
    if lens is None:
        raise ValueError("seqused_k or cache_seqlens is required when page_table/block_table is provided")
    if not causal:
        raise NotImplementedError("paged flash_attn_varlen_func only supports causal=True")
    scale = softmax_scale if softmax_scale is not None else q.shape[-1] ** -0.5
    if max_seqlen_q is None or int(max_seqlen_q) <= 0:
        # The reference kernel ignores max_seqlen_q; this one sizes its grid with it.
        max_seqlen_q = q.shape[0]
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return _PagedForward.apply(q, k, v, cu_seqlens_q, lens, table, float(scale), int(max_seqlen_q)), None
    return paged_attention(q, k, v, cu_seqlens_q, lens, table, scale, int(max_seqlen_q)), None


PACKED_PAGE = 16   # page size of the temporary cache behind the packed path
_KERNEL_HEAD_DIMS = ((128, 128), (192, 128), (64, 64))   # (key dim, value dim) the attention kernels tile


def packed_to_paged(k: torch.Tensor, v: torch.Tensor, cu_seqlens_k: torch.Tensor, max_seqlen_k: int,
                    page: int = PACKED_PAGE):
    """Packed K / V [total_k, kv_heads, d] -> (k_cache, v_cache, page_table [S, W], kv_lens [S]): every
    sequence gets its own consecutive pages.  All index math runs on the device (no host sync); the block
    count is the host-side upper bound total_k / page + S."""
    total_k, hkv, dk = k.shape
    S = cu_seqlens_k.numel() - 1
    dev = k.device
    cu = cu_seqlens_k.to(torch.int64)
    lens = cu[1:] - cu[:-1]
    pages = (lens + page - 1) // page
    base = torch.cumsum(pages, 0) - pages                               # first page of each sequence
    W = max(1, (int(max_seqlen_k) + page - 1) // page)
    cols = torch.arange(W, device=dev)
    table = torch.where(cols[None, :] < pages[:, None], base[:, None] + cols[None, :],
                        torch.full((), -1, device=dev, dtype=torch.int64)).to(torch.int32).contiguous()
    tok = torch.arange(total_k, device=dev)
    seq = torch.searchsorted(cu[1:].contiguous(), tok, right=True).clamp_(max=S - 1)
    pos = tok - cu[seq]
    slots = ((base[seq] + pos // page) * page + pos % page).to(torch.int32)
    nblocks = total_k // page + S + 1
    k_cache = torch.empty((nblocks, page, hkv, dk), device=dev, dtype=k.dtype)
    v_cache = torch.empty((nblocks, page, hkv, v.shape[-1]), device=dev, dtype=v.dtype)
    store_kvcache(k.contiguous(), v.contiguous(), k_cache, v_cache, slots)
    return k_cache, v_cache, table, lens.to(torch.int32)


def _pad_head_dims(q, k, v):
    """Head dims the kernels do not tile (the reference's packed path takes any, e.g. 40 or 96:
    tests/batch_invariant_ops/test_triton_attention_varlen.py:289) get zero columns up to the next tiled width:
    exact zeros in every dot product, cut from the outputs again.  The softmax scale is explicit, so the wider
    head does not touch it."""
    dk, dv = q.shape[-1], v.shape[-1]
    if (dk, dv) in _KERNEL_HEAD_DIMS:
        return q, k, v
    wide = next((d for d in (64, 128) if d >= max(dk, dv)), None)
    if wide is None:
        raise NotImplementedError(f"head dims ({dk}, {dv}) above 128 other than (192, 128)")
    pad = torch.nn.functional.pad
    return pad(q, (0, wide - dk)), pad(k, (0, wide - dk)), pad(v, (0, wide - dv))


class _PackedVarlenForward(torch.autograd.Function):
    """The packed path: forward through a temporary paged cache and the paged kernels, backward through
    `b200_varlen_attn_backward` (triton_invariant_attention.py:48-431)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, scale, max_seqlen_q, max_seqlen_k):
        dk, dv = q.shape[-1], v.shape[-1]
        qp, kp, vp = _pad_head_dims(q, k, v)
        k_cache, v_cache, table, lens = packed_to_paged(kp, vp, cu_seqlens_k, max_seqlen_k)
        cu_q = cu_seqlens_q if cu_seqlens_q.dtype == torch.int32 else cu_seqlens_q.to(torch.int32)
        # zero-filled: a sequence the kernel refuses (more queries than keys: reported through the status word)
        # leaves zeros, not whatever the allocator handed out
        out = torch.zeros((qp.shape[0], qp.shape[1], vp.shape[-1]), dtype=qp.dtype, device=qp.device)
        paged_attention(qp, k_cache, v_cache, cu_q, lens, table, scale, max_seqlen_q, out=out)
        if any(ctx.needs_input_grad[:3]):
            cu_k = cu_seqlens_k if cu_seqlens_k.dtype == torch.int32 else cu_seqlens_k.to(torch.int32)
            ctx.save_for_backward(qp.contiguous(), kp.contiguous(), vp.contiguous(), out, cu_q.contiguous(),
                                  cu_k.contiguous())
            ctx.scale, ctx.max_q, ctx.max_k, ctx.dims = float(scale), int(max_seqlen_q), int(max_seqlen_k), (dk, dv)
        return out if out.shape[-1] == dv else out[..., :dv].contiguous()

    @staticmethod
    def backward(ctx, grad_out):
        q, k, v, out, cu_q, cu_k = ctx.saved_tensors
        dk_dim, dv_dim = ctx.dims
        dout = grad_out.to(torch.bfloat16)
        if dout.shape[-1] != out.shape[-1]:
            dout = torch.nn.functional.pad(dout, (0, out.shape[-1] - dout.shape[-1]))
        dout = dout.contiguous()
        dq, dkk, dvv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
        lse = torch.empty(q.shape[:2], dtype=torch.float32, device=q.device)
        delta = torch.empty_like(lse)
        _lib.check(
            _lib.load().b200_varlen_attn_backward(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), cu_q.data_ptr(),
                cu_k.data_ptr(), dq.data_ptr(), dkk.data_ptr(), dvv.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                cu_q.numel() - 1, ctx.max_q, ctx.max_k, q.shape[0], k.shape[0], q.shape[1], k.shape[1], q.shape[2],
                v.shape[2], ctx.scale, _lib.current_stream()),
            "b200_varlen_attn_backward",
        )
        return dq[..., :dk_dim], dkk[..., :dk_dim], dvv[..., :dv_dim], None, None, None, None, None


class _PagedForward(torch.autograd.Function):
    """The paged call under autograd: forward only, as in the reference (triton_invariant_attention.py:889-902)."""

    @staticmethod
    def forward(ctx, q, k_cache, v_cache, cu_seqlens_q, lens, table, scale, max_seqlen_q):
        return paged_attention(q, k_cache, v_cache, cu_seqlens_q, lens, table, scale, max_seqlen_q)

    @staticmethod
    def backward(ctx, grad_out):
        raise NotImplementedError("paged triton flash_attn_varlen_func backward is not implemented")


def flash_attention_forward(
    module: nn.Module,
    query: torch.Tensor,
    key: Optional[torch.Tensor],
    value: Optional[torch.Tensor],
    attention_mask: Optional[torch.Tensor],
    scaling: float,
    dropout: float = 0.0,
    **kwargs,
):
    """HF attention-function adapter: (1, heads, T, d) in, (T', heads, dv) out, None for weights."""
    del attention_mask
    ctx = get_kv_cache_context()
    if ctx is None or not ctx.is_paged_attn:
        raise ValueError("a paged KV-cache context is required (set_kv_cache_context(is_paged_attn=True, ...))")
    query = query.transpose(1, 2)
    _, _, num_heads, head_dim = query.shape
    layer_idx = int(kwargs["layer_idx"]) if "layer_idx" in kwargs else int(getattr(module, "layer_idx", 0))
    k_cache = ctx.key_cache[layer_idx]
    v_cache = ctx.value_cache[layer_idx]
    if key is not None and value is not None:
        key = key.transpose(1, 2)
        value = value.transpose(1, 2)
        kv_heads = key.shape[2]
        key_flat = key.reshape(-1, kv_heads, head_dim)
        value_flat = value.reshape(-1, kv_heads, value.shape[-1])
        if key_flat.stride(1) != head_dim or key_flat.stride(2) != 1:
            key_flat = key_flat.contiguous()
        if value_flat.stride(1) != value.shape[-1] or value_flat.stride(2) != 1:
            value_flat = value_flat.contiguous()
        store_kvcache(key_flat, value_flat, k_cache, v_cache, ctx.slot_mapping)
    q_flat = query.reshape(-1, num_heads, head_dim)
    return flash_attn_varlen_func(
        q_flat, k_cache, v_cache,
        cu_seqlens_q=ctx.query_start_loc,
        max_seqlen_q=ctx.max_seqlen_q,
        seqused_k=ctx.context_lens,
        page_table=ctx.block_tables,
        dropout_p=dropout,
        softmax_scale=scaling,
        causal=True,
    )


def flex_attention_forward(
    module: nn.Module,
    query: torch.Tensor,
    key: Optional[torch.Tensor],
    value: Optional[torch.Tensor],
    attention_mask: Optional[torch.Tensor],
    scaling: float,
    dropout: float = 0.0,
    **kwargs,
):
    """The reference's `flex` attention key (flex_attention.py:280-407): (B, heads, q_len, d) in,
    (B * q_len, heads, dv) out, None for weights.

    Paged context: store the new K / V, then causal attention over the page table; the reference builds a
    block mask over the physical slots for this (flex_attention.py:187-268), here it is the paged kernel,
    so `flex` gives the bits of the other three keys.

    Packed context (`is_paged_attn=False`): K / V are the whole key sequence of ONE sequence
    (flex_attention.py:348-381 with the mask of :74-122: query i sits at absolute position
    context_len - q_len + i and sees keys 0..that position, capped at context_len).  The reference's mask
    for several sequences packed into one row compares a key's packed index with a query's position
    inside its own sequence, which is only meaningful for the first of them; that form raises here."""
    del attention_mask
    ctx = get_kv_cache_context()
    if ctx is None:
        raise RuntimeError("KV cache context not set. Call set_kv_cache_context() before forward pass.")
    if ctx.is_paged_attn:
        return flash_attention_forward(module, query, key, value, None, scaling, dropout, **kwargs)
    if key is None or value is None:
        raise ValueError("packed flex attention needs the key and value tensors")
    if dropout != 0.0:
        raise NotImplementedError("dropout is not supported")
    bsz, heads, q_len, head_dim = query.shape
    if bsz != 1 or ctx.query_start_loc.numel() != 2 or ctx.context_lens.numel() != 1:
        raise NotImplementedError("packed flex attention serves one sequence per call "
                                  "(batch 1, query_start_loc of two entries)")
    kv_len = key.shape[2]
    if q_len > kv_len:
        raise ValueError(f"packed flex attention: {q_len} queries but only {kv_len} keys")
    q = query[0].transpose(0, 1)                     # (q_len, heads, d)
    k = key[0].transpose(0, 1).contiguous()          # (kv_len, kv_heads, d)
    v = value[0].transpose(0, 1).contiguous()
    dev = query.device
    zero = torch.zeros(1, device=dev, dtype=torch.int32)
    # Keys past context_len are never visible (the mask's `kv_idx < context_lens` term); the length stays on
    # the device, so nothing here waits for the GPU.
    ctx_len = ctx.context_lens.to(torch.int32).reshape(1).clamp(max=kv_len)
    cu_k = torch.cat([zero, ctx_len])
    cu_q = torch.tensor([0, q_len], device=dev, dtype=torch.int32)
    out, _ = flash_attn_varlen_func(q, k, v, cu_q, cu_k, max_seqlen_q=q_len, max_seqlen_k=kv_len,
                                    softmax_scale=scaling, causal=True)
    return out, None


def register_attention_functions() -> None:
    """Install the adapters under the reference's attention keys (inferencer.py:51-55)."""
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    for key in ATTENTION_KEYS:
        ALL_ATTENTION_FUNCTIONS[key] = flash_attention_forward
    ALL_ATTENTION_FUNCTIONS[FLEX_KEY] = flex_attention_forward
