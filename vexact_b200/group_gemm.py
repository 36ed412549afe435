"""The forward operators of the reference's grouped-GEMM package under their own names.

Mirror of vexact/batch_invariant_ops/group_gemm/kernel/moe.py (`expert_histogram` :52, `moe_gather`
:131, `moe_scatter` :304, `moe_index_compute` :382) and group_gemm/kernel/group_gemm.py (`group_gemm_same_nk` :156), which
`FusedMoeExpertFunction.forward` (fused_moe.py:24-111) chains one after the other and which the
reference's tests call directly.  `fused_moe_forward` in this package runs the same steps with fewer
launches; these are for callers that hold the reference's intermediate tensors (a scatter index, an
inclusive cumulative sum of rows per expert) and want one step at a time.

The two GEMM forms of the backward are here too, correct but not tuned: `transpose_b=False` (dgrad) runs
the forward kernel over a transposed copy of the weights, `group_gemm_same_mn` (the ragged-K weight gradient)
is a CUDA-core kernel.  `moe_add_gather`, fused activations and accumulation into `c` raise NotImplementedError.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .fused_moe import _permute

_TWO_BYTE = (torch.bfloat16, torch.float16)


def _index_i32(index: torch.Tensor) -> torch.Tensor:
    if index.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"index must be int32 or int64, got {index.dtype}")
    return index if index.dtype == torch.int32 else index.to(torch.int32)


def _transpose_last2(x: torch.Tensor) -> torch.Tensor:
    """[G, R, C] -> contiguous [G, C, R] (tiled kernel for 2-byte elements with R, C multiples of 8)."""
    G, R, C = x.shape
    if x.element_size() != 2 or R % 8 or C % 8 or not x.is_contiguous() or x.data_ptr() % 16:
        return x.transpose(1, 2).contiguous()
    out = torch.empty((G, C, R), dtype=x.dtype, device=x.device)
    _lib.check(_lib.load().b200_transpose_last2(x.data_ptr(), out.data_ptr(), G, R, C, _lib.current_stream()),
               "b200_transpose_last2")
    return out


def expert_histogram(input: torch.Tensor, num_bins: int) -> torch.Tensor:
    """Counts of the values 0..num_bins-1 in `input` -> int32 [num_bins] (moe.py:52-83)."""
    assert input.is_cuda
    assert input.dtype == torch.int32 or input.dtype == torch.int64
    assert input.numel() < (1 << 31) - 1, "Too many elements."
    flat = input.flatten().contiguous()
    if flat.numel() == 0:
        return torch.zeros(num_bins, dtype=torch.int32, device=input.device)
    # the index kernel's exclusive prefix sum over the bins, differenced
    cu = _permute(flat.view(-1, 1), None, None, num_bins)["cu_seqlens"]
    return cu[1:] - cu[:-1]


def moe_index_compute(experts_for_tokens: torch.Tensor, expert_histogram_cumsum: torch.Tensor) -> torch.Tensor:
    """Row of the expert-sorted activation for every (token, k): [n_tokens, topk] int64 (moe.py:382-433).

    The reference reserves each expert's rows with atomics, so its order inside an expert varies from run to
    run; here it is the stable order (token, k ascending), i.e. the `scatter_index` of fused_moe.py:43, which
    satisfies the same contract.  `expert_histogram_cumsum` ([n_experts], inclusive) only tells the number of
    experts: the counts are recomputed in the same launch."""
    assert experts_for_tokens.is_contiguous()
    assert experts_for_tokens.numel() < (1 << 31) - 1
    assert expert_histogram_cumsum.is_contiguous()
    assert experts_for_tokens.device == expert_histogram_cumsum.device
    e = experts_for_tokens if experts_for_tokens.dim() == 2 else experts_for_tokens.reshape(-1, 1)
    plan = _permute(e, None, None, expert_histogram_cumsum.numel())
    return plan["scatter_index"].view(experts_for_tokens.shape).to(torch.int64)


def moe_scatter(x: torch.Tensor, index: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """out[index[t, k]] = x[t]: [M, N] -> [M * topk, N] (moe.py:304-336).  `index` must be a permutation of
    0..M*topk-1, as the reference assumes ("Holes in output?"); an index outside that range is skipped and
    shows up in `vexact_b200._lib.read_status()` as code 2."""
    assert x.is_cuda and index.is_cuda
    assert x.shape[0] == index.shape[0]
    assert x.device == index.device, f"x.device = {x.device}, index.device = {index.device}"
    if x.dtype not in _TWO_BYTE or (out_dtype or x.dtype) != x.dtype:
        raise NotImplementedError("moe_scatter moves bf16 / fp16 rows without a dtype change")
    M, N = x.shape
    topk = index.shape[1]
    if N % 8 != 0:
        raise NotImplementedError("moe_scatter needs a row length that is a multiple of 8")
    if x.stride(1) != 1 or x.stride(0) % 8 != 0:
        x = x.contiguous()
    index = _index_i32(index)
    out = torch.empty(M * topk, N, dtype=x.dtype, device=x.device)
    _lib.check(
        _lib.load().b200_moe_scatter(x.data_ptr(), x.stride(0), index.data_ptr(), index.stride(0), index.stride(1),
                                     out.data_ptr(), M * topk, M, topk, N, _lib.current_stream()),
        "b200_moe_scatter",
    )
    return out


def moe_gather(x: torch.Tensor, index: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """out[t] = sum over k of x[index[t, k]], added in fp32 in k order and rounded once: [M * topk, N] -> [M, N]
    (moe.py:86-163)."""
    assert x.is_cuda and index.is_cuda
    M, topk = index.shape
    assert x.shape[0] == M * topk
    assert x.device == index.device, f"x.device = {x.device}, index.device = {index.device}"
    if x.dtype != torch.bfloat16 or (out_dtype or x.dtype) != torch.bfloat16:
        raise NotImplementedError("moe_gather is implemented for bf16 in, bf16 out")
    N = x.shape[1]
    if N % 8 != 0:
        raise NotImplementedError("moe_gather needs a row length that is a multiple of 8")
    x = x.contiguous()
    index = _index_i32(index)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    _lib.check(
        _lib.load().b200_moe_gather(x.data_ptr(), x.shape[0], index.data_ptr(), index.stride(0), index.stride(1),
                                    out.data_ptr(), M, topk, N, _lib.current_stream()),
        "b200_moe_gather",
    )
    return out


def moe_add_gather(x: torch.Tensor, y: torch.Tensor, index: torch.Tensor, out_dtype=None):
    raise NotImplementedError("moe_add_gather (moe.py:214) serves the fused-MoE backward, which is not part of "
                              "this library")


def group_gemm_same_nk(
    a: torch.Tensor,
    b: torch.Tensor,
    cumsum_M: torch.Tensor,
    max_M: int,
    transpose_a: bool = False,
    transpose_b: bool = False,
    activation=None,
    save_activation: bool = False,
    c: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Rows [cumsum_M[g-1], cumsum_M[g]) of `a` [M, K] times b[g]^T, b [G, N, K] -> [M, N]
    (group_gemm.py:156-236 with `transpose_b=True`, the form every forward call of fused_moe.py:51-99 uses).

    `cumsum_M` is the INCLUSIVE cumulative sum of rows per group ([G], the reference's `torch.cumsum(splits)`).
    `max_M` only sizes the reference's launch grid and is ignored.  Rows past cumsum_M[-1] are left unwritten,
    as in the reference."""
    del max_M
    assert not transpose_a, "Transpose A not tested yet."
    if not transpose_b:
        # dgrad: b is [G, K, N] with N contiguous.  The tensor-core kernel reads weights K-major, so the weights
        # are transposed into scratch first (one extra pass over them); the products and their order are those
        # of the forward form on the transposed tensor.
        assert b.dim() == 3 and a.shape[1] == b.shape[1]
        return group_gemm_same_nk(a, _transpose_last2(b), cumsum_M, 0, transpose_b=True)
    if activation is not None or save_activation:
        raise NotImplementedError("a fused activation is not offered here; fused_moe_forward fuses SwiGLU itself")
    if c is not None:
        raise NotImplementedError("accumulating into c is not supported")
    assert a.dtype in [torch.bfloat16, torch.float16], a.dtype
    assert b.dtype in [torch.bfloat16, torch.float16], b.dtype
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise NotImplementedError("the grouped GEMM is implemented for bf16")
    assert a.is_cuda and a.device == b.device, f"a.device = {a.device}, b.device = {b.device}"
    G, N, K = b.shape
    assert len(cumsum_M) == G
    assert a.is_contiguous() and b.is_contiguous(), "Not implemented: Noncontiguous input."
    assert a.shape[1] == K
    cu = torch.zeros(G + 1, dtype=torch.int32, device=a.device)
    cu[1:] = cumsum_M
    out = torch.empty((a.shape[0], N), dtype=a.dtype, device=a.device)
    _lib.check(
        _lib.load().b200_moe_grouped_gemm_noalloc(a.data_ptr(), b.data_ptr(), None, out.data_ptr(), cu.data_ptr(),
                                                  a.shape[0], G, N, K, out.stride(0), 0, _lib.current_stream()),
        "b200_moe_grouped_gemm_noalloc",
    )
    return out


def group_gemm_same_mn(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, cumsum_K: torch.Tensor, max_K: int,
                       transpose_a: bool = False, transpose_b: bool = False) -> torch.Tensor:
    """c[g] = a[rows of g]^T @ b[rows of g], written into the caller's `c` [G, M, N] (group_gemm.py:360-400 with
    `transpose_a=True, transpose_b=False`, the only form fused_moe.py:154-236 uses): a [total_K, M], b [total_K, N],
    `cumsum_K` the INCLUSIVE cumulative sum of rows per group.  fp32 accumulation over a group's rows in ascending
    order, one rounding; an empty group gets zeros."""
    del max_K
    if not transpose_a or transpose_b:
        raise NotImplementedError("group_gemm_same_mn is implemented for transpose_a=True, transpose_b=False")
    G, M, N = c.shape
    assert a.dtype in [torch.bfloat16, torch.float16], a.dtype
    assert b.dtype in [torch.bfloat16, torch.float16], b.dtype
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or c.dtype != torch.bfloat16:
        raise NotImplementedError("group_gemm_same_mn is implemented for bf16")
    assert a.is_cuda and a.device == b.device, f"a.device = {a.device}, b.device = {b.device}"
    assert a.device == c.device, f"a.device = {a.device}, c.device = {c.device}"
    assert len(cumsum_K) == G, f"{len(cumsum_K), c.shape}"
    assert a.is_contiguous() and b.is_contiguous() and c.is_contiguous(), "Not implemented: Noncontiguous input."
    assert a.shape == (b.shape[0], M) and b.shape[1] == N
    if M % 4 or N % 4 or a.data_ptr() % 8 or b.data_ptr() % 8 or c.data_ptr() % 8:
        raise NotImplementedError("group_gemm_same_mn needs M and N that are multiples of 4 and 8-byte aligned data")
    cu = torch.zeros(G + 1, dtype=torch.int32, device=a.device)
    cu[1:] = cumsum_K
    _lib.check(
        _lib.load().b200_moe_grouped_wgrad(a.data_ptr(), b.data_ptr(), c.data_ptr(), cu.data_ptr(), a.shape[0], G, M,
                                           N, _lib.current_stream()),
        "b200_moe_grouped_wgrad",
    )
    return c
