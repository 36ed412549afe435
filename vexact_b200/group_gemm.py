"""The forward operators of the reference's grouped-GEMM package under their own names.

Mirror of vexact/batch_invariant_ops/group_gemm/kernel/moe.py (`expert_histogram` :52, `moe_gather`
:131, `moe_scatter` :304) and group_gemm/kernel/group_gemm.py (`group_gemm_same_nk` :156), which
`FusedMoeExpertFunction.forward` (fused_moe.py:24-111) chains one after the other and which the
reference's tests call directly.  `fused_moe_forward` in this package runs the same steps with fewer
launches; these are for callers that hold the reference's intermediate tensors (a scatter index, an
inclusive cumulative sum of rows per expert) and want one step at a time.

Forward only: `transpose_b=False` (the dgrad form), `group_gemm_same_mn` (the ragged-K wgrad),
`moe_add_gather` and accumulation into `c` belong to the training side's backward and raise
NotImplementedError.
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
        raise NotImplementedError("transpose_b=False is the dgrad form of the fused-MoE backward, which is not "
                                  "part of this library")
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


def group_gemm_same_mn(*args, **kwargs):
    raise NotImplementedError("group_gemm_same_mn (group_gemm.py:360, the ragged-K weight gradient) serves the "
                              "fused-MoE backward, which is not part of this library")
