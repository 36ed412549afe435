"""Host-side mirror of `vexact.batch_invariant_ops.batch_invariant_ops`.

Same function names, argument meaning and error behaviour as the reference
module (vexact/batch_invariant_ops/batch_invariant_ops.py), with every kernel
replaced by a call into libvexact_b200.so.  There is no fallback path: a CPU
tensor or a missing library raises.
"""
from __future__ import annotations

import contextlib
import os
from collections import namedtuple

import torch

from . import _lib

__all__ = [
    "set_batch_invariant_mode",
    "is_batch_invariant_mode_enabled",
    "disable_batch_invariant_mode",
    "enable_batch_invariant_mode",
    "matmul_persistent",
    "log_softmax",
    "mean_dim",
    "get_batch_invariant_attention_block_size",
    "AttentionBlockSize",
    "triton_bmm",
    "batch_invariant_rms_norm",
    "hf_rms_norm",
    "add_rms_norm",
    "linear",
    "linear_f32_from_bf16",
]

RMS_SINGLE_ROUND = 0
RMS_HF_DOUBLE_ROUND = 1


def _require_cuda(name: str, t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x[..., K] @ weight[N, K]^T (+ bias), the nn.Linear form the kernel consumes directly."""
    _require_cuda("x", x)
    _require_cuda("weight", weight)
    assert x.dtype == weight.dtype, "Incompatible dtypes"
    K = x.shape[-1]
    N = weight.shape[0]
    assert weight.shape[1] == K, "Incompatible dimensions"
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    if weight.stride(-1) != 1:
        weight = weight.contiguous()
    T = x2.shape[0]
    lib = _lib.load()
    if x.dtype in (torch.bfloat16, torch.float16):
        out_dtype = out_dtype or x.dtype
        if out_dtype not in (x.dtype, torch.float32):
            raise ValueError(f"unsupported output dtype {out_dtype}")
        if K % 8 or x2.stride(0) % 8 or weight.stride(0) % 8 or x2.data_ptr() % 16 or weight.data_ptr() % 16:
            # The tensor maps want 16-byte rows.  Any other layout (an odd K from some aten::mm caller under the
            # mode switch, a sliced view) goes through zero-padded copies: K grows to the next multiple of 8 and
            # the extra products are exact zeros, so the fp32 accumulation of every output is unchanged.
            K8 = (K + 7) // 8 * 8
            x2 = torch.nn.functional.pad(x2, (0, K8 - K)) if K8 != K else x2.clone(memory_format=torch.contiguous_format)
            weight = torch.nn.functional.pad(weight, (0, K8 - K)) if K8 != K else weight.clone(memory_format=torch.contiguous_format)
            K = K8
        if bias is not None:
            assert bias.dim() == 1, "bias must be 1-D"
            bias = bias.to(x.dtype).contiguous()
        out = torch.empty((T, N), device=x.device, dtype=out_dtype)
        fn, name = (lib.b200_gemm_bf16, "b200_gemm_bf16") if x.dtype == torch.bfloat16 else \
            (lib.b200_gemm_f16, "b200_gemm_f16")
        _lib.check(
            fn(x2.data_ptr(), weight.data_ptr(), _lib.ptr(bias), out.data_ptr(), T, N, K, x2.stride(0),
               weight.stride(0), out.stride(0), 0 if out_dtype == x.dtype else 1, _lib.current_stream()),
            name,
        )
    elif x.dtype == torch.float32:
        if bias is not None:
            bias = bias.float().contiguous()
        out = torch.empty((T, N), device=x.device, dtype=torch.float32)
        _lib.check(
            lib.b200_gemm_f32(x2.data_ptr(), weight.data_ptr(), _lib.ptr(bias), out.data_ptr(), T, N, K,
                              x2.stride(0), weight.stride(0), out.stride(0), _lib.current_stream()),
            "b200_gemm_f32",
        )
    else:
        raise NotImplementedError(f"matmul for dtype {x.dtype} is not implemented")
    return out.reshape(*x.shape[:-1], N)


def linear_f32_from_bf16(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """`F.linear(x.float(), weight.float())` for bf16 tensors without the fp32 copies (same bits): the
    DeepSeek-V3 router projection (modeling_deepseek_v3.py:97-100)."""
    _require_cuda("x", x)
    _require_cuda("weight", weight)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return linear(x.float(), weight.float())
    K, N = x.shape[-1], weight.shape[0]
    assert weight.shape[1] == K, "Incompatible dimensions"
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    if weight.stride(-1) != 1:
        weight = weight.contiguous()
    out = torch.empty((x2.shape[0], N), device=x.device, dtype=torch.float32)
    _lib.check(
        _lib.load().b200_gemm_f32_from_bf16(x2.data_ptr(), weight.data_ptr(), out.data_ptr(), x2.shape[0], N, K,
                                            x2.stride(0), weight.stride(0), out.stride(0), _lib.current_stream()),
        "b200_gemm_f32_from_bf16",
    )
    return out.reshape(*x.shape[:-1], N)


def matmul_persistent(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """C = A @ B (+ bias), fp32 accumulation.  Reference: batch_invariant_ops.py:159.

    `b` is [K, N]; the usual caller passes `weight.t()` (strides (1, K)), which is
    consumed without a copy.  A row-major `b` is transposed into a temporary first.
    """
    assert a.shape[1] == b.shape[0], "Incompatible dimensions"
    assert a.dtype == b.dtype, "Incompatible dtypes"
    assert bias is None or bias.dim() == 1, "bias must be 1-D"
    w = b.t()  # [N, K]
    if w.stride(-1) != 1:
        w = w.contiguous()
    return linear(a, w, bias)


def log_softmax(input: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Row log-softmax over the last dim.  Reference: batch_invariant_ops.py:295."""
    if dim != -1 and dim != input.ndim - 1:
        raise ValueError("This implementation only supports log_softmax along the last dimension")
    _require_cuda("input", input)
    original_shape = input.shape
    x2 = input.reshape(-1, input.shape[-1]).contiguous()
    if x2.dtype != torch.float32:
        # The reference kernel computes in the input dtype's fp32 upcast and stores the input dtype.
        out32 = log_softmax(x2.float(), dim=-1)
        return out32.to(input.dtype).reshape(original_shape)
    out = torch.empty_like(x2)
    rows, n = x2.shape
    _lib.check(
        _lib.load().b200_log_softmax_f32(x2.data_ptr(), out.data_ptr(), rows, n, x2.stride(0), out.stride(0),
                                         _lib.current_stream()),
        "b200_log_softmax_f32",
    )
    return out.reshape(original_shape)


def mean_dim(input: torch.Tensor, dim: int, keepdim: bool = False, dtype: torch.dtype | None = None) -> torch.Tensor:
    """Mean over one dimension.  Reference: batch_invariant_ops.py:385."""
    assert input.is_cuda, "Input must be a CUDA tensor"
    assert -input.ndim <= dim < input.ndim, f"Invalid dimension {dim} for tensor with {input.ndim} dimensions"
    if dim < 0:
        dim += input.ndim
    if dtype is None:
        dtype = torch.float32 if input.dtype in (torch.int8, torch.int16, torch.int32, torch.int64) else input.dtype
    if input.dtype != dtype:
        input = input.to(dtype)
    if dtype not in (torch.float32, torch.bfloat16):
        if not dtype.is_floating_point:
            raise NotImplementedError(f"mean_dim for dtype {dtype} is not implemented")
        # fp16 / fp64: the reference's kernel accumulates every dtype in fp32 and rounds once
        # (batch_invariant_ops.py:333-381); an exact upcast (fp16) or the fp32 view (fp64) through the fp32 kernel
        return mean_dim(input.float(), dim, keepdim=keepdim, dtype=torch.float32).to(dtype)
    moved = dim != input.ndim - 1
    x = input.movedim(dim, -1) if moved else input
    n = x.shape[-1]
    x2 = x.reshape(-1, n)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0],), device=input.device, dtype=dtype)
    _lib.check(
        _lib.load().b200_mean_lastdim(x2.data_ptr(), out.data_ptr(), x2.shape[0], n, x2.stride(0),
                                      0 if dtype == torch.float32 else 1, _lib.current_stream()),
        "b200_mean_lastdim",
    )
    out = out.reshape(x.shape[:-1])
    if keepdim:
        out = out.unsqueeze(dim)
    return out


def _rms_norm(input: torch.Tensor, weight: torch.Tensor, eps: float, mode: int) -> torch.Tensor:
    _require_cuda("input", input)
    if input.dtype != torch.bfloat16:
        raise NotImplementedError("rms_norm is implemented for bf16 activations")
    n = input.shape[-1]
    x2 = input.reshape(-1, n)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    w = weight.to(torch.bfloat16).contiguous()
    out = torch.empty((x2.shape[0], n), device=input.device, dtype=input.dtype)
    _lib.check(
        _lib.load().b200_rmsnorm(x2.data_ptr(), w.data_ptr(), out.data_ptr(), x2.shape[0], n, x2.stride(0),
                                 out.stride(0), float(eps), mode, _lib.current_stream()),
        "b200_rmsnorm",
    )
    return out.reshape(input.shape)


class BatchInvariantRMSNormFunction(torch.autograd.Function):
    """Batch-invariant RMSNorm with the backward the training side needs.
    Reference: batch_invariant_ops.py:691-725 (same saved tensors, same formulas)."""

    @staticmethod
    def forward(ctx, input, weight, eps):
        output = _rms_norm(input, weight, eps, RMS_SINGLE_ROUND)
        ctx.save_for_backward(input, weight)
        ctx.eps = eps
        return output

    @staticmethod
    def backward(ctx, grad_output):
        input, weight = ctx.saved_tensors
        n = input.shape[-1]
        if input.dtype != torch.bfloat16:
            raise NotImplementedError("the RMSNorm backward kernel is implemented for bf16")
        x2 = input.reshape(-1, n).contiguous()
        g2 = grad_output.reshape(-1, n).to(torch.bfloat16).contiguous()
        w = weight.to(torch.bfloat16).contiguous()
        rows = x2.shape[0]
        gx = torch.empty_like(x2)
        gw = torch.empty_like(w)
        scratch = torch.empty(rows + (rows + 63) // 64 * n, device=x2.device, dtype=torch.float32)
        _lib.check(
            _lib.load().b200_rmsnorm_backward(x2.data_ptr(), w.data_ptr(), g2.data_ptr(), gx.data_ptr(), gw.data_ptr(),
                                              scratch.data_ptr(), rows, n, float(ctx.eps), _lib.current_stream()),
            "b200_rmsnorm_backward",
        )
        return gx.reshape(input.shape), gw.to(weight.dtype), None


def batch_invariant_rms_norm(input: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """fp32 math, one rounding.  Reference: batch_invariant_ops.py:728 (an autograd Function there and here;
    without gradients in play this is a plain kernel call)."""
    if torch.is_grad_enabled() and (input.requires_grad or weight.requires_grad):
        return BatchInvariantRMSNormFunction.apply(input, weight, eps)
    return _rms_norm(input, weight, eps, RMS_SINGLE_ROUND)


def hf_rms_norm(input: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """HF eager RMSNorm: weight * (x * rsqrt(mean(x^2) + eps)).to(bf16).

    What the reference computes for Qwen3 / Qwen2 / Qwen3-MoE: the stock module forward with
    its `.mean(-1)` routed to mean_dim (batch_invariant_ops.py:619).
    """
    return _rms_norm(input, weight, eps, RMS_HF_DOUBLE_ROUND)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                 hf: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """(residual + x, rmsnorm(residual + x)) in one pass; the sum is rounded to bf16 first."""
    _require_cuda("x", x)
    n = x.shape[-1]
    x2 = x.reshape(-1, n).contiguous()
    r2 = residual.reshape(-1, n).contiguous()
    w = weight.to(torch.bfloat16).contiguous()
    s = torch.empty_like(x2)
    out = torch.empty_like(x2)
    _lib.check(
        _lib.load().b200_add_rmsnorm(x2.data_ptr(), r2.data_ptr(), w.data_ptr(), s.data_ptr(), out.data_ptr(),
                                     x2.shape[0], n, float(eps),
                                     RMS_HF_DOUBLE_ROUND if hf else RMS_SINGLE_ROUND, _lib.current_stream()),
        "b200_add_rmsnorm",
    )
    return s.reshape(x.shape), out.reshape(x.shape)


def triton_bmm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """[B, M, K] @ [B, K, N].  Reference: batch_invariant_ops.py:567.

    The reference uses it for the DeepSeek-V3 rotary frequencies (K = 1,
    modeling_deepseek_v3.py:428); an outer product is a single exact multiply per
    element, so that case is a broadcast multiply.  bf16 batches run the GEMM per batch.
    """
    assert a.ndim == 3 and b.ndim == 3 and a.shape[0] == b.shape[0] and a.shape[2] == b.shape[1]
    if a.shape[2] == 1:
        return a * b  # [B, M, 1] * [B, 1, N]
    return torch.stack([matmul_persistent(a[i], b[i]) for i in range(a.shape[0])])


def mm_batch_invariant(a, b):
    return matmul_persistent(a, b)


def addmm_batch_invariant(bias, a, b):
    return matmul_persistent(a, b, bias=bias)


def bmm_batch_invariant(a, b):
    return triton_bmm(a, b)


def _log_softmax_batch_invariant(input, dim, _half_to_float):
    assert not _half_to_float, "not implemented"
    return log_softmax(input, dim=dim)


def mean_batch_invariant(input, dim, keepdim=False, dtype: torch.dtype | None = None):
    assert dtype is None or dtype == torch.float32, f"unsupported dtype: {dtype}"
    if len(dim) == 1:
        return mean_dim(input, dim[0], keepdim=keepdim)
    assert input.dtype in {torch.float16, torch.bfloat16, torch.float32}, "only float types supported for now"
    if len(dim) == 0:
        dim = list(range(input.ndim))
    n_elems = 1
    for d in dim:
        n_elems *= input.shape[d]
    return torch.sum(input, dim=dim, keepdim=keepdim, dtype=torch.float32).to(dtype or input.dtype) / n_elems


_batch_invariant_MODE = False
_batch_invariant_LIB = None


def is_batch_invariant_mode_enabled():
    return _batch_invariant_MODE


def enable_batch_invariant_mode():
    """Route aten::mm / addmm / _log_softmax / mean.dim on CUDA tensors to the B200 kernels.

    Reference: batch_invariant_ops.py:741-759 (same four ops, same global switches).
    """
    global _batch_invariant_MODE, _batch_invariant_LIB
    if _batch_invariant_MODE:
        return
    _lib.load()
    _batch_invariant_MODE = True
    _batch_invariant_LIB = torch.library.Library("aten", "IMPL")
    _batch_invariant_LIB.impl("aten::mm", mm_batch_invariant, "CUDA")
    _batch_invariant_LIB.impl("aten::addmm", addmm_batch_invariant, "CUDA")
    _batch_invariant_LIB.impl("aten::_log_softmax", _log_softmax_batch_invariant, "CUDA")
    _batch_invariant_LIB.impl("aten::mean.dim", mean_batch_invariant, "CUDA")

    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":16:8")
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    torch.use_deterministic_algorithms(True, warn_only=False)
    torch.backends.cudnn.deterministic = True


def disable_batch_invariant_mode():
    global _batch_invariant_MODE, _batch_invariant_LIB
    if _batch_invariant_LIB is not None:
        _batch_invariant_LIB._destroy()
    _batch_invariant_MODE = False
    _batch_invariant_LIB = None


@contextlib.contextmanager
def set_batch_invariant_mode(enabled: bool = True):
    global _batch_invariant_MODE, _batch_invariant_LIB
    old_data = (_batch_invariant_MODE, _batch_invariant_LIB)
    if enabled:
        enable_batch_invariant_mode()
    else:
        disable_batch_invariant_mode()
    yield
    if _batch_invariant_LIB is not None:
        _batch_invariant_LIB._destroy()
    _batch_invariant_MODE, _batch_invariant_LIB = old_data


AttentionBlockSize = namedtuple("AttentionBlockSize", ["block_m", "block_n"])


def get_batch_invariant_attention_block_size(head_dim: int = 128, decode: bool = False) -> AttentionBlockSize:
    """Tiling of the default (tcgen05) paged-attention kernel: block_n = 128 keys per KV block for
    every shape; block_m = (query position, head) columns per tile: 16 in a decode step, otherwise 64
    for head_dim 128 and 32 for the 192 / 128 MLA dims.  (Head dims the tcgen05 kernel does not cover
    run the mma.sync kernel: 8 columns, 64-key blocks.)  A row's arithmetic does not depend on block_m.
    Reference: batch_invariant_ops.py:787 (same name, reports its own kernel's tiles)."""
    if head_dim not in (128, 192):
        return AttentionBlockSize(block_m=8, block_n=64)
    return AttentionBlockSize(block_m=16 if decode else (64 if head_dim == 128 else 32), block_n=128)
