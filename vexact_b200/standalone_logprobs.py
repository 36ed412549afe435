"""Per-token log-probabilities from logits.

Mirror of vexact/batch_invariant_ops/standalone_logprobs.py:28
(`logprobs_from_logits_flash_attn`): logprob = logits[label] - logsumexp(logits),
computed in fp32 by one streaming pass per row.
"""
from __future__ import annotations

import torch

from . import _lib

IGNORE_INDEX = -100


class _GatherLogprob(torch.autograd.Function):
    """Per-token log-probability with the gradient flash-attn's cross-entropy gives (sign flipped)."""

    @staticmethod
    def forward(ctx, logits, labels, inplace_backward):
        with torch.no_grad():
            out = logprobs_from_logits_flash_attn(logits, labels)
        ctx.save_for_backward(logits, labels)
        ctx.inplace = bool(inplace_backward)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        logits, labels = ctx.saved_tensors
        vocab = logits.shape[-1]
        x = logits.reshape(-1, vocab)
        if x.stride(-1) != 1:
            x = x.contiguous()
        inplace = ctx.inplace and x.data_ptr() == logits.data_ptr()
        dx = x if inplace else torch.empty_like(x)
        lab = labels.reshape(-1).to(torch.int64).contiguous()
        g = grad_out.reshape(-1).to(torch.float32).contiguous()
        _lib.check(
            _lib.load().b200_gather_logprob_backward(x.data_ptr(), lab.data_ptr(), g.data_ptr(), dx.data_ptr(),
                                                     x.shape[0], vocab, x.stride(0), dx.stride(0),
                                                     0 if x.dtype == torch.float32 else 1, IGNORE_INDEX,
                                                     _lib.current_stream()),
            "b200_gather_logprob_backward",
        )
        return dx.reshape(logits.shape), None, None


def logprobs_from_logits_flash_attn(logits: torch.Tensor, labels: torch.Tensor,
                                    inplace_backward: bool = False) -> torch.Tensor:
    if not logits.is_cuda:
        raise ValueError("logits must be a CUDA tensor")
    if torch.is_grad_enabled() and logits.requires_grad:
        if logits.dtype not in (torch.float32, torch.bfloat16):
            raise NotImplementedError(f"logits dtype {logits.dtype} is not supported")
        return _GatherLogprob.apply(logits, labels, inplace_backward)
    if logits.dtype not in (torch.float32, torch.bfloat16):
        raise NotImplementedError(f"logits dtype {logits.dtype} is not supported")
    batch_shape = logits.shape[:-1]
    vocab = logits.shape[-1]
    x = logits.reshape(-1, vocab)
    if x.stride(-1) != 1:
        x = x.contiguous()
    lab = labels.reshape(-1).to(torch.int64).contiguous()
    assert lab.numel() == x.shape[0], "labels must have one entry per logits row"
    out = torch.empty((x.shape[0],), device=logits.device, dtype=torch.float32)
    _lib.check(
        _lib.load().b200_gather_logprob(x.data_ptr(), lab.data_ptr(), out.data_ptr(), x.shape[0], vocab,
                                        x.stride(0), 0 if x.dtype == torch.float32 else 1, IGNORE_INDEX,
                                        _lib.current_stream()),
        "b200_gather_logprob",
    )
    return out.reshape(batch_shape)


def greedy_token_and_logprob(logits: torch.Tensor):
    """(argmax token ids int64, their log-probabilities fp32) per row, one kernel, one pass.

    Same values as `torch.argmax(logits, -1)` followed by `logprobs_from_logits_flash_attn`.
    """
    if not logits.is_cuda:
        raise ValueError("logits must be a CUDA tensor")
    if logits.dtype not in (torch.float32, torch.bfloat16):
        raise NotImplementedError(f"logits dtype {logits.dtype} is not supported")
    vocab = logits.shape[-1]
    x = logits.reshape(-1, vocab)
    if x.stride(-1) != 1:
        x = x.contiguous()
    tokens = torch.empty((x.shape[0],), device=logits.device, dtype=torch.int64)
    lp = torch.empty((x.shape[0],), device=logits.device, dtype=torch.float32)
    _lib.check(
        _lib.load().b200_greedy_logprob(x.data_ptr(), tokens.data_ptr(), lp.data_ptr(), x.shape[0], vocab, x.stride(0),
                                        0 if x.dtype == torch.float32 else 1, _lib.current_stream()),
        "b200_greedy_logprob",
    )
    return tokens.reshape(logits.shape[:-1]), lp.reshape(logits.shape[:-1])


def lm_head_greedy(hidden: torch.Tensor, lm_head_weight: torch.Tensor):
    """(argmax token ids int64 [T], their log-probabilities fp32 [T]) of `hidden @ lm_head_weight.T` without
    materialising the [T, vocab] logits: the lm_head GEMM reduces every 128-row weight tile to a
    (max, sum exp, argmax) triple per token in its epilogue and a second kernel folds the triples in a
    fixed order.  Same tokens as `linear` + `greedy_token_and_logprob` (logits rounded to bf16, lowest
    index on ties); log-probabilities within 2e-5 of theirs; a token's result does not depend on T."""
    if not hidden.is_cuda or not lm_head_weight.is_cuda:
        raise ValueError("hidden and lm_head_weight must be CUDA tensors")
    if hidden.dtype != torch.bfloat16 or lm_head_weight.dtype != torch.bfloat16:
        raise NotImplementedError("the fused head is implemented for bf16")
    x = hidden.reshape(-1, hidden.shape[-1])
    if x.stride(-1) != 1:
        x = x.contiguous()
    w = lm_head_weight if lm_head_weight.stride(-1) == 1 else lm_head_weight.contiguous()
    T, K = x.shape
    V = w.shape[0]
    assert w.shape[1] == K, "Incompatible dimensions"
    partials = torch.empty((T, (V + 127) // 128, 4), device=x.device, dtype=torch.float32)
    tokens = torch.empty((T,), device=x.device, dtype=torch.int64)
    lp = torch.empty((T,), device=x.device, dtype=torch.float32)
    _lib.check(
        _lib.load().b200_lm_head_greedy(x.data_ptr(), w.data_ptr(), partials.data_ptr(), tokens.data_ptr(),
                                        lp.data_ptr(), T, V, K, x.stride(0), w.stride(0), _lib.current_stream()),
        "b200_lm_head_greedy",
    )
    return tokens, lp
