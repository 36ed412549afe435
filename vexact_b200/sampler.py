"""Token sampler: mirror of `vexact.inferencer.sampler.Sampler` (sampler.py:29-212) on one kernel.

`batch_sample_token(batched_logits, gen_configs, sampling_positions=None)` keeps the reference's
signature and rules (uniform parameters across the batch, greedy unless do_sample with
temperature > 0 and top_p > 0, top_k <= 0 means off).  Temperature, top-k, top-p, the
exponential-noise arg-max and the chosen tokens' log-probabilities run in `b200_sample_token`; the
noise is one `exponential_()` draw of the logits' shape from torch's CUDA generator, exactly the
draw the reference's `_random_sample` makes, so both consume the random stream alike.
Per-request seeds (the reference delegates those to vLLM's Gumbel kernel) are not covered.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _lib


def sample_token_and_logprob(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None,
                             top_p: float = 1.0, do_sample: bool = True, noise: Optional[torch.Tensor] = None):
    """(tokens int64 [rows], logprobs fp32 [rows]) for 2-D fp32 / bf16 CUDA logits."""
    if logits.dim() != 2:
        raise ValueError("logits must be [rows, vocab]")
    if not logits.is_cuda:
        raise _lib.B200Error("the sampler is a CUDA kernel: no CPU path")
    if logits.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"unsupported logits dtype {logits.dtype}")
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    rows, n = logits.shape
    k = 0 if (top_k is None or int(top_k) <= 0) else int(top_k)
    sampling = bool(do_sample) and temperature > 0 and float(top_p) > 0
    if sampling and noise is None:
        noise = torch.empty(rows, n, dtype=torch.float32, device=logits.device).exponential_()
    if sampling and (noise.shape != logits.shape or noise.dtype != torch.float32 or noise.stride(1) != 1):
        raise ValueError("noise must be fp32 with the logits' shape")
    tokens = torch.empty(rows, dtype=torch.long, device=logits.device)
    logprobs = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lib = _lib.load()
    rc = lib.b200_sample_token(
        logits.data_ptr(), noise.data_ptr() if sampling else None, tokens.data_ptr(), logprobs.data_ptr(), rows, n,
        logits.stride(0), noise.stride(0) if sampling else 0, 0 if logits.dtype == torch.float32 else 1,
        float(temperature) if sampling else 1.0, k, float(top_p), _lib.current_stream())
    _lib.check(rc, "b200_sample_token")
    return tokens, logprobs


class Sampler:
    """Drop-in for the reference's `Sampler` (uniform sampling parameters, unseeded requests)."""

    @torch.inference_mode()
    def batch_sample_token(self, batched_logits: torch.Tensor, gen_configs: Sequence,
                           sampling_positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        tokens, self.last_logprobs = self.batch_sample_token_and_logprob(batched_logits, gen_configs)
        return tokens

    @torch.inference_mode()
    def batch_sample_token_and_logprob(self, batched_logits: torch.Tensor, gen_configs: Sequence):
        cfg = gen_configs[0]
        p = cfg.top_p
        assert p is not None, "top_p must be set (use 1.0 to disable)"
        if any(getattr(c, "seed", None) is not None for c in gen_configs):
            raise NotImplementedError("per-request seeded sampling is not covered")
        do_sample = bool(cfg.do_sample) and cfg.temperature > 0 and float(p) > 0
        return sample_token_and_logprob(batched_logits, float(cfg.temperature), cfg.top_k, float(p), do_sample)
