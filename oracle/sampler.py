"""CPU restatement of the reference's token sampler (TEST INFRASTRUCTURE ONLY: nothing in the
product imports this file).

Follows vexact/inferencer/sampler.py: `Sampler.batch_sample_token` (:32-87: fp32 cast :47,
temperature :70-71, top-k / top-p :73, softmax + `_random_sample` :80-81, greedy :84),
`apply_top_k_top_p` (:148-186, the sort-based form: top-k threshold :168-173, ascending cumulative
probability <= 1 - p masked with the last element kept :175-181) and `_random_sample` (:120-146:
argmax of probs / q with q ~ Exp(1)).  The exponential noise is an argument here, so a test can
hand over the very draw the reference made.  Pinned against tests/golden/sampler.pt, which the
reference's own sampler produced.
"""
from __future__ import annotations

from typing import Optional

import torch


def apply_top_k_top_p(logits: torch.Tensor, k: Optional[int], p: Optional[float]) -> torch.Tensor:
    """Masked fp32 logits (-inf outside the kept set), sampler.py:148-186."""
    if k is None and p is None:
        return logits
    logits_sort, logits_idx = logits.sort(dim=-1, descending=False)
    if k is not None:
        kth = logits_sort[:, logits_sort.size(1) - k].unsqueeze(1)
        logits_sort = logits_sort.masked_fill(logits_sort < kth, -float("inf"))
    if p is not None:
        probs_sum = torch.cumsum(logits_sort.softmax(dim=-1), dim=-1)
        mask = probs_sum <= 1 - p
        mask[:, -1] = False
        logits_sort = logits_sort.masked_fill(mask, -float("inf"))
    return logits_sort.scatter(dim=-1, index=logits_idx, src=logits_sort)


def sample(logits: torch.Tensor, do_sample: bool, temperature: float, top_k: Optional[int], top_p: float,
           q: Optional[torch.Tensor]) -> torch.Tensor:
    """Tokens `batch_sample_token` returns for uniform sampling parameters and the noise q."""
    x = logits.to(torch.float32).clone()
    k = None if (top_k is None or int(top_k) <= 0) else int(top_k)
    if not (do_sample and temperature > 0 and float(top_p) > 0):
        return x.argmax(dim=-1).view(-1)
    if temperature != 1.0:
        x.div_(temperature)
    x = apply_top_k_top_p(x, k, float(top_p))
    probs = torch.softmax(x, dim=-1)
    return probs.div_(q).argmax(dim=-1).view(-1)


def kept_mask(logits: torch.Tensor, temperature: float, top_k: Optional[int], top_p: float) -> torch.Tensor:
    """Boolean mask of the tokens that survive temperature + top-k + top-p."""
    x = logits.to(torch.float32).clone()
    if temperature != 1.0:
        x.div_(temperature)
    k = None if (top_k is None or int(top_k) <= 0) else int(top_k)
    return apply_top_k_top_p(x, k, float(top_p)) > -float("inf")
