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


def philox4x32_10(counter, key):
    """Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11) on
    numpy uint32 arrays: counter = (c0, c1, c2, c3), key = (k0, k1); returns the four output words."""
    import numpy as np

    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) for c in counter)
    k0, k1 = (np.asarray(k, dtype=np.uint64) for k in key)
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return c0, c1, c2, c3


def seeded_exponential(seeds, positions, vocab: int) -> torch.Tensor:
    """Exp(1) noise [rows, vocab] for seeded requests, the construction of sampler.py:57-63, 90-118 (a
    stream per request seed, advanced by the position of the sampled token): Philox key = the 64-bit seed,
    counter = (column // 4, position low, position high, 0), u = (x + 0.5) * 2^-32, q = -ln(u).  The uniforms
    are exact here; the logarithm is float64 rounded to fp32, so a device result may differ by an ulp."""
    import numpy as np

    rows = len(seeds)
    out = np.empty((rows, vocab), dtype=np.float32)
    quads = (vocab + 3) // 4
    quad = np.arange(quads, dtype=np.uint64)
    for r in range(rows):
        seed, pos = int(seeds[r]) & (2**64 - 1), int(positions[r]) & (2**64 - 1)
        words = philox4x32_10((quad, np.full(quads, pos & 0xFFFFFFFF), np.full(quads, pos >> 32), np.zeros(quads)),
                              (np.full(quads, seed & 0xFFFFFFFF), np.full(quads, seed >> 32)))
        x = np.stack(words, axis=1).reshape(-1)[:vocab].astype(np.float32)       # the kernel converts to fp32 first
        u = (x + np.float32(0.5)) * np.float32(2.3283064365386963e-10)
        out[r] = (-np.log(u.astype(np.float64))).astype(np.float32)
    return torch.from_numpy(out)
