"""Generates tests/golden/sampler.pt from the reference's own sampler.

    python tests/golden/make_sampler_golden.py /path/to/vexact

`Sampler.batch_sample_token` (vexact/inferencer/sampler.py:32-87) runs on CPU through its torch
path: the two optional vLLM hooks are switched off (`vllm_apply_top_k_top_p = None` selects the
sort-based `apply_top_k_top_p` of :148-186, and no request sets a seed, so `_random_sample`
:120-146 draws `q.exponential_()` from the default generator).  The generator is seeded right
before each call, and the same seed regenerates the noise `q` the sampler drew, which is stored
with the logits, the sampling parameters and the tokens the reference chose.
"""
from __future__ import annotations

import os
import sys

os.environ.setdefault("VEXACT_DISABLE_MODEL_PATCH", "1")
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("VEXACT_SRC", "")
if not os.path.isdir(REF):
    raise SystemExit("usage: pass the path of a vexact checkout (or set VEXACT_SRC)")
sys.path.insert(0, REF)

import torch  # noqa: E402
from transformers import GenerationConfig  # noqa: E402

import vexact.inferencer.sampler as ref_sampler  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def run_case(seed, rows, vocab, dtype, std, do_sample, temperature, top_k, top_p):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(rows, vocab, generator=g) * std).to(dtype)
    cfgs = [GenerationConfig(do_sample=do_sample, temperature=temperature, top_k=top_k, top_p=top_p)
            for _ in range(rows)]
    torch.manual_seed(1000 + seed)
    tokens = ref_sampler.Sampler().batch_sample_token(logits.clone(), cfgs)
    torch.manual_seed(1000 + seed)
    q = torch.empty(rows, vocab, dtype=torch.float32).exponential_()   # what _random_sample drew
    return dict(logits=logits, q=q if do_sample else None, do_sample=do_sample, temperature=temperature,
                top_k=top_k, top_p=top_p, tokens=tokens)


def main():
    ref_sampler.vllm_apply_top_k_top_p = None
    ref_sampler.vllm_gumbel_sample = None
    f32, bf16 = torch.float32, torch.bfloat16
    cases = [
        run_case(1, 6, 4096, f32, 2.0, True, 0.7, 50, 0.9),
        run_case(2, 1, 151936, bf16, 2.0, True, 1.0, -1, 1.0),     # the usual rollout setting
        run_case(3, 4, 16000, f32, 3.0, True, 1.3, -1, 0.8),
        run_case(4, 4, 16000, f32, 3.0, True, 0.5, 1000, 1.0),
        run_case(5, 4, 8192, bf16, 4.0, True, 0.9, 20, 0.95),
        run_case(6, 2, 20000, f32, 2.0, True, 1.0, 1, 1.0),        # top-1 == greedy
        run_case(7, 3, 20000, bf16, 2.0, False, 1.0, -1, 1.0),     # do_sample off: argmax
        run_case(8, 4, 1000, f32, 1.0, True, 2.0, 1000, 0.3),      # k == vocab, small p
    ]
    torch.save(cases, os.path.join(OUT, "sampler.pt"))
    for c in cases:
        print(tuple(c["logits"].shape), c["logits"].dtype, c["temperature"], c["top_k"], c["top_p"], c["tokens"].tolist())


if __name__ == "__main__":
    main()
