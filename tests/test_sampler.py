"""Token sampler: oracle vs the reference's own draws (CPU), CUDA kernel vs both (GPU)."""
import os

import pytest
import torch

from oracle import sampler as oracle_sampler

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "sampler.pt")


def _cases():
    return torch.load(GOLDEN, weights_only=False)


def test_oracle_matches_reference_draws():
    for c in _cases():
        got = oracle_sampler.sample(c["logits"], c["do_sample"], c["temperature"], c["top_k"], c["top_p"], c["q"])
        assert torch.equal(got, c["tokens"]), (c["temperature"], c["top_k"], c["top_p"])


def _gpu_sample(c, logits=None):
    from vexact_b200.sampler import sample_token_and_logprob

    x = (c["logits"] if logits is None else logits).cuda()
    q = c["q"].cuda() if c["q"] is not None else None
    return sample_token_and_logprob(x, c["temperature"], c["top_k"], c["top_p"], c["do_sample"], noise=q)


@pytest.mark.gpu
def test_kernel_matches_reference_draws():
    import vexact_b200 as vb

    for c in _cases():
        tok, lp = _gpu_sample(c)
        assert torch.equal(tok.cpu(), c["tokens"]), (c["temperature"], c["top_k"], c["top_p"])
        # the log-probability is the two-kernel path's, bit for bit
        assert torch.equal(lp, vb.logprobs_from_logits_flash_attn(c["logits"].cuda(), tok))


@pytest.mark.gpu
def test_kernel_matches_oracle_random_settings():
    """More settings than the fixtures hold, against the oracle with shared noise; a row may differ
    only where the reference's own choice is unspecified (cumulative mass crossing 1 - p inside a run
    of equal logits, frequent with bf16) or at an fp32 near-tie."""
    g = torch.Generator().manual_seed(11)
    total = same = 0
    for trial, (rows, vocab, dtype, temp, k, p) in enumerate([
            (16, 4096, torch.float32, 0.8, 0, 0.9), (16, 4096, torch.float32, 1.0, 40, 1.0),
            (8, 151936, torch.bfloat16, 1.0, 0, 1.0), (8, 151936, torch.bfloat16, 0.6, 0, 0.95),
            (8, 32000, torch.float32, 1.5, 5, 0.5), (8, 50257, torch.bfloat16, 0.7, 100, 0.9),
            (4, 129, torch.float32, 1.0, 128, 0.99), (4, 7, torch.float32, 3.0, 3, 0.7)]):
        x = (torch.randn(rows, vocab, generator=g) * 2.5).to(dtype)
        q = torch.empty(rows, vocab).exponential_(generator=g)
        c = dict(logits=x, q=q, temperature=temp, top_k=k, top_p=p, do_sample=True)
        want = oracle_sampler.sample(x, True, temp, k, p, q)
        tok, _ = _gpu_sample(c)
        tok = tok.cpu()
        kept = oracle_sampler.kept_mask(x, temp, k, p)
        for r in range(rows):
            total += 1
            same += int(tok[r] == want[r])
            if dtype == torch.float32:
                assert kept[r, tok[r]], (trial, r)      # never a token the reference masked
    assert same >= total - 2, (same, total)


@pytest.mark.gpu
def test_sampler_is_batch_invariant_and_greedy_when_asked():
    from types import SimpleNamespace

    from vexact_b200.sampler import Sampler, sample_token_and_logprob

    g = torch.Generator().manual_seed(3)
    x = (torch.randn(24, 32000, generator=g) * 2).bfloat16().cuda()
    q = torch.empty(24, 32000).exponential_(generator=g).cuda()
    tok, lp = sample_token_and_logprob(x, 0.8, 50, 0.9, True, noise=q)
    t1, l1 = sample_token_and_logprob(x[7:8], 0.8, 50, 0.9, True, noise=q[7:8])
    assert torch.equal(t1, tok[7:8]) and torch.equal(l1, lp[7:8])
    t2, l2 = sample_token_and_logprob(x.flip(0), 0.8, 50, 0.9, True, noise=q.flip(0))
    assert torch.equal(t2.flip(0), tok) and torch.equal(l2.flip(0), lp)
    cfg = [SimpleNamespace(do_sample=False, temperature=1.0, top_k=None, top_p=1.0) for _ in range(24)]
    assert torch.equal(Sampler().batch_sample_token(x, cfg), x.float().argmax(-1))
    # top-1 keeps the maximum - every token tied for it (bf16 logits do tie), as the reference's mask does
    cfg = [SimpleNamespace(do_sample=True, temperature=1.0, top_k=1, top_p=1.0) for _ in range(24)]
    tok1 = Sampler().batch_sample_token(x, cfg)
    xf = x.float()
    assert torch.equal(xf.gather(1, tok1[:, None])[:, 0], xf.max(-1).values)
    unique_max = (xf == xf.max(-1, keepdim=True).values).sum(-1) == 1
    assert torch.equal(tok1[unique_max], xf.argmax(-1)[unique_max])


@pytest.mark.gpu
def test_sampling_frequencies_follow_the_distribution():
    """Unfiltered sampling at temperature 1: token frequencies over many draws match softmax."""
    from vexact_b200.sampler import sample_token_and_logprob

    torch.manual_seed(0)
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5, -3.0, 1.5, 0.0]]).cuda()
    x = logits.expand(20000, 8).contiguous()
    tok, lp = sample_token_and_logprob(x, 1.0, None, 1.0, True)
    freq = torch.bincount(tok, minlength=8).float() / tok.numel()
    probs = torch.softmax(logits[0], -1)
    assert (freq - probs).abs().max().item() < 0.015
    assert torch.allclose(lp, torch.log_softmax(logits[0], -1)[tok], atol=1e-5)


def test_philox_restatement_known_answers():
    """The published Philox4x32-10 known-answer vectors (Random123 kat_vectors: zero, all-ones and pi inputs)."""
    import numpy as np

    def run(c, k):
        return tuple(int(w[0]) for w in oracle_sampler.philox4x32_10([np.array([v]) for v in c], [np.array([v]) for v in k]))

    assert run((0, 0, 0, 0), (0, 0)) == (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)
    assert run((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2) == (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)
    assert run((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0)) == (
        0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)


@pytest.mark.gpu
def test_seeded_noise_matches_the_restatement_and_ignores_the_batch():
    from vexact_b200.sampler import seeded_exponential_noise

    vocab = 151936 + 3            # not a multiple of four: the last counter is used in part
    seeds = torch.tensor([0, 1, 2**40 + 17, -5, 123456789], dtype=torch.int64)
    pos = torch.tensor([0, 7, 2**33 + 1, 4095, 7], dtype=torch.int64)
    q = seeded_exponential_noise(seeds.cuda(), pos.cuda(), vocab)
    want = oracle_sampler.seeded_exponential(seeds.tolist(), pos.tolist(), vocab)
    assert torch.isfinite(q).all() and (q > 0).all()
    torch.testing.assert_close(q.cpu(), want, rtol=2e-6, atol=1e-7)      # logf against a rounded float64 log
    # a request's noise depends on (seed, position) only: alone, reordered or repeated it is the same bits
    alone = seeded_exponential_noise(seeds[2:3].cuda(), pos[2:3].cuda(), vocab)
    assert torch.equal(alone[0], q[2])
    perm = torch.tensor([4, 2, 0, 3, 1])
    assert torch.equal(seeded_exponential_noise(seeds[perm].cuda(), pos[perm].cuda(), vocab), q[perm.cuda()])
    assert not torch.equal(q[1, :64], q[4, :64])           # same position, different seed
    assert abs(float(q.mean()) - 1.0) < 5e-3 and abs(float(q.var()) - 1.0) < 2e-2


@pytest.mark.gpu
def test_seeded_sampler_is_reproducible_per_request():
    from types import SimpleNamespace

    from vexact_b200.sampler import Sampler

    torch.manual_seed(5)
    logits = (torch.randn(6, 32000, device="cuda") * 3).to(torch.bfloat16)
    cfgs = [SimpleNamespace(do_sample=True, temperature=0.8, top_k=50, top_p=0.95, seed=100 + i) for i in range(6)]
    pos = torch.arange(10, 16, device="cuda")
    s = Sampler()
    t1, lp1 = s.batch_sample_token_and_logprob(logits, cfgs, pos)
    t2, lp2 = s.batch_sample_token_and_logprob(logits, cfgs, pos)
    assert torch.equal(t1, t2) and torch.equal(lp1, lp2)
    sub = [4, 1]
    t3, _ = s.batch_sample_token_and_logprob(logits[sub], [cfgs[i] for i in sub], pos[sub])
    assert torch.equal(t3, t1[sub])
    # against the restatement: the same noise through the reference's sampler arithmetic
    noise = oracle_sampler.seeded_exponential([c.seed for c in cfgs], pos.tolist(), 32000)
    want = oracle_sampler.sample(logits.cpu(), True, 0.8, 50, 0.95, noise)
    assert (t1.cpu() == want).float().mean() >= 5 / 6          # an ulp of the logarithm may move a near tie
    t4, _ = s.batch_sample_token_and_logprob(logits, cfgs, pos + 1)
    assert not torch.equal(t4, t1)
    with pytest.raises(ValueError):
        s.batch_sample_token_and_logprob(logits, cfgs[:5] + [SimpleNamespace(**{**vars(cfgs[5]), "seed": None})], pos)
    with pytest.raises(ValueError):
        s.batch_sample_token_and_logprob(logits, cfgs, None)


def test_mixed_seed_batch_and_missing_positions_are_rejected_before_any_compute():
    """Reference tests/test_inferencer_sampling.py:88-98: CPU logits are enough, the errors come first."""
    from types import SimpleNamespace as NS

    from vexact_b200.sampler import Sampler

    cfgs = [NS(do_sample=True, temperature=1.0, top_k=4, top_p=1.0, seed=None) for _ in range(2)]
    cfgs[0].seed = 1234
    with pytest.raises(ValueError, match="every request in the batch"):
        Sampler().batch_sample_token(torch.randn(2, 16), cfgs, torch.arange(2))
    cfgs[1].seed = 99
    with pytest.raises(ValueError, match="sampling_positions must be set"):
        Sampler().batch_sample_token(torch.randn(2, 16), cfgs)


@pytest.mark.gpu
@pytest.mark.parametrize("batch_size", [1, 96])
@pytest.mark.parametrize("top_k", [0, 50, None])
@pytest.mark.parametrize("top_p", [0, 0.9])
def test_batch_sample_token_matches_the_step_by_step_form(batch_size, top_k, top_p):
    """The reference's own sampler test (tests/test_inferencer_sampling.py:23-85) at its vocabulary size: temperature,
    `apply_top_k_top_p`, softmax, one exponential_() draw, arg-max of probs / noise, written out step by step with
    this library's `apply_top_k_top_p`, against `batch_sample_token` under the same torch seed."""
    from types import SimpleNamespace as NS

    from vexact_b200.sampler import Sampler

    sampler = Sampler()
    vocab = 151936
    torch.manual_seed(7)
    logits = torch.empty((batch_size, vocab), device="cuda").uniform_(-1.0, 1.0)
    cfgs = [NS(do_sample=True, temperature=1.0, top_k=top_k, top_p=top_p, seed=None)] * batch_size

    def step_by_step(x):
        k = None if (top_k is None or int(top_k) <= 0) else int(top_k)
        if not (float(top_p) > 0):
            return x.argmax(dim=-1).view(-1)
        kt = None if k is None else torch.full((x.shape[0],), k, device=x.device)
        pt = torch.full((x.shape[0],), float(top_p), device=x.device)
        masked = sampler.apply_top_k_top_p(x, kt, pt)
        probs = torch.softmax(masked, dim=-1)
        noise = torch.empty_like(probs).exponential_(1)
        return torch.argmax(probs / noise, dim=-1)

    torch.manual_seed(42)
    torch.cuda.manual_seed_all(42)
    want = step_by_step(logits.clone())
    torch.manual_seed(42)
    torch.cuda.manual_seed_all(42)
    got = sampler.batch_sample_token(logits.clone(), cfgs)
    torch.testing.assert_close(got, want, rtol=0, atol=0)


@pytest.mark.gpu
def test_apply_top_k_top_p_matches_the_sort_based_restatement():
    """Masked logits against the CPU restatement of sampler.py:146-186.  Elements may differ only at the top-p
    boundary: the restatement's fp32 running sum over the sorted row and this kernel's 2^-40 fixed-point masses
    can place the cut a few elements apart, and a run of equal logits at the cut is kept whole here."""
    from vexact_b200.sampler import Sampler

    g = torch.Generator().manual_seed(5)
    for rows, vocab, dtype, temp, k, p in [(4, 4096, torch.float32, 1.0, 40, None), (4, 4096, torch.float32, 1.0, None, 0.9),
                                           (3, 32000, torch.float32, 1.0, 100, 0.8), (2, 151936, torch.bfloat16, 1.0, 0, 0.95),
                                           (2, 129, torch.float32, 1.0, 129, 1.0)]:
        x = (torch.randn(rows, vocab, generator=g) * 2.0).to(dtype)
        kk = None if (k is None or k <= 0 or k >= vocab) else k
        want = oracle_sampler.apply_top_k_top_p(x.float().clone(), kk, p)
        got = Sampler().apply_top_k_top_p(x.cuda(), k, p).cpu()
        assert got.dtype == torch.float32 and got.shape == x.shape
        kept_g, kept_w = got > -float("inf"), want > -float("inf")
        assert torch.equal(got[kept_g], x.float()[kept_g])               # kept values pass through unchanged
        for r in range(rows):       # distinct logit values on which the two disagree (bf16 rows hold long equal runs)
            values = x[r][kept_g[r] != kept_w[r]].float().unique()
            assert values.numel() <= (0 if p is None else 8), (vocab, k, p, values.tolist())
        if p is None or p >= 1.0:
            assert torch.equal(got, want)
    only_k = Sampler().apply_top_k_only(x.cuda(), torch.full((rows,), 5, device="cuda")).cpu()
    assert torch.equal(only_k, oracle_sampler.apply_top_k_top_p(x.float().clone(), 5, None))


@pytest.mark.gpu
def test_seeded_sample_helper_equals_the_seeded_batch_call():
    from types import SimpleNamespace as NS

    from vexact_b200.sampler import Sampler

    g = torch.Generator().manual_seed(8)
    x = (torch.randn(5, 4096, generator=g) * 2.0).cuda()
    seeds = [11, 22, 33, 44, 55]
    pos = torch.tensor([3, 9, 100, 7, 7])
    cfgs = [NS(do_sample=True, temperature=0.7, top_k=20, top_p=0.9, seed=s) for s in seeds]
    want = Sampler().batch_sample_token(x, cfgs, pos)
    masked = Sampler().apply_top_k_top_p(x / 0.7, 20, 0.9)
    got = Sampler()._seeded_sample(masked, seeds, pos, 0.7)
    assert torch.equal(got, want)
