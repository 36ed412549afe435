"""BASELINE configurations 2, 3, 4 and 5 at (or near) their stated sizes, checked through
size-independent properties: a sequence's logits are the same bits alone or inside the full batch,
captured-graph replay equals eager execution, and chunked prefill equals one-shot prefill.
(Configuration 1 is the operator sweep in test_gpu_gemm / test_gpu_rowops.)"""
import dataclasses

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _decode_inputs(shape, S, ctx, page, dev, seed):
    from vexact_b200.inferencer import StepInputs

    g = torch.Generator().manual_seed(seed)
    pages = (ctx + page - 1) // page
    ptab = torch.randperm(S * pages, generator=g).view(S, pages).to(torch.int32)   # seeded random page table
    slots = (ptab[:, (ctx - 1) // page].long() * page + (ctx - 1) % page).to(torch.int32)
    inp = StepInputs(input_ids=torch.randint(0, shape.vocab, (S,), generator=g).to(dev), hidden_in=None,
                     positions=torch.full((S,), ctx - 1, dtype=torch.int64, device=dev), slot_mapping=slots.to(dev),
                     query_start_loc=torch.arange(S + 1, dtype=torch.int32, device=dev),
                     context_lens=torch.full((S,), ctx, dtype=torch.int32, device=dev), block_tables=ptab.to(dev),
                     max_seqlen_q=1)
    return inp, S * pages


def _single(inp, s, dev):
    return dataclasses.replace(
        inp, input_ids=inp.input_ids[s:s + 1], positions=inp.positions[s:s + 1], slot_mapping=inp.slot_mapping[s:s + 1],
        query_start_loc=torch.tensor([0, 1], dtype=torch.int32, device=dev), context_lens=inp.context_lens[s:s + 1],
        block_tables=inp.block_tables[s:s + 1].contiguous())


def _check_decode_invariance(shape, S, ctx, page, picks, router_bias=None):
    from vexact_b200.inferencer import StageRunner, StageWeights, allocate_kv_cache

    dev = torch.device("cuda")
    w = StageWeights.random_init(shape, device=dev, seed=5)
    if router_bias is not None:
        for lw in w.layers:
            lw.router_logit_bias = router_bias.to(dev)
    inp, nblocks = _decode_inputs(shape, S, ctx, page, dev, seed=6)
    kc, vc = allocate_kv_cache(shape, 0, shape.num_layers, nblocks, page, device=dev, fill_std=1.0, seed=7)
    r = StageRunner(w, kc, vc)
    tok, lp, logits = [t.clone() for t in r.step(inp)]
    assert torch.isfinite(logits.float()).all() and torch.isfinite(lp).all()
    graph, out = r.capture(inp)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out[2], logits) and torch.equal(out[1], lp) and torch.equal(out[0], tok)
    for s in picks:
        t1, l1, g1 = r.step(_single(inp, s, dev))
        assert torch.equal(g1[0], logits[s]), f"sequence {s}: logits differ between batch {S} and batch 1"
        assert torch.equal(l1[0], lp[s]) and t1[0] == tok[s]
    from vexact_b200 import _lib

    assert _lib.read_status()[0] == 0
    del kc, vc, w
    torch.cuda.empty_cache()


def test_config2_qwen3_1p7b_decode_batch64_ctx1024_page16():
    from vexact_b200.inferencer import QWEN3_1P7B

    _check_decode_invariance(QWEN3_1P7B, S=64, ctx=1024, page=16, picks=(0, 17, 63))


@pytest.mark.parametrize("skew", [False, True])
def test_config4_qwen3_30b_a3b_shape_decode_batch512_ctx2048_page16(skew):
    """Full width (hidden 2048, 32 / 4 heads, 128 experts top-8, expert FFN 768, vocab 151936), 2 of the
    48 layers, batch 512 x 2048-token context in 16-token pages: sequences 0, 255 and 511 get the same
    bits alone as inside the batch of 512, and a captured-graph replay equals eager execution; once with
    std-0.02 routers (near-uniform expert load) and once with a Zipf(1.1) router bias (tiles of up to 64
    rows per expert, the many-rows-per-expert route of fc1)."""
    from bench import zipf_router_bias
    from vexact_b200.inferencer import QWEN3_30B_A3B

    shape = dataclasses.replace(QWEN3_30B_A3B, num_layers=2)
    bias = zipf_router_bias(shape.moe.num_experts, seed=11) if skew else None
    _check_decode_invariance(shape, S=512, ctx=2048, page=16, picks=(0, 255, 511), router_bias=bias)


def test_config5_moonlight_shape_decode_batch256_ctx4096():
    """27-layer shape cut to its first 3 layers (1 dense + 2 MoE): the full KV cache of this workload
    (290 GB as the reference stores it) does not fit one GPU, which is why the workload is PP >= 2."""
    from vexact_b200.inferencer import MOONLIGHT_16B_A3B

    shape = dataclasses.replace(MOONLIGHT_16B_A3B, num_layers=3)
    _check_decode_invariance(shape, S=256, ctx=4096, page=16, picks=(0, 100, 255))


def test_config3_qwen2_1p5b_chunked_prefill_then_decode():
    """Prompts of mixed length prefilled in 2048-token chunks give, token for token, the bits of a
    one-shot prefill; the following decode step is batch invariant.  4 of the 28 layers."""
    from vexact_b200.inferencer import QWEN2_1P5B, StageRunner, StageWeights, StepInputs, allocate_kv_cache

    dev = torch.device("cuda")
    shape = dataclasses.replace(QWEN2_1P5B, num_layers=4)
    page, chunk = 16, 2048
    lens = [256, 2500, 1031]
    g = torch.Generator().manual_seed(8)
    pages = [(n + 1 + page - 1) // page for n in lens]
    maxp = max(pages)
    perm = torch.randperm(sum(pages), generator=g).tolist()
    ptab = torch.full((len(lens), maxp), -1, dtype=torch.int32)
    k = 0
    for s, p in enumerate(pages):
        ptab[s, :p] = torch.tensor(perm[k:k + p], dtype=torch.int32)
        k += p
    ids = [torch.randint(0, shape.vocab, (n + 1,), generator=g) for n in lens]   # prompt + one decoded token
    w = StageWeights.random_init(shape, device=dev, seed=9)

    def make(parts):
        """parts: list of (seq, start, end) token ranges processed in one step."""
        tok = torch.cat([ids[s][a:b] for s, a, b in parts])
        pos = torch.cat([torch.arange(a, b) for s, a, b in parts])
        slots = torch.cat([ptab[s, torch.arange(a, b) // page].long() * page + torch.arange(a, b) % page
                           for s, a, b in parts]).to(torch.int32)
        cu = torch.tensor([0] + torch.tensor([b - a for _, a, b in parts]).cumsum(0).tolist(), dtype=torch.int32)
        return StepInputs(input_ids=tok.to(dev), hidden_in=None, positions=pos.to(dev), slot_mapping=slots.to(dev),
                          query_start_loc=cu.to(dev), context_lens=torch.tensor([b for _, _, b in parts], dtype=torch.int32, device=dev),
                          block_tables=torch.stack([ptab[s] for s, _, _ in parts]).to(dev),
                          max_seqlen_q=max(b - a for _, a, b in parts))

    def run(plan):
        kc, vc = allocate_kv_cache(shape, 0, shape.num_layers, sum(pages), page, device=dev)
        r = StageRunner(w, kc, vc)
        last = {}
        for parts in plan:
            _, _, logits = r.step(make(parts))
            for i, (s, a, b) in enumerate(parts):
                if b == lens[s]:
                    last[s] = logits[i].clone()
        return r, kc, vc, last

    one_shot = [[(s, 0, lens[s]) for s in range(len(lens))]]
    # token budget 2048 per step, sequences packed in order (the reference scheduler's chunking rule)
    chunked = [[(0, 0, 256), (1, 0, chunk - 256)], [(1, chunk - 256, 2500), (2, 0, 1031)]]
    r1, kc1, vc1, last1 = run(one_shot)
    r2, kc2, vc2, last2 = run(chunked)
    for s in range(len(lens)):
        assert torch.equal(last1[s], last2[s]), f"sequence {s}: chunked prefill changed the last-token logits"
    for li in kc1:
        assert torch.equal(kc1[li], kc2[li]) and torch.equal(vc1[li], vc2[li])
    # decode one token for every sequence: batch vs single
    dec = make([(s, lens[s], lens[s] + 1) for s in range(len(lens))])
    _, lp, logits = [t.clone() for t in r1.step(dec)]
    for s in range(len(lens)):
        _, l1, g1 = r1.step(_single(dec, s, dev))
        assert torch.equal(g1[0], logits[s]) and torch.equal(l1[0], lp[s])
