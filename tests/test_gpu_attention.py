"""GPU parity: paged causal attention vs the reference kernel's golden outputs, the fp32 eager
ground truth the reference tests use, and the bitwise invariance properties of
tests/batch_invariant_ops/test_triton_attention_varlen.py:398-558 (batched == single sequence,
prefill last token == decode, chunked == full prefill, MLA head dims)."""
import os

import pytest
import torch

from conftest import load_golden
from oracle import ops

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def vb():
    import vexact_b200 as vb

    vb._lib.load()
    return vb


def _build(q_lens, kv_lens, hq, hkv, dk, dv, page, seed=0, extra_blocks=3):
    g = torch.Generator().manual_seed(seed)
    S = len(q_lens)
    max_pages = max((kl + page - 1) // page for kl in kv_lens)
    nblocks = S * max_pages + extra_blocks
    perm = torch.randperm(nblocks, generator=g)
    kc = (torch.randn(nblocks, page, hkv, dk, generator=g)).to(BF)
    vc = (torch.randn(nblocks, page, hkv, dv, generator=g)).to(BF)
    ptab = torch.full((S, max_pages), -1, dtype=torch.int32)
    nxt = 0
    for s in range(S):
        for pg in range((kv_lens[s] + page - 1) // page):
            ptab[s, pg] = perm[nxt]
            nxt += 1
    q = torch.randn(sum(q_lens), hq, dk, generator=g).to(BF)
    cu = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32)
    used = torch.tensor(kv_lens, dtype=torch.int32)
    return q, kc, vc, cu, used, ptab


def _run(vb, q, kc, vc, cu, used, ptab, scale, max_q):
    out, none = vb.flash_attn_varlen_func(q.cuda(), kc.cuda(), vc.cuda(), cu_seqlens_q=cu.cuda(),
                                          max_seqlen_q=max_q, seqused_k=used.cuda(), page_table=ptab.cuda(),
                                          softmax_scale=scale, causal=True)
    assert none is None
    return out.cpu()


def test_golden_reference_kernel(vb):
    for c in load_golden("paged_attention"):
        qlens = (c["cu_seqlens_q"][1:] - c["cu_seqlens_q"][:-1]).tolist()
        out = _run(vb, c["q"], c["k_cache"], c["v_cache"], c["cu_seqlens_q"], c["seqused_k"], c["page_table"],
                   c["scale"], max(qlens))
        # reference tolerance, bf16 paged vs fp32 eager: atol 3e-3 on unit-variance inputs
        # (test_triton_attention_varlen.py:415); outputs here reach |o| ~ 3, one bf16 ulp = 1.6e-2
        torch.testing.assert_close(out.float(), c["out_triton_fp32"], rtol=2 ** -7, atol=3e-3)
        torch.testing.assert_close(out.float(), c["out_eager_fp32"], rtol=2 ** -7, atol=3e-3)


@pytest.mark.parametrize("hq,hkv,dk,dv,page", [(32, 4, 128, 128, 16), (16, 8, 128, 128, 16), (12, 2, 128, 128, 64),
                                               (16, 8, 128, 128, 256), (16, 16, 192, 128, 16), (4, 4, 64, 64, 16),
                                               (32, 2, 128, 128, 16), (6, 2, 128, 128, 8), (5, 1, 128, 128, 32)])
def test_oracle_mixed_batch(vb, hq, hkv, dk, dv, page):
    q_lens = [1, 5, 1, 17, 64, 1]
    kv_lens = [1, 5, 130, 200, 64, 257]
    q, kc, vc, cu, used, ptab = _build(q_lens, kv_lens, hq, hkv, dk, dv, page, seed=1)
    scale = dk ** -0.5
    out = _run(vb, q, kc, vc, cu, used, ptab, scale, max(q_lens))
    ref = ops.paged_attention(q, kc, vc, cu, used, ptab, scale, block_n=64)
    eager = ops.paged_attention(q, kc, vc, cu, used, ptab, scale)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2 ** -7, atol=3e-3)
    torch.testing.assert_close(out.float(), eager.float(), rtol=2 ** -6, atol=6e-3)
    assert (out == ref).float().mean() > 0.9


def test_batched_equals_single_sequence_bitwise(vb):
    q_lens = [1, 9, 1, 33]
    kv_lens = [300, 9, 77, 140]
    hq, hkv, d, page = 32, 4, 128, 16
    q, kc, vc, cu, used, ptab = _build(q_lens, kv_lens, hq, hkv, d, d, page, seed=2)
    scale = d ** -0.5
    full = _run(vb, q, kc, vc, cu, used, ptab, scale, max(q_lens))
    for s in range(len(q_lens)):
        cu1 = torch.tensor([0, q_lens[s]], dtype=torch.int32)
        one = _run(vb, q[cu[s]:cu[s + 1]], kc, vc, cu1, used[s:s + 1], ptab[s:s + 1], scale, q_lens[s])
        assert torch.equal(one, full[cu[s]:cu[s + 1]]), f"sequence {s} differs when batched"


@pytest.mark.parametrize("hq,hkv,dk,dv,page", [(16, 8, 128, 128, 256), (32, 4, 128, 128, 16), (16, 16, 192, 128, 16)])
def test_prefill_chunked_decode_bitwise(vb, hq, hkv, dk, dv, page):
    """Token p's output is the same bits whether it is computed in a full prefill, in a prefill
    chunk, or as a single decode query over p cached tokens."""
    L = 150
    q, kc, vc, cu, used, ptab = _build([L], [L], hq, hkv, dk, dv, page, seed=3)
    scale = dk ** -0.5
    full = _run(vb, q, kc, vc, cu, used, ptab, scale, L)
    # chunked: queries [0,70) over 70 keys, then [70,150) over 150 keys
    c1 = _run(vb, q[:70], kc, vc, torch.tensor([0, 70], dtype=torch.int32), torch.tensor([70], dtype=torch.int32),
              ptab, scale, 70)
    c2 = _run(vb, q[70:], kc, vc, torch.tensor([0, 80], dtype=torch.int32), torch.tensor([150], dtype=torch.int32),
              ptab, scale, 80)
    assert torch.equal(torch.cat([c1, c2]), full)
    # decode: every position as its own one-query sequence of a batch, all sharing the same pages
    pos = [0, 1, 63, 64, 65, 127, 128, 149]
    S = len(pos)
    qd = torch.stack([q[p] for p in pos])
    cu_d = torch.arange(S + 1, dtype=torch.int32)
    used_d = torch.tensor([p + 1 for p in pos], dtype=torch.int32)
    dec = _run(vb, qd, kc, vc, cu_d, used_d, ptab.expand(S, -1).contiguous(), scale, 1)
    for i, p in enumerate(pos):
        assert torch.equal(dec[i], full[p]), f"decode at position {p} differs from prefill"


def test_padding_and_empty_sequences_are_noops(vb):
    # CUDA-graph buckets pad with zero-length sequences (inferencer.py:318-324)
    q_lens = [1, 0, 1, 0]
    kv_lens = [40, 0, 17, 0]
    hq, hkv, d, page = 8, 1, 128, 16
    g = torch.Generator().manual_seed(4)
    kc = torch.randn(8, page, hkv, d, generator=g).to(BF)
    vc = torch.randn(8, page, hkv, d, generator=g).to(BF)
    ptab = torch.tensor([[0, 1, 2], [-1, -1, -1], [3, 4, -1], [-1, -1, -1]], dtype=torch.int32)
    q = torch.randn(2, hq, d, generator=g).to(BF)
    cu = torch.tensor([0, 1, 1, 2, 2], dtype=torch.int32)
    used = torch.tensor(kv_lens, dtype=torch.int32)
    out = _run(vb, q, kc, vc, cu, used, ptab, d ** -0.5, 1)
    ref = ops.paged_attention(q, kc, vc, cu, used, ptab, d ** -0.5, block_n=64)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2 ** -7, atol=3e-3)


def test_unwritten_cache_slots_do_not_leak(vb):
    """Slots past the sequence end may hold anything, NaN bit patterns included."""
    hq, hkv, d, page = 8, 1, 128, 16
    q, kc, vc, cu, used, ptab = _build([1], [21], hq, hkv, d, d, page, seed=5)
    out = _run(vb, q, kc, vc, cu, used, ptab, d ** -0.5, 1)
    kc2, vc2 = kc.clone(), vc.clone()
    blk = int(ptab[0, 1])
    kc2[blk, 5:] = float("nan")
    vc2[blk, 5:] = float("nan")
    out2 = _run(vb, q, kc2, vc2, cu, used, ptab, d ** -0.5, 1)
    assert torch.equal(out, out2)


def test_hf_adapter_stores_then_attends(vb):
    hq, hkv, d, page, L = 16, 8, 128, 16, 40
    g = torch.Generator().manual_seed(6)
    q = torch.randn(1, hq, L, d, generator=g).to(BF).cuda()
    k = torch.randn(1, hkv, L, d, generator=g).to(BF).cuda()
    v = torch.randn(1, hkv, L, d, generator=g).to(BF).cuda()
    kc = {0: torch.zeros(4, page, hkv, d, dtype=BF).cuda()}
    vc = {0: torch.zeros(4, page, hkv, d, dtype=BF).cuda()}
    ptab = torch.tensor([[2, 0, 3]], dtype=torch.int32)
    slots = torch.tensor(ops.slot_mapping([[2, 0, 3]], [0], [L], page))
    vb.set_kv_cache_context(is_paged_attn=True, key_cache=kc, value_cache=vc, block_tables=ptab.cuda(),
                            context_lens=torch.tensor([L], dtype=torch.int32).cuda(), slot_mapping=slots.cuda(),
                            query_start_loc=torch.tensor([0, L], dtype=torch.int32).cuda(), max_seqlen_q=L)
    mod = torch.nn.Module()
    mod.layer_idx = 0
    out, w = vb.flash_attention_forward(mod, q, k, v, None, scaling=d ** -0.5)
    assert w is None and out.shape == (L, hq, d)
    ref = ops.paged_attention(q[0].transpose(0, 1).cpu(), kc[0].cpu(), vc[0].cpu(), [0, L], [L], ptab, d ** -0.5,
                              block_n=64)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2 ** -7, atol=3e-3)


def test_argument_errors(vb):
    q, kc, vc, cu, used, ptab = _build([1], [5], 8, 1, 128, 128, 16)
    with pytest.raises(NotImplementedError):
        vb.flash_attn_varlen_func(q.cuda(), kc.cuda(), vc.cuda(), cu_seqlens_q=cu.cuda(), seqused_k=used.cuda(),
                                  page_table=ptab.cuda(), causal=False)
    with pytest.raises(ValueError):
        vb.flash_attn_varlen_func(q.cuda(), kc.cuda(), vc.cuda(), cu_seqlens_q=cu.cuda(), seqused_k=used.cuda(),
                                  page_table=ptab.cuda(), block_table=ptab.cuda(), causal=True)
    with pytest.raises(ValueError):
        vb.flash_attn_varlen_func(q.cuda(), kc.cuda(), vc.cuda(), cu_seqlens_q=cu.cuda(), seqused_k=used.cuda().long(),
                                  page_table=ptab.cuda(), causal=True)


def test_status_word_clean(vb):
    torch.cuda.synchronize()
    assert vb._lib.read_status()[0] == 0


@pytest.mark.parametrize("case", ["more_queries_than_the_bucket", "fewer_keys_than_queries"])
def test_inconsistent_lengths_are_skipped_and_reported(vb, case):
    """A sequence whose q_len exceeds the max_seqlen_q the grid was sized for (a captured graph replayed with a
    longer chunk), or whose key count is below its query count, is skipped and named in the status word
    (code 2, detail = sequence); the other sequences of the batch are computed as if it were not there."""
    hq, hkv, d, page = 8, 2, 128, 16
    if case == "more_queries_than_the_bucket":
        q_lens, kv_lens, max_q, bad = [1, 5, 1], [40, 70, 33], 1, 1
    else:
        q_lens, kv_lens, max_q, bad = [3, 4, 2], [50, 2, 20], 4, 1
    q, kc, vc, cu, used, ptab = _build(q_lens, kv_lens, hq, hkv, d, d, page, seed=9)
    assert vb._lib.read_status()[0] == 0
    got = _run(vb, q, kc, vc, cu, used, ptab, d ** -0.5, max_q)
    torch.cuda.synchronize()
    code, detail, _, _ = vb._lib.read_status()          # reading clears the word
    assert (code, detail) == (2, bad)
    assert vb._lib.read_status()[0] == 0
    for s in (0, 2):                                    # the well-formed sequences: same bits as when run alone
        a, b = int(cu[s]), int(cu[s + 1])
        alone = _run(vb, q[a:b], kc, vc, torch.tensor([0, b - a], dtype=torch.int32), used[s:s + 1],
                     ptab[s:s + 1], d ** -0.5, max(q_lens[s], 1))
        assert torch.equal(got[a:b], alone)


def test_mma_sync_kernel_cross_check():
    """The mma.sync kernel (fallback for head dims the tcgen05 kernel does not cover) against the same
    oracle, golden and bitwise cases: the kernel choice is read once per process, so a child runs it."""
    import os
    import subprocess
    import sys

    env = dict(os.environ, B200_ATTN="simt")
    here = os.path.abspath(__file__)
    res = subprocess.run([sys.executable, "-m", "pytest", here, "-q", "-m", "gpu", "-x", "-k",
                          "golden or oracle or bitwise or padding or unwritten"], env=env, capture_output=True,
                         text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]


def test_sequence_order_changes_no_result(vb):
    """A processing order (longest context first) only moves tiles between CTAs."""
    g = torch.Generator().manual_seed(21)
    S, hq, hkv, d, page = 37, 16, 4, 128, 16
    lens = torch.randint(1, 700, (S,), generator=g)
    qlens = torch.where(torch.rand(S, generator=g) < 0.3, torch.minimum(lens, torch.randint(1, 90, (S,), generator=g)),
                        torch.ones(S, dtype=torch.long))
    pages = int((int(lens.max()) + page - 1) // page)
    kc = torch.randn(S * pages, page, hkv, d, generator=g).bfloat16().cuda()
    vc = torch.randn(S * pages, page, hkv, d, generator=g).bfloat16().cuda()
    table = torch.randperm(S * pages, generator=g).view(S, pages).int().cuda()
    cu = torch.zeros(S + 1, dtype=torch.int32)
    cu[1:] = qlens.cumsum(0)
    q = torch.randn(int(cu[-1]), hq, d, generator=g).bfloat16().cuda()
    cu, used = cu.cuda(), lens.int().cuda()
    base = vb.paged_attention(q, kc, vc, cu, used, table, d ** -0.5, int(qlens.max()))
    for order in (torch.argsort(lens, descending=True), torch.randperm(S, generator=g), torch.arange(S).flip(0)):
        got = vb.paged_attention(q, kc, vc, cu, used, table, d ** -0.5, int(qlens.max()),
                                 seq_order=order.int().cuda())
        assert torch.equal(got, base)
    with pytest.raises(ValueError):
        vb.paged_attention(q, kc, vc, cu, used, table, d ** -0.5, int(qlens.max()),
                           seq_order=torch.arange(S - 1).int().cuda())


def test_rows_kernel_and_columns_kernel_give_the_same_bits(vb):
    """Head dim 128 prefill runs the rows-on-lanes kernel; B200_ATTN_PREFILL=cols runs the keys-on-lanes
    kernel on the same step.  Both are written to perform the same operations per (position, head), so a
    mixed prefill / chunk / decode batch must come out bit-identical (and equal to decode steps, which
    test_prefill_chunked_decode_bitwise checks against whichever prefill kernel is active)."""
    g = torch.Generator().manual_seed(77)
    for (hq, hkv, page, q_lens, ctx) in [(32, 4, 16, [130, 40, 1, 7], [130, 200, 257, 7]),
                                         (16, 8, 256, [300, 1], [300, 513]),
                                         (12, 2, 16, [257, 64], [1000, 64]),
                                         (16, 1, 16, [70], [70])]:
        S, d = len(ctx), 128
        pages = max((c + page - 1) // page for c in ctx)
        kc = torch.randn(S * pages + 1, page, hkv, d, generator=g).to(BF).cuda()
        vc = torch.randn(S * pages + 1, page, hkv, d, generator=g).to(BF).cuda()
        table = torch.randperm(S * pages, generator=g).view(S, pages).to(torch.int32).cuda()
        q = torch.randn(sum(q_lens), hq, d, generator=g).to(BF).cuda()
        cu = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32).cuda()
        used = torch.tensor(ctx, dtype=torch.int32).cuda()
        kw = dict(cu_seqlens_q=cu, max_seqlen_q=max(q_lens), seqused_k=used, page_table=table,
                  softmax_scale=d ** -0.5, causal=True)
        rows, _ = vb.flash_attn_varlen_func(q, kc, vc, **kw)
        os.environ["B200_ATTN_PREFILL"] = "cols"
        try:
            cols, _ = vb.flash_attn_varlen_func(q, kc, vc, **kw)
        finally:
            del os.environ["B200_ATTN_PREFILL"]
        torch.cuda.synchronize()
        assert torch.equal(rows, cols), f"{(hq, hkv, page, q_lens)}: max diff {(rows.float() - cols.float()).abs().max()}"


def test_query_and_output_tiles_by_tma_change_no_bit(vb):
    """The rows-on-lanes kernel fetches its query tile by TMA and stores a warp's output rows by one TMA store
    when the tile shape allows it, and through a loader warp / per-lane stores otherwise (B200_ATTN_Q_TMA=0,
    B200_ATTN_O_TMA=0 force those): same bits; rows outside the tiles' valid positions (a sequence's last,
    partial tile; the canary rows behind q) are never written."""
    g = torch.Generator().manual_seed(78)
    for (hq, hkv, page, q_lens, ctx) in [(32, 4, 16, [130, 40, 1, 7], [130, 200, 257, 7]),     # groups of 8
                                         (16, 8, 16, [300, 33], [300, 513]),                # groups of 2
                                         (12, 2, 16, [257, 64], [1000, 64]),               # groups of 6: no output box
                                         (16, 1, 16, [70], [70])]:                          # two chunks of 8 heads
        S, d = len(ctx), 128
        pages = max((c + page - 1) // page for c in ctx)
        kc = torch.randn(S * pages + 1, page, hkv, d, generator=g).to(BF).cuda()
        vc = torch.randn(S * pages + 1, page, hkv, d, generator=g).to(BF).cuda()
        table = torch.randperm(S * pages, generator=g).view(S, pages).to(torch.int32).cuda()
        q = torch.randn(sum(q_lens), hq, d, generator=g).to(BF).cuda()
        cu = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32).cuda()
        used = torch.tensor(ctx, dtype=torch.int32).cuda()
        kw = dict(cu_seqlens_q=cu, max_seqlen_q=max(q_lens), seqused_k=used, page_table=table,
                  softmax_scale=d ** -0.5, causal=True)
        with_tma, _ = vb.flash_attn_varlen_func(q, kc, vc, **kw)
        os.environ["B200_ATTN_Q_TMA"] = "0"
        os.environ["B200_ATTN_O_TMA"] = "0"
        try:
            without, _ = vb.flash_attn_varlen_func(q, kc, vc, **kw)
        finally:
            del os.environ["B200_ATTN_Q_TMA"], os.environ["B200_ATTN_O_TMA"]
        torch.cuda.synchronize()
        assert torch.equal(with_tma, without), f"{(hq, hkv, page, q_lens)}"
        # only the first sequence's rows are asked for: the rows of the others must stay untouched
        from vexact_b200.attention import paged_attention

        canary = torch.full_like(with_tma, 7.0)
        paged_attention(q, kc, vc, cu[:2].contiguous(), used[:1].contiguous(), table[:1].contiguous(), d ** -0.5,
                        q_lens[0], out=canary)
        torch.cuda.synchronize()
        assert torch.equal(canary[:q_lens[0]], with_tma[:q_lens[0]])
        assert bool((canary[q_lens[0]:] == 7.0).all())


def test_packed_varlen_forward_equals_paged_prefill_bitwise(vb):
    """The training-side packed call (no page table) must give the rollout's bits: same tokens through the
    packed path and through a paged prefill with another page size and a shuffled page table."""
    g = torch.Generator().manual_seed(91)
    hq, hkv, d = 16, 8, 128
    lens = [70, 1, 300, 33]
    total = sum(lens)
    q = torch.randn(total, hq, d, generator=g).to(BF).cuda()
    k = torch.randn(total, hkv, d, generator=g).to(BF).cuda()
    v = torch.randn(total, hkv, d, generator=g).to(BF).cuda()
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32).cuda()
    packed, _ = vb.flash_attn_varlen_func(q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=max(lens),
                                          max_seqlen_k=max(lens), causal=True)
    page = 64
    pages = max((n + page - 1) // page for n in lens)
    table = torch.randperm(len(lens) * pages, generator=g).view(len(lens), pages).to(torch.int32)
    kc = torch.zeros(len(lens) * pages, page, hkv, d, dtype=BF).cuda()
    vc = torch.zeros_like(kc)
    slots = torch.cat([table[s, torch.arange(n) // page].long() * page + torch.arange(n) % page
                       for s, n in enumerate(lens)]).to(torch.int32).cuda()
    vb.store_kvcache(k, v, kc, vc, slots)
    paged, _ = vb.flash_attn_varlen_func(q, kc, vc, cu_seqlens_q=cu, max_seqlen_q=max(lens),
                                         seqused_k=torch.tensor(lens, dtype=torch.int32).cuda(),
                                         page_table=table.cuda(), causal=True)
    assert torch.equal(packed, paged)
    # the paged call is forward-only under autograd, as the reference's (test_triton_attention_varlen.py:561-569)
    qq = q.clone().requires_grad_(True)
    out, _ = vb.flash_attn_varlen_func(qq, kc, vc, cu_seqlens_q=cu, max_seqlen_q=max(lens),
                                       seqused_k=torch.tensor(lens, dtype=torch.int32).cuda(),
                                       page_table=table.cuda(), causal=True)
    assert torch.equal(out, paged)
    with pytest.raises(NotImplementedError, match="paged triton flash_attn_varlen_func backward"):
        out.float().sum().backward()


def test_flex_key_paged_gives_the_other_keys_bits_and_packed_one_sequence(vb):
    """`attn_impl="flex"` (reference flex_attention.py:280): with a paged context it is the same store + paged
    call as the other keys (same bits); with a packed context it serves one sequence whose q_len queries sit
    at the end of context_len keys, and gives the paged path's bits for the same tokens."""
    hq, hkv, d, page = 16, 8, 128, 16
    past, new = 45, 19
    L = past + new
    g = torch.Generator().manual_seed(17)
    q = torch.randn(1, hq, new, d, generator=g).to(BF).cuda()
    k_all = torch.randn(1, hkv, L, d, generator=g).to(BF).cuda()
    v_all = torch.randn(1, hkv, L, d, generator=g).to(BF).cuda()
    mod = torch.nn.Module()
    mod.layer_idx = 0
    blocks = [3, 0, 2, 4]
    ptab = torch.tensor([blocks], dtype=torch.int32).cuda()
    outs = {}
    for name, fn in (("flash", vb.flash_attention_forward), ("flex", vb.flex_attention_forward)):
        kc = {0: torch.zeros(5, page, hkv, d, dtype=BF).cuda()}
        vc = {0: torch.zeros(5, page, hkv, d, dtype=BF).cuda()}
        past_slots = torch.tensor(ops.slot_mapping([blocks], [0], [past], page)).cuda()
        vb.store_kvcache(k_all[0, :, :past].transpose(0, 1).contiguous(), v_all[0, :, :past].transpose(0, 1).contiguous(),
                         kc[0], vc[0], past_slots)
        slots = torch.tensor(ops.slot_mapping([blocks], [past], [new], page)).cuda()
        vb.set_kv_cache_context(is_paged_attn=True, key_cache=kc, value_cache=vc, block_tables=ptab,
                                context_lens=torch.tensor([L], dtype=torch.int32).cuda(), slot_mapping=slots,
                                query_start_loc=torch.tensor([0, new], dtype=torch.int32).cuda(), max_seqlen_q=new)
        out, w = fn(mod, q, k_all[:, :, past:], v_all[:, :, past:], None, scaling=d ** -0.5)
        assert w is None and out.shape == (new, hq, d)
        outs[name] = out
    assert torch.equal(outs["flash"], outs["flex"])

    # Packed context: the whole key sequence is handed over, with keys past context_len that must stay unseen.
    pad = 7
    k_pad = torch.cat([k_all, torch.full((1, hkv, pad, d), 50.0, dtype=BF).cuda()], dim=2)
    v_pad = torch.cat([v_all, torch.full((1, hkv, pad, d), 50.0, dtype=BF).cuda()], dim=2)
    vb.set_kv_cache_context(is_paged_attn=False, context_lens=torch.tensor([L], dtype=torch.int32).cuda(),
                            query_start_loc=torch.tensor([0, new], dtype=torch.int32).cuda())
    packed, w = vb.flex_attention_forward(mod, q, k_pad, v_pad, None, scaling=d ** -0.5)
    assert w is None and torch.equal(packed, outs["flash"])
    # fp32 statement of the reference's mask (flex_attention.py:104-120): kv_idx <= offset + q_idx, kv_idx < context_len
    qf, kf, vf = q[0].float(), k_pad[0].float().repeat_interleave(hq // hkv, 0), v_pad[0].float().repeat_interleave(hq // hkv, 0)
    s = torch.einsum("hqd,hkd->hqk", qf, kf) * d ** -0.5
    qi = torch.arange(new).cuda()[:, None] + past
    ki = torch.arange(L + pad).cuda()[None, :]
    s = s.masked_fill(~((ki <= qi) & (ki < L)), float("-inf"))
    ref = torch.einsum("hqk,hkd->qhd", torch.softmax(s, -1), vf)
    torch.testing.assert_close(packed.float(), ref, rtol=2 ** -7, atol=3e-3)

    # Several sequences packed into one row: the reference's mask is not meaningful there; this library refuses.
    vb.set_kv_cache_context(is_paged_attn=False, context_lens=torch.tensor([10, 9], dtype=torch.int32).cuda(),
                            query_start_loc=torch.tensor([0, 10, 19], dtype=torch.int32).cuda())
    with pytest.raises(NotImplementedError):
        vb.flex_attention_forward(mod, q, k_all[:, :, :new], v_all[:, :, :new], None, scaling=d ** -0.5)


@pytest.mark.parametrize("head_dim", [32, 40, 96])
def test_packed_varlen_forward_takes_other_head_dims(vb, head_dim):
    """The packed (training-side) call with head dims the kernels do not tile (reference
    tests/batch_invariant_ops/test_triton_attention_varlen.py:289-301 uses 40 and 96): against fp32 eager attention
    (`_eager_attention`, :52-72 there), causal with the queries at the end of the keys."""
    g = torch.Generator().manual_seed(202)
    hq, hkv = 6, 3
    q_lens, kv_lens = [9, 23], [41, 57]
    q = torch.randn(sum(q_lens), hq, head_dim, generator=g).to(BF).cuda()
    k = torch.randn(sum(kv_lens), hkv, head_dim, generator=g).to(BF).cuda()
    v = torch.randn(sum(kv_lens), hkv, head_dim, generator=g).to(BF).cuda()
    cu_q = torch.tensor([0, 9, 32], dtype=torch.int32).cuda()
    cu_k = torch.tensor([0, 41, 98], dtype=torch.int32).cuda()
    out, _ = vb.flash_attn_varlen_func(q, k, v, cu_q, cu_k, max_seqlen_q=max(q_lens), max_seqlen_k=max(kv_lens),
                                       softmax_scale=head_dim ** -0.5, causal=True)
    assert out.shape == q.shape
    qo = ko = 0
    for ql, kl in zip(q_lens, kv_lens):
        qs, ks, vs = q[qo:qo + ql].float(), k[ko:ko + kl].float(), v[ko:ko + kl].float()
        s = torch.einsum("qhd,khd->hqk", qs, ks.repeat_interleave(hq // hkv, 1)) * head_dim ** -0.5
        qi = torch.arange(ql).cuda()[:, None] + (kl - ql)
        s = s.masked_fill(~(torch.arange(kl).cuda()[None, :] <= qi), float("-inf"))
        ref = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vs.repeat_interleave(hq // hkv, 1))
        torch.testing.assert_close(out[qo:qo + ql].float(), ref, rtol=2 ** -7, atol=7e-3)
        qo, ko = qo + ql, ko + kl


def _eager_packed(q, k, v, scale):
    """fp32 causal attention of one sequence, queries at the end of the keys (the reference tests' `_eager_attention`,
    test_triton_attention_varlen.py:52-72, without its bf16 cast of the probabilities)."""
    ql, kl, g = q.shape[0], k.shape[0], q.shape[1] // k.shape[1]
    s = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(g, 1)) * scale
    seen = torch.arange(kl, device=q.device)[None, :] <= torch.arange(ql, device=q.device)[:, None] + (kl - ql)
    s = s.masked_fill(~seen, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v.repeat_interleave(g, 1))


@pytest.mark.parametrize("q_lens,kv_lens,hq,hkv,dk,dv", [
    ([9, 23], [41, 57], 6, 3, 64, 64),          # decode-like chunks at the end of longer contexts, GQA
    ([65, 129], [65, 129], 4, 2, 128, 128),     # full causal prefill, tiles with ragged edges
    ([9, 23], [41, 57], 6, 3, 40, 40),          # a head dim the kernels do not tile (zero columns)
    ([5, 40], [33, 40], 4, 4, 192, 128),        # MLA dims
])
def test_packed_varlen_backward_matches_autograd_of_fp32_attention(vb, q_lens, kv_lens, hq, hkv, dk, dv):
    """dq, dk, dv of the packed call (reference kernels: triton_invariant_attention.py:194-431; reference tests:
    test_triton_attention_varlen.py:75-150, :254-335) against torch autograd on fp32 eager attention.  bf16 inputs and
    bf16 roundings of p and ds inside: the reference's own bf16 tolerance, 3e-2 of each gradient's largest
    magnitude, and cosine similarity > 0.999.  A sequence's gradients are the same bits alone and in the batch."""
    g = torch.Generator().manual_seed(77)
    q = torch.randn(sum(q_lens), hq, dk, generator=g).to(BF).cuda()
    k = torch.randn(sum(kv_lens), hkv, dk, generator=g).to(BF).cuda()
    v = torch.randn(sum(kv_lens), hkv, dv, generator=g).to(BF).cuda()
    dout = torch.randn(sum(q_lens), hq, dv, generator=g).to(BF).cuda()
    cu_q = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32).cuda()
    cu_k = torch.tensor([0] + torch.tensor(kv_lens).cumsum(0).tolist(), dtype=torch.int32).cuda()
    scale = dk ** -0.5

    def run(q, k, v, dout, cu_q, cu_k, mq, mk):
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
        out, _ = vb.flash_attn_varlen_func(*leaves, cu_q, cu_k, max_seqlen_q=mq, max_seqlen_k=mk, softmax_scale=scale,
                                           causal=True)
        out.backward(dout)
        return [t.grad for t in leaves]

    got = run(q, k, v, dout, cu_q, cu_k, max(q_lens), max(kv_lens))
    ref_leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v)]
    qo = ko = 0
    outs = []
    for ql, kl in zip(q_lens, kv_lens):
        outs.append(_eager_packed(ref_leaves[0][qo:qo + ql], ref_leaves[1][ko:ko + kl], ref_leaves[2][ko:ko + kl], scale))
        qo, ko = qo + ql, ko + kl
    torch.cat(outs).backward(dout.float())
    for name, a, b in zip("qkv", got, ref_leaves):
        want = b.grad
        assert a.shape == want.shape and a.dtype == BF
        torch.testing.assert_close(a.float(), want, rtol=0, atol=3e-2 * want.abs().max().item(),
                                   msg=lambda m, name=name: f"d{name}: {m}")
        cos = torch.nn.functional.cosine_similarity(a.float().flatten(), want.flatten(), dim=0).item()
        assert cos > 0.999, (name, cos)
    # sequence 1 alone: the same bits
    a, b = q_lens[0], kv_lens[0]
    alone = run(q[a:], k[b:], v[b:], dout[a:], torch.tensor([0, q_lens[1]], dtype=torch.int32).cuda(),
                torch.tensor([0, kv_lens[1]], dtype=torch.int32).cuda(), q_lens[1], kv_lens[1])
    assert torch.equal(alone[0], got[0][a:]) and torch.equal(alone[1], got[1][b:]) and torch.equal(alone[2], got[2][b:])
    torch.cuda.synchronize()
    assert vb._lib.read_status()[0] == 0


def test_packed_varlen_backward_tensor_core_and_cuda_core_forms_agree(vb, tmp_path):
    """The default backward runs on the tensor cores (mma.sync); B200_ATTN_BWD_SIMT=1 selects the CUDA-core kernels
    (read once per process, hence the child process).  Same rounding points, different summation order inside a
    16-wide step: the two agree to 2^-6 of each gradient's largest magnitude."""
    import subprocess
    import sys

    script = """
import sys, torch
import vexact_b200 as vb
BF = torch.bfloat16
g = torch.Generator().manual_seed(5)
q_lens, kv_lens, hq, hkv, d = [70, 33], [100, 33], 4, 2, 128
q = torch.randn(sum(q_lens), hq, d, generator=g).to(BF).cuda().requires_grad_(True)
k = torch.randn(sum(kv_lens), hkv, d, generator=g).to(BF).cuda().requires_grad_(True)
v = torch.randn(sum(kv_lens), hkv, d, generator=g).to(BF).cuda().requires_grad_(True)
dout = torch.randn(sum(q_lens), hq, d, generator=g).to(BF).cuda()
cu_q = torch.tensor([0, 70, 103], dtype=torch.int32).cuda()
cu_k = torch.tensor([0, 100, 133], dtype=torch.int32).cuda()
out, _ = vb.flash_attn_varlen_func(q, k, v, cu_q, cu_k, max_seqlen_q=70, max_seqlen_k=100, causal=True)
out.backward(dout)
torch.cuda.synchronize()
assert vb._lib.read_status()[0] == 0
torch.save([q.grad.cpu(), k.grad.cpu(), v.grad.cpu()], sys.argv[1])
"""
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    grads = {}
    for form, knob in (("mma", "0"), ("simt", "1")):
        path = str(tmp_path / f"{form}.pt")
        env = dict(os.environ, B200_ATTN_BWD_SIMT=knob, PYTHONPATH=root)
        subprocess.run([sys.executable, "-c", script, path], check=True, env=env, cwd=root, timeout=180)
        grads[form] = torch.load(path)
    for a, b in zip(grads["mma"], grads["simt"]):
        torch.testing.assert_close(a.float(), b.float(), rtol=0, atol=2 ** -6 * b.float().abs().max().item())
