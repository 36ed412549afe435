"""GPU parity: MoE routing (bit-exact expert selection), permutation indices (bit-exact),
grouped GEMM + fused SwiGLU vs the CPU oracle, and batch invariance
(reference: tests/batch_invariant_ops/test_fused_moe.py:75-133, test_naive_moe.py:114-136)."""
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


def _seeded(*shape, seed=0, std=1.0, dtype=BF):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def test_route_softmax_topk_exact_indices(vb):
    for c in load_golden("route_softmax_topk"):
        w_ref, idx_ref = ops.route_softmax_topk(c["logits"], c["top_k"], True)
        w, idx = vb.route_softmax_topk(c["logits"].cuda(), c["top_k"], True)
        assert torch.equal(idx.cpu(), idx_ref)          # same tie rule as the oracle: bit-exact
        torch.testing.assert_close(w.cpu().float(), w_ref.float(), rtol=2 ** -7, atol=1e-6)
        # and against the reference's torch.topk wherever the boundary is not a tie
        probs = torch.softmax(c["logits"].float(), 1)
        srt = torch.sort(probs, descending=True).values
        distinct = (srt[:, : c["top_k"] + 1].diff(dim=1) != 0).all(dim=1)
        assert torch.equal(idx.cpu()[distinct], c["experts"][distinct])
    logits = _seeded(512, 128, seed=1, std=0.9)
    w_ref, idx_ref = ops.route_softmax_topk(logits, 8, True)
    w, idx = vb.route_softmax_topk(logits.cuda(), 8, True)
    # fp32 softmax sums may differ in the last bit between device and host; a flip needs two
    # probabilities within one fp32 ulp, so report rather than hide: require >= 99.9 % exact rows
    same = (idx.cpu() == idx_ref).all(dim=1).float().mean().item()
    assert same >= 0.999, f"expert selection differs from the oracle on {1 - same:.4%} of tokens"
    w1, idx1 = vb.route_softmax_topk(logits[:1].cuda(), 8, True)
    assert torch.equal(idx1, idx[:1]) and torch.equal(w1, w[:1])


def test_route_sigmoid_group_topk(vb):
    for c in load_golden("route_sigmoid_group_topk"):
        idx_ref, w_ref = ops.route_sigmoid_group_topk(c["logits"], c["bias"], c["n_group"], c["topk_group"],
                                                      c["top_k"], True, c["scale"])
        idx, w = vb.route_sigmoid_group_topk(c["logits"].cuda(), c["bias"].cuda(), c["n_group"], c["topk_group"],
                                             c["top_k"], True, c["scale"])
        assert torch.equal(idx.cpu(), idx_ref)
        torch.testing.assert_close(w.cpu(), w_ref, rtol=1e-5, atol=1e-6)
        assert torch.equal(torch.sort(idx.cpu(), 1).values, torch.sort(c["experts"], 1).values)


@pytest.mark.parametrize("T,k,E", [(12, 4, 8), (512, 8, 128), (2048, 8, 128), (256, 6, 64), (1, 8, 128), (3000, 2, 5)])
def test_moe_indices_bit_exact(vb, T, k, E):
    from vexact_b200.fused_moe import build_moe_indices

    g = torch.Generator().manual_seed(2)
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    cu_ref, a_ref, sc_ref = ops.build_moe_indices(sel, E)
    cu, a_idx, sc = build_moe_indices(sel.cuda(), E)
    assert (cu.cpu().numpy() == cu_ref).all()
    assert (sc.cpu().numpy() == sc_ref).all()
    assert (a_idx.cpu().numpy() == a_ref).all()
    cu32, _, sc32 = build_moe_indices(sel.int().cuda(), E)
    assert torch.equal(cu32, cu) and torch.equal(sc32, sc)


def test_moe_indices_golden(vb):
    from vexact_b200.fused_moe import build_moe_indices

    c = load_golden("moe_indices")
    cu, a_idx, sc = build_moe_indices(c["experts"].cuda(), c["num_experts"])
    assert torch.equal(cu.cpu(), c["cu_seqlens"]) and torch.equal(a_idx.cpu(), c["a_idx"])
    assert torch.equal(sc.cpu(), c["scatter_index"])


def _moe_case(T, E, k, H, I, seed, skew=False):
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(T, H, generator=g).to(BF)
    gate_up = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(BF)
    down = (torch.randn(E, H, I, generator=g) * 0.05).to(BF)
    if skew:
        sel = torch.stack([torch.cat([torch.zeros(1, dtype=torch.long), 1 + torch.randperm(E - 1, generator=g)[:k - 1]])
                           for _ in range(T)])
    else:
        sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    rw = torch.rand(T, k, generator=g)
    rw = (rw / rw.sum(-1, keepdim=True)).to(BF)
    return hidden, gate_up, down, sel, rw


@pytest.mark.parametrize("T,E,k,H,I,skew", [(12, 8, 4, 64, 32, False), (64, 16, 4, 256, 128, False),
                                            (300, 8, 2, 512, 192, True), (40, 128, 8, 2048, 768, False)])
def test_fused_moe_oracle(vb, T, E, k, H, I, skew):
    hidden, gate_up, down, sel, rw = _moe_case(T, E, k, H, I, seed=3, skew=skew)
    ref = ops.fused_moe_batched(E, rw, sel, hidden, gate_up[:, :I], gate_up[:, I:], down)
    out = vb.fused_moe_forward(E, rw.cuda(), sel.cuda(), hidden.cuda(), fc2_weight=down.cuda(),
                               fc1_1_2_weight=gate_up.cuda())
    # Each of the k expert rows summed into a token is a bf16 tensor, and a one-ulp flip of an
    # intermediate (device expf / accumulation order) moves a row by one bf16 ulp of the ROW's
    # magnitude, which can exceed an ulp of a sum that cancels.  Stated tolerance: 2^-6 of the
    # largest output magnitude, absolute; and at least 95 % of elements bit-identical.
    tol = 2 ** -6 * max(ref.float().abs().max().item(), 1e-3)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=0, atol=tol)
    assert (out.cpu() == ref).float().mean() > 0.95
    # split gate / up weights (the reference's positional signature) give the same bits
    out_split = vb.fused_moe_forward(E, rw.cuda(), sel.cuda(), hidden.cuda(), gate_up[:, :I].contiguous().cuda(),
                                     gate_up[:, I:].contiguous().cuda(), down.cuda())
    assert torch.equal(out_split, out)


def test_fused_moe_golden_naive(vb):
    c = load_golden("moe_naive")
    E = c["gate_up"].shape[0]
    out = vb.fused_moe_forward(E, c["weights"].cuda(), c["experts"].cuda(), c["hidden"].cuda(),
                               fc2_weight=c["down"].cuda(), fc1_1_2_weight=c["gate_up"].cuda())
    err = (out.cpu().float() - c["out_fp32"]).abs().max().item()
    assert err < 2e-3 * max(1.0, c["out_fp32"].abs().max().item())


def test_fused_moe_batch_invariance_bitwise(vb):
    """Full batch vs token by token: identical bits (the reference allows 1e-3 here)."""
    T, E, k, H, I = 96, 32, 4, 512, 256
    hidden, gate_up, down, sel, rw = _moe_case(T, E, k, H, I, seed=4)
    args = (down.cuda(), gate_up.cuda())
    full = vb.fused_moe_forward(E, rw.cuda(), sel.cuda(), hidden.cuda(), fc2_weight=args[0], fc1_1_2_weight=args[1])
    for t in (0, 1, 17, 95):
        one = vb.fused_moe_forward(E, rw[t:t + 1].cuda(), sel[t:t + 1].cuda(), hidden[t:t + 1].cuda(),
                                   fc2_weight=args[0], fc1_1_2_weight=args[1])
        assert torch.equal(one, full[t:t + 1]), f"token {t} differs between batch {T} and batch 1"
    half = vb.fused_moe_forward(E, rw[:40].cuda(), sel[:40].cuda(), hidden[:40].cuda(), fc2_weight=args[0],
                                fc1_1_2_weight=args[1])
    assert torch.equal(half, full[:40])


def test_status_word_clean(vb):
    torch.cuda.synchronize()
    assert vb._lib.read_status()[0] == 0


def test_deferred_topk_sum_fused_with_add_rmsnorm_bitwise(vb):
    """PendingMoE.add_norm == finish() followed by add_rms_norm, bit for bit (with and without addend)."""
    for H in (2048, 512):      # one-CTA-per-row norm (fused kernel) and the short-row fallback
        _check_deferred_sum(vb, H)


def _check_deferred_sum(vb, H):
    g = torch.Generator().manual_seed(5)
    T, E, k, I = 96, 16, 4, 256
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16().cuda()
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16().cuda()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16().cuda()
    logits = torch.randn(T, E, generator=g).bfloat16().cuda()
    rw, sel = vb.route_softmax_topk(logits, k, True)
    residual = torch.randn(T, H, generator=g).bfloat16().cuda()
    norm_w = (1 + 0.02 * torch.randn(H, generator=g)).bfloat16().cuda()
    for addend in (None, (torch.randn(T, H, generator=g) * 0.3).bfloat16().cuda()):
        for hf in (True, False):
            plain = vb.fused_moe_forward(E, rw, sel, x, fc2_weight=w2, fc1_1_2_weight=w13, addend=addend)
            want_sum, want_norm = vb.add_rms_norm(plain, residual, norm_w, 1e-6, hf=hf)
            pend = vb.fused_moe_forward(E, rw, sel, x, fc2_weight=w2, fc1_1_2_weight=w13, addend=addend,
                                        defer_reduce=True)
            got_sum, got_norm = pend.add_norm(residual, norm_w, 1e-6, hf=hf)
            assert torch.equal(got_sum, want_sum) and torch.equal(got_norm, want_norm)
            assert torch.equal(pend.finish(), plain)


def test_fc1_routes_agree_bitwise(vb):
    """fc1 with the fused SwiGLU epilogue (few rows per expert) and as plain grouped GEMM + elementwise
    kernel (many rows per expert): the same token gets the same bits."""
    g = torch.Generator().manual_seed(31)
    T, E, k, H, I = 600, 8, 2, 256, 128          # 150 rows per expert: split route
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16().cuda()
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16().cuda()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16().cuda()
    logits = torch.randn(T, E, generator=g).bfloat16().cuda()
    rw, sel = vb.route_softmax_topk(logits, k, True)
    big = vb.fused_moe_forward(E, rw, sel, x, fc2_weight=w2, fc1_1_2_weight=w13)
    small = vb.fused_moe_forward(E, rw[:100], sel[:100], x[:100], fc2_weight=w2, fc1_1_2_weight=w13)   # 25 per expert: fused
    assert torch.equal(big[:100], small)


@pytest.mark.parametrize("T,E,k,H,I,skew", [(1, 8, 2, 64, 32, False), (7, 16, 4, 256, 128, False),
                                            (300, 8, 2, 512, 192, True), (512, 128, 8, 2048, 768, False),
                                            (600, 8, 2, 256, 128, False)])
def test_fc1_gathering_its_rows_equals_the_permuted_copy_bitwise(vb, monkeypatch, T, E, k, H, I, skew):
    """fc1 reading x[gather_index[r]] (one-row TMA boxes, four rows per gather) against fc1 over the
    expert-sorted copy of x: the same bytes land in the same shared-memory rows, so every output bit agrees;
    with fused and with split fc1 weights, and from a strided view of the activations."""
    hidden, gate_up, down, sel, rw = _moe_case(T, E, k, H, I, seed=11, skew=skew)
    args = (E, rw.cuda(), sel.cuda())
    wide = torch.zeros(T, H + 64, dtype=BF, device="cuda")
    wide[:, :H] = hidden.cuda()
    outs = {}
    for mode in ("0", "1"):
        monkeypatch.setenv("B200_MOE_GATHER", mode)
        outs[mode] = (
            vb.fused_moe_forward(*args, hidden.cuda(), fc2_weight=down.cuda(), fc1_1_2_weight=gate_up.cuda()),
            vb.fused_moe_forward(*args, hidden.cuda(), gate_up[:, :I].contiguous().cuda(),
                                 gate_up[:, I:].contiguous().cuda(), down.cuda()),
            vb.fused_moe_forward(*args, wide[:, :H], fc2_weight=down.cuda(), fc1_1_2_weight=gate_up.cuda()),
        )
    for a, b in zip(outs["0"], outs["1"]):
        assert torch.equal(a, b)
    assert torch.equal(outs["1"][0], outs["1"][2])


@pytest.mark.parametrize("T,E,k,H,I,skew", [(1, 8, 2, 64, 32, False), (40, 128, 8, 2048, 768, False),
                                            (512, 128, 8, 2048, 768, False), (300, 8, 2, 512, 192, True)])
def test_routing_with_its_plan_equals_route_index_scatter_bitwise(vb, T, E, k, H, I, skew):
    """Routing that hands out the permutation itself (two launches) against route -> index -> scatter (three):
    same routing weights and experts, cu_seqlens and tile table; the rows of an expert's group may sit in another
    order, and every output of the MoE is the same bits.  Twice in a row: the counters come back clean."""
    from vexact_b200.fused_moe import _PLAN_COUNTERS, _permute, route_plan_softmax_topk

    hidden, gate_up, down, _, _ = _moe_case(T, E, k, H, I, seed=21, skew=skew)
    g = torch.Generator().manual_seed(4)
    logits = (torch.randn(T, E, generator=g) * (3.0 if skew else 1.0)).to(BF).cuda()
    x, gu, dn = hidden.cuda(), gate_up.cuda(), down.cuda()
    rw0, sel0 = vb.route_softmax_topk(logits, k, True)
    want = vb.fused_moe_forward(E, rw0, sel0, x, fc2_weight=dn, fc1_1_2_weight=gu)
    classic = _permute(sel0, rw0, None, E)
    for _ in range(2):
        rw, sel, plan = route_plan_softmax_topk(logits, k, True, E)
        assert torch.equal(rw, rw0) and torch.equal(sel, sel0)
        assert torch.equal(plan["cu_seqlens"], classic["cu_seqlens"])
        assert torch.equal(plan["tile_count"], classic["tile_count"])
        nt = int(plan["tile_count"])
        assert torch.equal(plan["tile_table"][:nt], classic["tile_table"][:nt])
        # ranks: within every expert exactly 0 .. count-1
        cnt = torch.bincount(sel.flatten(), minlength=E)
        for e in range(E):
            r = plan["rank"][(sel.flatten() == e)].sort().values
            assert torch.equal(r, torch.arange(int(cnt[e]), device="cuda", dtype=torch.int32))
        got = vb.fused_moe_forward(E, rw, sel, x, fc2_weight=dn, fc1_1_2_weight=gu, plan=plan)
        assert torch.equal(got, want)
        torch.cuda.synchronize()
        assert int(_PLAN_COUNTERS[torch.cuda.current_device()].abs().sum()) == 0


def test_gather_index_is_the_inverse_of_scatter_index(vb):
    from vexact_b200.fused_moe import _permute

    g = torch.Generator().manual_seed(5)
    T, k, E = 333, 6, 64
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).cuda()
    rw = torch.rand(T, k, generator=g).bfloat16().cuda()
    plan = _permute(sel, rw, None, E, gather=True)
    scatter = plan["scatter_index"].long()
    n = T * k
    assert torch.equal(scatter.sort().values, torch.arange(n, device="cuda"))
    want = torch.empty(n, dtype=torch.int32, device="cuda")
    want[scatter] = (torch.arange(n, device="cuda") // k).int()
    assert torch.equal(plan["gather_index"], want)
    scale = torch.empty(n, dtype=BF, device="cuda")
    scale[scatter] = rw.flatten()
    assert torch.equal(plan["row_scale"], scale)
    # within an expert the rows keep token order (stable sort), as the reference's argsort(stable=True) gives
    cu = plan["cu_seqlens"].tolist()
    gi = plan["gather_index"].tolist()
    assert all(gi[a:b] == sorted(gi[a:b]) for a, b in zip(cu[:-1], cu[1:]))


@pytest.mark.gpu
def test_routing_of_nan_rows_stays_in_range():
    """Padded tokens of a captured batch carry undefined (possibly NaN) hidden states; their routing must
    still name experts inside [0, E) so that nothing downstream indexes out of range."""
    import vexact_b200 as vb

    E, k = 64, 6
    logits = torch.randn(5, E, device="cuda")
    logits[1] = float("nan")
    logits[3, 7] = float("nan")
    _, sel = vb.route_softmax_topk(logits, k, True)
    assert int(sel.min()) >= 0 and int(sel.max()) < E
    idx, _ = vb.route_sigmoid_group_topk(logits, torch.zeros(E, device="cuda"), 4, 2, k, True, 2.5)
    assert int(idx.min()) >= 0 and int(idx.max()) < E
    # rows without NaN are untouched by the guard
    clean = logits[[0, 2, 4]].contiguous()
    _, sel_c = vb.route_softmax_topk(clean, k, True)
    assert torch.equal(sel_c, sel[[0, 2, 4]])
    torch.cuda.synchronize()
    assert vb._lib.read_status()[0] == 0


def test_group_gemm_operators_under_the_reference_names(vb):
    """`expert_histogram`, `moe_scatter`, `group_gemm_same_nk`, `moe_gather` (reference group_gemm/kernel/moe.py:52,
    :304, :131; group_gemm.py:156) one at a time, chained as FusedMoeExpertFunction.forward chains them
    (fused_moe.py:24-111): index and copy steps bit-exact, the GEMM equal to the dense GEMM's bits per expert,
    the chain equal to `fused_moe_forward` up to the activation's rounding."""
    from vexact_b200 import group_gemm as gg

    T, E, k, H, I = 70, 16, 4, 256, 128
    hidden, gate_up, down, sel, rw = _moe_case(T, E, k, H, I, seed=11)
    x, sel_d, rw_d = hidden.cuda(), sel.cuda(), rw.cuda()
    w1, w2, w3 = gate_up[:, :I].contiguous().cuda(), gate_up[:, I:].contiguous().cuda(), down.cuda()

    splits = gg.expert_histogram(sel_d, E)
    assert splits.dtype == torch.int32
    assert torch.equal(splits.cpu().long(), torch.bincount(sel.flatten(), minlength=E))
    assert torch.equal(gg.expert_histogram(sel_d.int(), E), splits)

    scatter_index = sel_d.flatten().argsort(stable=True).argsort().int().view(sel_d.shape)   # fused_moe.py:43
    cu, a_idx, scatter_ours = vb.fused_moe.build_moe_indices(sel_d, E)
    assert torch.equal(scatter_ours, scatter_index)

    rows = gg.moe_index_compute(sel_d, torch.cumsum(splits, dim=0))     # moe.py:382: any order inside an expert;
    assert rows.dtype == torch.int64 and torch.equal(rows, scatter_index.long())   # here the stable one

    scattered = gg.moe_scatter(x, scatter_index)
    assert torch.equal(scattered, x[a_idx.long()])
    assert torch.equal(gg.moe_scatter(x.half(), scatter_index.long()), x.half()[a_idx.long()])   # fp16 rows, int64 index

    cumsum_t = torch.cumsum(splits, dim=0)
    fc1_1 = gg.group_gemm_same_nk(a=scattered, b=w1, cumsum_M=cumsum_t, max_M=scattered.shape[0], transpose_b=True)
    fc1_2 = gg.group_gemm_same_nk(a=scattered, b=w2, cumsum_M=cumsum_t, max_M=scattered.shape[0], transpose_b=True)
    bounds = [0] + cumsum_t.tolist()
    for e in range(E):          # a token's dot products do not depend on the tile it sits in: the dense GEMM's bits
        lo, hi = bounds[e], bounds[e + 1]
        if hi > lo:
            assert torch.equal(fc1_1[lo:hi], vb.matmul_persistent(scattered[lo:hi], w1[e].t()))
    ref32 = torch.cat([scattered[bounds[e]:bounds[e + 1]].float() @ w2[e].float().t() for e in range(E)])
    torch.testing.assert_close(fc1_2.float(), ref32, rtol=2 ** -7, atol=2 ** -7 * ref32.abs().max().item())

    gate_w = torch.empty(T * k, 1, dtype=BF, device="cuda")
    gate_w[scatter_index.flatten().long()] = rw_d.reshape(-1, 1)                               # fused_moe.py:84-86
    weighted = torch.ops.aten.silu(fc1_1) * fc1_2 * gate_w
    fc2 = gg.group_gemm_same_nk(a=weighted, b=w3, cumsum_M=cumsum_t, max_M=weighted.shape[0], transpose_b=True)

    out = gg.moe_gather(fc2, scatter_index)
    acc = torch.zeros(T, H, device="cuda")
    for j in range(k):                                   # fp32 sum in k order, one rounding (moe.py:113-127)
        acc += fc2[scatter_index[:, j].long()].float()
    assert torch.equal(out, acc.to(BF))

    fused = vb.fused_moe_forward(E, rw_d, sel_d, x, w1, w2, w3)
    tol = 2 ** -6 * max(fused.float().abs().max().item(), 1e-3)
    torch.testing.assert_close(out.float(), fused.float(), rtol=0, atol=tol)
    assert (out == fused).float().mean() > 0.95

    # the two GEMM forms of the backward (group_gemm.py:156 with transpose_b=False, :360 group_gemm_same_mn)
    dgrad = gg.group_gemm_same_nk(fc1_1, w1, cumsum_t, T * k, transpose_b=False)        # [R, I] x [E, I, H] -> [R, H]
    assert torch.equal(dgrad, gg.group_gemm_same_nk(fc1_1, w1.transpose(1, 2).contiguous(), cumsum_t, T * k,
                                                    transpose_b=True))
    ref32 = torch.cat([fc1_1[bounds[e]:bounds[e + 1]].float() @ w1[e].float() for e in range(E)])
    torch.testing.assert_close(dgrad.float(), ref32, rtol=2 ** -7, atol=2 ** -7 * ref32.abs().max().item())
    wgrad = gg.group_gemm_same_mn(fc1_1, scattered, torch.full_like(w1, 7.0), cumsum_t, T * k, transpose_a=True,
                                  transpose_b=False)                                  # [E, I, H]
    ref32 = torch.stack([fc1_1[bounds[e]:bounds[e + 1]].float().t() @ scattered[bounds[e]:bounds[e + 1]].float()
                         for e in range(E)])
    torch.testing.assert_close(wgrad.float(), ref32, rtol=2 ** -7, atol=2 ** -8 * ref32.abs().max().item())
    lonely = torch.cumsum(torch.tensor([3, 0, T * k - 3] + [0] * (E - 3), device="cuda"), 0)   # empty groups: zeros
    wz = gg.group_gemm_same_mn(fc1_1, scattered, torch.full_like(w1, 7.0), lonely, T * k, transpose_a=True,
                               transpose_b=False)
    assert not wz[1].any() and not wz[3:].any() and wz[0].any() and wz[2].any()
    torch.cuda.synchronize()
    assert vb._lib.read_status()[0] == 0
    overrun = lonely.clone()
    overrun[-1] = T * k + 9                                  # past the last row: clipped and reported
    wo = gg.group_gemm_same_mn(fc1_1, scattered, torch.full_like(w1, 7.0), overrun, T * k, transpose_a=True,
                               transpose_b=False)
    torch.cuda.synchronize()
    assert vb._lib.read_status()[:2] == (2, E - 1)
    assert torch.equal(wo[2], wz[2]) and not wo[E - 1].any()

    for call in (lambda: gg.group_gemm_same_mn(scattered, scattered, w1, cumsum_t, T * k),
                 lambda: gg.moe_add_gather(fc2, fc2, scatter_index)):
        with pytest.raises(NotImplementedError):
            call()


def test_scatter_and_gather_skip_and_report_an_index_out_of_range(vb):
    from vexact_b200 import group_gemm as gg

    T, k, H = 6, 2, 64
    x = _seeded(T, H, seed=2).cuda()
    index = torch.randperm(T * k, generator=torch.Generator().manual_seed(3)).int().view(T, k).cuda()
    good = gg.moe_scatter(x, index)
    torch.cuda.synchronize()
    assert vb._lib.read_status()[0] == 0
    bad = index.clone()
    bad[4, 1] = T * k + 5
    gg.moe_scatter(x, bad)
    torch.cuda.synchronize()
    code, detail, _, _ = vb._lib.read_status()
    assert (code, detail) == (2, 4 * k + 1)
    rows = _seeded(T * k, H, seed=4).cuda()
    bad[4, 1] = -3
    out = gg.moe_gather(rows, bad)
    torch.cuda.synchronize()
    code, detail, _, _ = vb._lib.read_status()
    assert (code, detail) == (2, 4 * k + 1)
    assert torch.equal(out[4], rows[bad[4, 0].long()])          # the bad term contributes nothing
    assert torch.equal(out[:4], gg.moe_gather(rows, index)[:4])
    assert vb._lib.read_status()[0] == 0
    assert good.shape == (T * k, H)


def test_expert_function_classes_take_the_reference_arguments(vb):
    """`FusedMoeExpertFunction.apply` / `QuackFusedMoeExpertFunction.apply` (fused_moe.py:22, :295) with the
    reference's seven positional arguments: the fused forward's bits."""
    from vexact_b200.fused_moe import FusedMoeExpertFunction, QuackFusedMoeExpertFunction

    T, E, k, H, I = 33, 8, 2, 128, 64
    hidden, gate_up, down, sel, rw = _moe_case(T, E, k, H, I, seed=21)
    args = (E, rw.cuda(), sel.cuda(), hidden.cuda(), gate_up[:, :I].contiguous().cuda(),
            gate_up[:, I:].contiguous().cuda(), down.cuda())
    fused = vb.fused_moe_forward(*args)
    assert torch.equal(FusedMoeExpertFunction.apply(*args), fused)
    assert torch.equal(QuackFusedMoeExpertFunction.apply(*args), fused)


@pytest.mark.parametrize("fused_weights", [False, True])
def test_fused_moe_backward_against_autograd_of_the_fp32_formula(vb, fused_weights):
    """Gradients of `fused_moe_forward` (reference backward: fused_moe.py:113-265) for the hidden states, the routing
    weights and the three weight tensors, against torch autograd on the fp32 statement of the same function
    (sum over k of w_k * fc2_e(silu(fc1_1_e x) * fc1_2_e x)).  The chain rounds to bf16 after every step, as the
    reference's does: stated tolerance 2^-5 of each gradient's largest magnitude, and cosine similarity > 0.999.
    One expert is never selected: its weight gradients are exact zeros."""
    T, E, k, H, I = 48, 8, 2, 128, 64
    hidden, gate_up, down, sel, rw = _moe_case(T, E, k, H, I, seed=31)
    sel = torch.where(sel == E - 1, torch.zeros_like(sel), sel)          # expert E-1 unused
    dup = sel[:, 0] == sel[:, 1]
    sel[dup, 1] = (sel[dup, 0] + 1) % (E - 1)
    g_out = _seeded(T, H, seed=32)
    leaves = dict(x=hidden.cuda(), rw=rw.cuda(), w1=gate_up[:, :I].contiguous().cuda(),
                  w2=gate_up[:, I:].contiguous().cuda(), w3=down.cuda())
    ours = {n: t.clone().requires_grad_(True) for n, t in leaves.items()}
    if fused_weights:       # the model files' keyword form: one [E, 2I, H] tensor, gate rows first
        gu = torch.cat([ours["w1"], ours["w2"]], dim=1)
        out = vb.fused_moe_forward(E, ours["rw"], sel.cuda(), ours["x"], fc2_weight=ours["w3"], fc1_1_2_weight=gu)
    else:
        out = vb.fused_moe_forward(E, ours["rw"], sel.cuda(), ours["x"], ours["w1"], ours["w2"], ours["w3"])
    assert torch.equal(out, vb.fused_moe_forward(E, leaves["rw"], sel.cuda(), leaves["x"], leaves["w1"], leaves["w2"],
                                                 leaves["w3"]))
    out.backward(g_out.cuda())

    ref = {n: t.float().clone().requires_grad_(True) for n, t in leaves.items()}
    s = sel.cuda()
    acc = torch.zeros(T, H, device="cuda")
    for j in range(k):
        e = s[:, j]
        a = torch.einsum("th,tih->ti", ref["x"], ref["w1"][e])
        b = torch.einsum("th,tih->ti", ref["x"], ref["w2"][e])
        acc = acc + torch.einsum("ti,thi->th", torch.nn.functional.silu(a) * b * ref["rw"][:, j:j + 1], ref["w3"][e])
    acc.backward(g_out.cuda().float())
    for n in leaves:
        got, want = ours[n].grad.float(), ref[n].grad
        assert got.shape == want.shape and ours[n].grad.dtype == leaves[n].dtype
        tol = 2 ** -5 * want.abs().max().item()
        torch.testing.assert_close(got, want, rtol=0, atol=tol, msg=lambda m, n=n: f"grad of {n}: {m}")
        cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
        assert cos > 0.999, (n, cos)
    for n in ("w1", "w2", "w3"):
        assert not ours[n].grad[E - 1].any()




def test_weight_gradient_kernels_tensor_core_and_cuda_core_forms(vb):
    """`group_gemm_same_mn` runs on the tensor cores when M and N are multiples of 8 and on the CUDA cores
    otherwise; both against the fp32 product, with ragged and empty groups and tiles that overhang M and N."""
    from vexact_b200 import group_gemm as gg

    g = torch.Generator().manual_seed(41)
    counts = [0, 37, 1, 200, 0, 16, 90]
    R, G = sum(counts), len(counts)
    cs = torch.cumsum(torch.tensor(counts), 0).cuda()
    bounds = [0] + cs.tolist()
    for M, N in [(200, 136), (128, 256), (36, 20)]:
        a = torch.randn(R, M, generator=g).to(BF).cuda()
        b = torch.randn(R, N, generator=g).to(BF).cuda()
        c = gg.group_gemm_same_mn(a, b, torch.full((G, M, N), 7.0, dtype=BF, device="cuda"), cs, R, transpose_a=True,
                                  transpose_b=False)
        ref = torch.stack([a[bounds[e]:bounds[e + 1]].float().t() @ b[bounds[e]:bounds[e + 1]].float() for e in range(G)])
        torch.testing.assert_close(c.float(), ref, rtol=2 ** -7, atol=2 ** -8 * ref.abs().max().item())
        assert not c[0].any() and not c[4].any()
    torch.cuda.synchronize()
    assert vb._lib.read_status()[0] == 0
