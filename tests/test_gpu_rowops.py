"""GPU parity: RMSNorm, mean, log_softmax, gather-logprob, KV store, q/k-norm + RoPE + store.
CUDA path (through the C ABI) vs the CPU oracle and the reference's golden fixtures."""
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


def _seeded(*shape, seed=0, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def test_rmsnorm_golden_and_oracle(vb):
    for c in load_golden("rms_norm_single"):
        out = vb.batch_invariant_rms_norm(c["x"].cuda(), c["w"].cuda(), c["eps"]).cpu()
        # fp32 sum order differs from the reference kernel: at most one bf16 ulp, nearly always equal
        torch.testing.assert_close(out.float(), c["out"].float(), rtol=2 ** -7, atol=1e-6)
        assert (out == c["out"]).float().mean() > 0.995
    for c in load_golden("rms_norm_hf"):
        out = vb.hf_rms_norm(c["x"].cuda(), c["w"].cuda(), c["eps"]).cpu()
        torch.testing.assert_close(out.float(), c["out"].float(), rtol=2 ** -7, atol=1e-6)
        assert (out == c["out"]).float().mean() > 0.995


@pytest.mark.parametrize("n", [2048, 128, 512, 1000, 1536, 7168])
@pytest.mark.parametrize("mode", ["single", "hf"])
def test_rmsnorm_oracle_and_row_invariance(vb, n, mode):
    x = _seeded(257, n, seed=1, dtype=BF)
    w = (1 + 0.02 * _seeded(n, seed=2)).to(BF)
    fn = vb.batch_invariant_rms_norm if mode == "single" else vb.hf_rms_norm
    ref = (ops.rms_norm_single_round if mode == "single" else ops.rms_norm_hf)(x, w, 1e-6)
    full = fn(x.cuda(), w.cuda(), 1e-6)
    torch.testing.assert_close(full.cpu().float(), ref.float(), rtol=2 ** -7, atol=1e-6)
    assert (full.cpu() == ref).float().mean() > 0.995
    for m in (1, 7, 64):
        part = fn(x[:m].cuda(), w.cuda(), 1e-6)
        assert torch.equal(part, full[:m]), f"row results depend on the batch size (M={m})"
    # strided input rows (a column slice of a wider tensor)
    wide = _seeded(9, 2 * n, seed=3, dtype=BF).cuda()
    assert torch.equal(fn(wide[:, :n], w.cuda(), 1e-6), fn(wide[:, :n].contiguous(), w.cuda(), 1e-6))


def test_add_rmsnorm_matches_separate_ops(vb):
    x = _seeded(33, 2048, seed=4, dtype=BF).cuda()
    r = _seeded(33, 2048, seed=5, dtype=BF).cuda()
    w = (1 + 0.02 * _seeded(2048, seed=6)).to(BF).cuda()
    s, y = vb.add_rms_norm(x, r, w, 1e-6, hf=True)
    assert torch.equal(s, r + x)
    assert torch.equal(y, vb.hf_rms_norm(r + x, w, 1e-6))


def test_mean_lastdim(vb):
    for c in load_golden("mean_lastdim"):
        out = vb.mean_dim(c["x"].cuda(), -1).cpu()
        torch.testing.assert_close(out, c["out"], rtol=0, atol=3e-7)
    x = _seeded(50, 4, 2048, seed=7).cuda()
    full = vb.mean_dim(x, -1, keepdim=True)
    assert full.shape == (50, 4, 1)
    assert torch.equal(vb.mean_dim(x[:3], -1, keepdim=True), full[:3])
    torch.testing.assert_close(vb.mean_dim(x, 1).cpu(), x.cpu().mean(1), rtol=1e-6, atol=1e-6)
    # other float types accumulate in fp32 and round once, as the reference's kernel does for every dtype
    h = x.float().half()
    assert torch.equal(vb.mean_dim(h, -1), vb.mean_dim(h.float(), -1).half())
    with vb.set_batch_invariant_mode(True):
        under_mode = h.mean(-1)
        torch.use_deterministic_algorithms(False)
    assert torch.equal(under_mode, vb.mean_dim(h, -1))


def test_log_softmax_golden_and_invariance(vb):
    for c in load_golden("log_softmax"):
        out = vb.log_softmax(c["x"].cuda()).cpu()
        torch.testing.assert_close(out, c["out"], rtol=0, atol=6e-6)
    x = _seeded(64, 151936, seed=8, std=2.0).cuda()
    full = vb.log_softmax(x)
    perm = torch.randperm(64, generator=torch.Generator().manual_seed(0)).cuda()
    assert torch.equal(vb.log_softmax(x[perm].contiguous()), full[perm])
    assert torch.equal(vb.log_softmax(x[:1].contiguous()), full[:1])
    with pytest.raises(ValueError):
        vb.log_softmax(x, dim=0)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_gather_logprob(vb, dtype):
    V = 151936
    x = _seeded(48, V, seed=9, std=2.0).to(dtype)
    labels = torch.randint(0, V, (48,), generator=torch.Generator().manual_seed(1))
    ref = ops.gather_logprob(x, labels)
    xg, lg = x.cuda(), labels.cuda()
    out = vb.logprobs_from_logits_flash_attn(xg, lg)
    # stated tolerance for per-token logprob: 2e-5 absolute (fp32 sum order)
    torch.testing.assert_close(out.cpu(), ref, rtol=0, atol=2e-5)
    # permutation / batch-size invariance is bitwise (reference: test_batch_invariance.py:131-157)
    perm = torch.randperm(48, generator=torch.Generator().manual_seed(2)).cuda()
    assert torch.equal(vb.logprobs_from_logits_flash_attn(xg[perm].contiguous(), lg[perm]), out[perm])
    assert torch.equal(vb.logprobs_from_logits_flash_attn(xg[:1], lg[:1]), out[:1])
    lg2 = lg.clone()
    lg2[3] = -100
    assert vb.logprobs_from_logits_flash_attn(xg, lg2)[3].item() == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_greedy_token_and_logprob(vb, dtype):
    from vexact_b200.standalone_logprobs import greedy_token_and_logprob

    x = _seeded(40, 151936, seed=30, std=2.0).to(dtype)
    x[3, 100] = x[3, 70000] = x[3].max() + 1        # a tie: the lower index wins, as torch.argmax
    xg = x.cuda()
    tok, lp = greedy_token_and_logprob(xg)
    assert torch.equal(tok.cpu(), torch.argmax(x.float(), dim=-1)) and tok[3].item() == 100
    assert torch.equal(lp, vb.logprobs_from_logits_flash_attn(xg, tok))      # same bits as the two-kernel path
    torch.testing.assert_close(lp.cpu(), ops.gather_logprob(x, tok.cpu()), rtol=0, atol=2e-5)
    t1, l1 = greedy_token_and_logprob(xg[5:6])
    assert torch.equal(t1, tok[5:6]) and torch.equal(l1, lp[5:6])


def test_kv_store_golden_exact(vb):
    c = load_golden("kv_store")
    kc = torch.zeros_like(c["k_cache"]).cuda()
    vc = torch.zeros_like(c["v_cache"]).cuda()
    vb.store_kvcache(c["key"].cuda(), c["value"].cuda(), kc, vc, c["slots"].cuda())
    assert torch.equal(kc.cpu(), c["k_cache"]) and torch.equal(vc.cpu(), c["v_cache"])


def test_kv_store_mla_dims_and_strided_source(vb):
    # different K / V head dims (reference: tests/test_fa4_deepseek_shape.py:306-332)
    N, H, dk, dv, blocks, page = 37, 16, 192, 128, 8, 16
    big = _seeded(N, H, dk + dv, seed=10, dtype=BF).cuda()
    key = big[..., :dk].contiguous()
    val = big[..., dk:].contiguous()
    slots = torch.randperm(blocks * page, generator=torch.Generator().manual_seed(3))[:N].to(torch.int32)
    slots[5] = -1
    kc = torch.zeros(blocks, page, H, dk, dtype=BF).cuda()
    vc = torch.zeros(blocks, page, H, dv, dtype=BF).cuda()
    vb.store_kvcache(key, val, kc, vc, slots.cuda())
    kc_ref = torch.zeros(blocks, page, H, dk, dtype=BF)
    vc_ref = torch.zeros(blocks, page, H, dv, dtype=BF)
    ops.kv_store(key.cpu(), val.cpu(), kc_ref, vc_ref, slots)
    assert torch.equal(kc.cpu(), kc_ref) and torch.equal(vc.cpu(), vc_ref)


@pytest.mark.parametrize("with_norm", [True, False])
def test_qknorm_rope_store(vb, with_norm):
    from vexact_b200 import _lib

    T, hq, hkv, D, blocks, page = 19, 8, 2, 128, 6, 16
    qkv = _seeded(T, (hq + 2 * hkv) * D, seed=11, dtype=BF)
    pos = torch.tensor([0, 1, 2, 3, 17, 100, 1023, 2047, 4095, 8191, 5, 6, 7, 8, 9, 10, 11, 12, 13])
    qw = (1 + 0.1 * _seeded(D, seed=12)).to(BF) if with_norm else None
    kw = (1 + 0.1 * _seeded(D, seed=13)).to(BF) if with_norm else None
    slots = torch.randperm(blocks * page, generator=torch.Generator().manual_seed(4))[:T].to(torch.int32)
    slots[2] = -1
    q_ref, k_ref, v_ref = ops.qknorm_rope(qkv, pos, hq, hkv, D, qw, kw, 1e6, 1e-6)
    _, _, inv_freq = ops.rope_cos_sin(pos, D, 1e6)
    kc = torch.zeros(blocks, page, hkv, D, dtype=BF).cuda()
    vc = torch.zeros(blocks, page, hkv, D, dtype=BF).cuda()
    q_out = torch.empty(T, hq, D, dtype=BF).cuda()
    qkv_g, pos_g, slots_g, inv_g = qkv.cuda(), pos.cuda(), slots.cuda(), inv_freq.cuda()
    qw_g = qw.cuda() if with_norm else None
    kw_g = kw.cuda() if with_norm else None
    _lib.check(_lib.load().b200_qknorm_rope_store(
        qkv_g.data_ptr(), qkv_g.stride(0), pos_g.data_ptr(), slots_g.data_ptr(), _lib.ptr(qw_g), _lib.ptr(kw_g),
        inv_g.data_ptr(), q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), T, hq, hkv, D, blocks * page, 1e-6,
        _lib.current_stream()), "b200_qknorm_rope_store")
    kc_ref = torch.zeros(blocks, page, hkv, D, dtype=BF)
    vc_ref = torch.zeros(blocks, page, hkv, D, dtype=BF)
    ops.kv_store(k_ref, v_ref, kc_ref, vc_ref, slots)
    assert torch.equal(vc.cpu(), vc_ref)
    # cos/sin come from the device math library: allow one bf16 ulp, require near-total equality
    for got, want in ((q_out.cpu(), q_ref), (kc.cpu(), kc_ref)):
        torch.testing.assert_close(got.float(), want.float(), rtol=2 ** -6, atol=2e-2)
        assert (got == want).float().mean() > 0.99


def test_mla_rope_store(vb):
    """Interleaved rotary embedding + K/V assembly of DeepSeek-V3 attention vs the oracle
    (reference: modeling_deepseek_v3.py:240-261; HF apply_rotary_pos_emb_interleave)."""
    from oracle import cpu_model
    from vexact_b200 import _lib

    T, heads, nope, rope, dv, blocks, page = 11, 4, 128, 64, 128, 4, 16
    q = _seeded(T, heads * (nope + rope), seed=20, dtype=BF)
    kvb = _seeded(T, heads * (nope + dv), seed=21, dtype=BF)
    ckv = _seeded(T, 96 + rope, seed=22, dtype=BF)          # k_rot is a column slice of a wider tensor
    pos = torch.tensor([0, 1, 2, 3, 17, 100, 1023, 2047, 4095, 8191, 5])
    slots = torch.randperm(blocks * page, generator=torch.Generator().manual_seed(5))[:T].to(torch.int32)
    slots[4] = -1
    cos, sin, inv_freq = ops.rope_cos_sin(pos, rope, 50000.0)
    qv = q.view(T, heads, nope + rope)
    q_ref = torch.cat((qv[..., :nope], cpu_model.rope_interleave(qv[..., nope:].contiguous(), cos, sin)), -1)
    kv = kvb.view(T, heads, nope + dv)
    k_rot = cpu_model.rope_interleave(ckv[:, 96:].reshape(T, 1, rope).contiguous(), cos, sin).expand(T, heads, rope)
    k_ref = torch.cat((kv[..., :nope], k_rot), -1).contiguous()
    v_ref = kv[..., nope:].contiguous()
    kc_ref = torch.zeros(blocks, page, heads, nope + rope, dtype=BF)
    vc_ref = torch.zeros(blocks, page, heads, dv, dtype=BF)
    ops.kv_store(k_ref, v_ref, kc_ref, vc_ref, slots)
    qg, kvbg, ckvg = q.cuda(), kvb.cuda(), ckv.cuda()
    krg = ckvg[:, 96:]
    q_out = torch.empty(T, heads, nope + rope, dtype=BF).cuda()
    kc = torch.zeros_like(kc_ref).cuda()
    vc = torch.zeros_like(vc_ref).cuda()
    pg, sg, fg = pos.cuda(), slots.cuda(), inv_freq.cuda()
    _lib.check(_lib.load().b200_mla_rope_store(
        qg.data_ptr(), qg.stride(0), kvbg.data_ptr(), kvbg.stride(0), krg.data_ptr(), krg.stride(0), pg.data_ptr(),
        sg.data_ptr(), fg.data_ptr(), q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), T, heads, nope, rope, dv,
        blocks * page, _lib.current_stream()), "b200_mla_rope_store")
    assert torch.equal(vc.cpu(), vc_ref)
    assert torch.equal(q_out.cpu()[..., :nope], q_ref[..., :nope]) and torch.equal(kc.cpu()[..., :nope], kc_ref[..., :nope])
    for got, want in ((q_out.cpu(), q_ref), (kc.cpu(), kc_ref)):
        torch.testing.assert_close(got.float(), want.float(), rtol=2 ** -6, atol=5e-2)
        assert (got == want).float().mean() > 0.99


def test_status_word_clean(vb):
    torch.cuda.synchronize()
    assert vb._lib.read_status()[0] == 0


@pytest.mark.gpu
def test_rms_norm_backward_matches_reference_formula_and_is_row_invariant():
    """BatchInvariantRMSNormFunction.backward (batch_invariant_ops.py:701-725) restated in fp32 torch."""
    import vexact_b200 as vb

    g = torch.Generator().manual_seed(5)
    rows, n, eps = 200, 2048, 1e-6
    x = torch.randn(rows, n, generator=g).to(BF).cuda().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(n, generator=g)).to(BF).cuda().requires_grad_(True)
    go = torch.randn(rows, n, generator=g).to(BF).cuda()
    y = vb.batch_invariant_rms_norm(x, w, eps)
    y.backward(go)
    xf, wf, gf = x.detach().float(), w.detach().float(), go.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    normed = xf * inv
    d = gf * wf
    gx_ref = inv * (d - normed * (d * normed).mean(-1, keepdim=True))
    gw_ref = (gf * normed).sum(0)
    torch.testing.assert_close(x.grad.float(), gx_ref, rtol=2 ** -7, atol=2e-3)
    torch.testing.assert_close(w.grad.float(), gw_ref, rtol=2 ** -6, atol=5e-2)
    # a row's input gradient does not depend on the batch it is in
    x1 = x.detach()[7:8].clone().requires_grad_(True)
    w1 = w.detach().clone().requires_grad_(True)
    vb.batch_invariant_rms_norm(x1, w1, eps).backward(go[7:8])
    assert torch.equal(x1.grad[0], x.grad[7])


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_gather_logprob_backward_matches_autograd(vb, dtype):
    """Gradient of `logprobs_from_logits_flash_attn` with respect to the logits (the reference wraps flash-attn's
    cross_entropy_loss, whose backward is softmax - onehot; standalone_logprobs.py:28-55): against torch autograd on
    log_softmax + gather in fp32; an ignored label gives a zero row; `inplace_backward=True` writes into the logits."""
    g = torch.Generator().manual_seed(12)
    rows, vocab = 7, 5003
    x = (torch.randn(rows, vocab, generator=g) * 3).to(dtype).cuda()
    labels = torch.randint(0, vocab, (rows,), generator=g).cuda()
    labels[3] = -100
    go = torch.randn(rows, generator=g).cuda()
    leaf = x.clone().requires_grad_(True)
    out = vb.logprobs_from_logits_flash_attn(leaf, labels)
    assert torch.equal(out, vb.logprobs_from_logits_flash_attn(x, labels))
    out.backward(go)
    ref = x.float().clone().requires_grad_(True)
    lp = torch.log_softmax(ref, -1).gather(-1, labels.clamp(min=0).unsqueeze(-1)).squeeze(-1)
    (lp * (labels != -100)).backward(go)
    assert leaf.grad.dtype == dtype and not leaf.grad[3].any()
    tol = 2e-6 if dtype == torch.float32 else 2 ** -8
    torch.testing.assert_close(leaf.grad.float(), ref.grad, rtol=tol, atol=tol * ref.grad.abs().max().item())
    # in place: the gradient lands in the logits' own storage
    buf = x.clone()
    leaf2 = buf.detach().requires_grad_(True)
    vb.logprobs_from_logits_flash_attn(leaf2, labels, inplace_backward=True).backward(go)
    assert leaf2.grad.data_ptr() == leaf2.data_ptr() and torch.equal(leaf2.grad, leaf.grad)
