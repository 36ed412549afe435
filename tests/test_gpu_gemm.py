"""GPU parity: tcgen05 weight-streaming GEMM vs the CPU oracle and the reference's golden
fixtures, and bitwise row invariance across batch sizes
(reference: tests/batch_invariant_ops/test_matmul.py:27-46, test_batch_invariance.py:30-128)."""
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


def _close_bf16(got, want, k):
    # stated tolerance: one bf16 ulp (rtol 2^-7) plus fp32 accumulation-order noise for results
    # that cancel towards zero; and the vast majority of elements bit-identical
    torch.testing.assert_close(got.float(), want.float(), rtol=2 ** -7, atol=1e-6 * k ** 0.5 + 1e-5)
    assert (got == want).float().mean() > 0.98


def test_gemm_golden(vb):
    for c in load_golden("matmul"):
        a, w, bias = c["a"].cuda(), c["w"].cuda(), c["bias"].cuda()
        _close_bf16(vb.matmul_persistent(a, w.t()).cpu(), c["out"], a.shape[1])
        _close_bf16(vb.matmul_persistent(a, w.t(), bias).cpu(), c["out_bias"], a.shape[1])


@pytest.mark.parametrize("M,K,N", [(1, 2048, 6144), (7, 2048, 6144), (64, 2048, 6144), (256, 2048, 6144),
                                   (300, 768, 2048), (512, 4096, 2048), (5, 72, 40), (129, 1536, 576)])
def test_gemm_oracle(vb, M, K, N):
    x = _seeded(M, K, seed=1)
    w = _seeded(N, K, seed=2, std=0.02)
    ref = ops.matmul(x, w.t())
    out = vb.matmul_persistent(x.cuda(), w.cuda().t())
    _close_bf16(out.cpu(), ref, K)
    # row-major B ([K, N] contiguous) and fp32 output
    out2 = vb.matmul_persistent(x.cuda(), w.t().contiguous().cuda())
    assert torch.equal(out, out2)
    out32 = vb.linear(x.cuda(), w.cuda(), out_dtype=torch.float32)
    assert torch.equal(out32.to(BF), out)


def test_gemm_bias_fp32_before_cast(vb):
    x = _seeded(33, 1536, seed=3)
    w = _seeded(256, 1536, seed=4, std=0.02)
    b = _seeded(256, seed=5, std=0.5)
    ref = ops.matmul(x, w.t(), b)
    out = torch.addmm(b.cuda(), x.cuda(), w.cuda().t()) if False else vb.matmul_persistent(x.cuda(), w.cuda().t(), b.cuda())
    _close_bf16(out.cpu(), ref, 1536)


def test_gemm_row_invariance_sweep(vb):
    """Row i of X @ W^T is bit-identical for every batch size 1..512 (BASELINE config 1)."""
    K, N = 2048, 6144
    x = _seeded(512, K, seed=6).cuda()
    w = _seeded(N, K, seed=7, std=0.02).cuda()
    full = vb.matmul_persistent(x, w.t())
    sizes = sorted(set([1, 2, 3, 7, 8, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300, 384,
                        511, 512] + list(range(1, 513, 37))))
    for m in sizes:
        part = vb.matmul_persistent(x[:m], w.t())
        assert torch.equal(part, full[:m]), f"rows differ between batch {m} and batch 512"
    # a row's result does not depend on its position in the batch either
    perm = torch.randperm(512, generator=torch.Generator().manual_seed(0)).cuda()
    assert torch.equal(vb.matmul_persistent(x[perm].contiguous(), w.t()), full[perm])


def test_gemm_large_m_prefill_shape(vb):
    x = _seeded(2048, 2048, seed=8)
    w = _seeded(1024, 2048, seed=9, std=0.02)
    out = vb.matmul_persistent(x.cuda(), w.cuda().t())
    ref = ops.matmul(x, w.t())
    _close_bf16(out.cpu(), ref, 2048)
    assert torch.equal(vb.matmul_persistent(x[:5].cuda(), w.cuda().t()), out[:5])


def test_aten_override_routes_linear(vb):
    lin = torch.nn.Linear(512, 384, bias=True).to(BF).cuda()
    x = _seeded(9, 512, seed=10).cuda()
    with vb.set_batch_invariant_mode(True):
        y = lin(x)
        y1 = lin(x[:1])
        lsm = torch.log_softmax(x.float(), dim=-1)
    assert torch.equal(y[:1], y1)
    _close_bf16(y.cpu(), ops.matmul(x.cpu(), lin.weight.detach().cpu().t(), lin.bias.detach().cpu()), 512)
    torch.testing.assert_close(lsm.cpu(), ops.log_softmax(x.float().cpu()), rtol=0, atol=6e-6)
    assert not vb.is_batch_invariant_mode_enabled()


def test_gemm_f32_router(vb):
    x = _seeded(40, 2048, seed=11, dtype=torch.float32)
    w = _seeded(64, 2048, seed=12, std=0.02, dtype=torch.float32)
    out = vb.matmul_persistent(x.cuda(), w.cuda().t())
    torch.testing.assert_close(out.cpu(), x @ w.t(), rtol=1e-5, atol=1e-5)
    assert torch.equal(vb.matmul_persistent(x[:3].cuda(), w.cuda().t()), out[:3])


def test_status_word_clean(vb):
    torch.cuda.synchronize()
    assert vb._lib.read_status()[0] == 0


@pytest.mark.gpu
def test_fused_lm_head_greedy_matches_two_kernel_path_and_is_batch_invariant():
    """lm_head -> greedy token + logprob without the logits tensor: same tokens as GEMM + greedy_logprob,
    log-probabilities within 2e-5, and a token's (token, logprob) are the same bits at batch 1 and 512."""
    import vexact_b200 as vb
    from vexact_b200.standalone_logprobs import greedy_token_and_logprob, lm_head_greedy

    g = torch.Generator().manual_seed(21)
    for (T, K, V) in [(512, 2048, 151936), (300, 512, 4097), (7, 256, 130)]:
        x = torch.randn(T, K, generator=g).to(BF).cuda()
        w = (torch.randn(V, K, generator=g) * 0.02).to(BF).cuda()
        tok, lp = lm_head_greedy(x, w)
        tok_ref, lp_ref = greedy_token_and_logprob(vb.linear(x, w))
        assert torch.equal(tok, tok_ref), f"{(T, K, V)}: {(tok != tok_ref).sum().item()} tokens differ"
        torch.testing.assert_close(lp, lp_ref, rtol=0, atol=2e-5)
        for sub in ([0], [T - 1], list(range(0, T, max(1, T // 5)))):
            t1, l1 = lm_head_greedy(x[sub].contiguous(), w)
            assert torch.equal(t1, tok[sub]) and torch.equal(l1, lp[sub]), f"{(T, K, V)}: rows {sub} depend on the batch"
    # a tie: two identical weight rows give identical logits; the lower vocabulary index wins
    w[100] = w[3]
    x1 = (w[3].float() * 50).to(BF)[None].contiguous()
    t1, _ = lm_head_greedy(x1, w)
    tr, _ = greedy_token_and_logprob(vb.linear(x1, w))
    assert t1.item() == tr.item()
    from vexact_b200 import _lib
    assert _lib.read_status()[0] == 0


def test_fp16_matmul_and_batch_invariance(vb):
    """matmul_persistent on fp16 tensors (the reference serves bf16, fp16 and fp32): fp32 accumulation, bias in
    fp32, one rounding to fp16; a row's bits do not depend on the batch it is computed in."""
    g = torch.Generator().manual_seed(12)
    for (M, K, N) in [(1, 2048, 768), (7, 512, 200), (64, 2048, 6144), (300, 1536, 256)]:
        a = (torch.randn(M, K, generator=g)).half()
        w = (torch.randn(N, K, generator=g) * 0.05).half()
        bias = torch.randn(N, generator=g).half()
        ad, wd, bd = a.cuda(), w.cuda(), bias.cuda()
        out = vb.matmul_persistent(ad, wd.t())
        outb = vb.matmul_persistent(ad, wd.t(), bd)
        assert out.dtype == torch.float16
        ref = a.double() @ w.double().t()
        for got, want in ((out, ref), (outb, ref + bias.double())):
            err = (got.cpu().double() - want).abs()
            tol = 2.0 ** -10 * want.abs().clamp(min=0.5)           # one fp16 ulp, with a floor for cancellation
            assert bool((err <= tol).all()), (M, K, N, float(err.max()))
        assert torch.equal(vb.matmul_persistent(ad[:1], wd.t(), bd), outb[:1])
        if M > 8:
            assert torch.equal(vb.matmul_persistent(ad[5:8], wd.t(), bd), outb[5:8])


def test_mm_under_the_mode_takes_any_layout(vb):
    """Under the mode switch every aten::mm / addmm on CUDA tensors lands here, not only nn.Linear: a reduction
    length that is no multiple of 8, a row-major right operand, operands sliced at an odd element offset.  The
    reference's Triton kernel takes any strides (batch_invariant_ops.py:54-156); here such operands go through
    zero-padded copies, which leaves every fp32 accumulation as it was: the padded-K result equals the result
    for the same numbers laid out at K + pad with explicit zeros, and rows stay batch-invariant."""
    a = _seeded(33, 77, seed=21).cuda()
    b = _seeded(77, 50, seed=22).cuda()                     # row-major [K, N], K = 77
    with vb.set_batch_invariant_mode(True):
        c = torch.mm(a, b)
        c1 = torch.mm(a[:1], b)
        cb = torch.addmm(_seeded(50, seed=23).cuda(), a, b)
    assert torch.equal(c[:1], c1)
    a_pad = torch.nn.functional.pad(a, (0, 3))
    b_pad = torch.nn.functional.pad(b, (0, 0, 0, 3))
    assert torch.equal(c, vb.matmul_persistent(a_pad, b_pad))
    _close_bf16(c.cpu(), ops.matmul(a.cpu(), b.cpu()), 77)
    _close_bf16(cb.cpu(), ops.matmul(a.cpu(), b.cpu(), _seeded(50, seed=23)), 77)
    big = _seeded(9 * 64 + 1, seed=24).cuda()
    odd = big[1:].view(9, 64)                               # K fine, data pointer off by one element
    w = _seeded(64, 32, seed=25).cuda()
    assert torch.equal(vb.matmul_persistent(odd, w), vb.matmul_persistent(odd.clone(), w))


def test_conv3d_under_the_mode_is_deterministic_and_batch_invariant(vb):
    """Reference tests/batch_invariant_ops/test_torch_conv3d.py:50-115 (the Qwen3-VL patch embedding, cuDNN off):
    ten identical runs, and sample 0 alone equal to sample 0 of the batch."""
    import torch.nn.functional as F

    cout, cin, kt, kh, kw, batch = 1024, 3, 2, 16, 16, 8
    d, h, w = kt * 2, kh * 2, kw * 2
    a = torch.linspace(-1.0, 1.0, batch * cin * d * h * w, dtype=BF, device="cuda").reshape(batch, cin, d, h, w)
    weight = torch.linspace(-1.0, 1.0, cout * cin * kt * kh * kw, dtype=BF, device="cuda").reshape(cout, cin, kt, kh, kw)
    bias = torch.linspace(-1.0, 1.0, cout, dtype=BF, device="cuda")
    cudnn_was = torch.backends.cudnn.enabled
    torch.backends.cudnn.enabled = False
    try:
        with vb.set_batch_invariant_mode(True):
            out1 = F.conv3d(a, weight, bias=bias, stride=(kt, kh, kw))
            for _ in range(10):
                assert torch.equal(out1, F.conv3d(a, weight, bias=bias, stride=(kt, kh, kw)))
            single = F.conv3d(a[:1], weight, bias=bias, stride=(kt, kh, kw))
        assert torch.equal(single, out1[:1])
    finally:
        torch.backends.cudnn.enabled = cudnn_was
        torch.use_deterministic_algorithms(False)
