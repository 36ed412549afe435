"""Pins the CPU oracle to the fixtures produced by the reference itself
(tests/golden/make_golden.py).  Integer / index results must match exactly; floating
point results within the tolerance written beside each check."""
import torch

from conftest import load_golden
from oracle import ops

BF = torch.bfloat16


def _ulp_diff_bf16(a, b):
    """Difference in units of bf16 spacing at the larger magnitude."""
    a, b = a.float(), b.float()
    scale = torch.maximum(a.abs(), b.abs()).clamp(min=1e-30)
    ulp = 2.0 ** (torch.floor(torch.log2(scale)) - 7)
    return ((a - b).abs() / ulp).max().item()


def test_matmul_matches_reference_kernel():
    for c in load_golden("matmul"):
        out = ops.matmul(c["a"], c["w"].t())
        outb = ops.matmul(c["a"], c["w"].t(), c["bias"])
        # both are fp32 accumulations of exact products, in different orders: <= 1 bf16 ulp
        # (rtol 2^-7 is one bf16 ulp; atol covers results that cancel to near zero)
        torch.testing.assert_close(out.float(), c["out"].float(), rtol=2 ** -7, atol=2e-5)
        torch.testing.assert_close(outb.float(), c["out_bias"].float(), rtol=2 ** -7, atol=2e-5)
        assert (out == c["out"]).float().mean() > 0.99


def test_rms_norm_single_round():
    for c in load_golden("rms_norm_single"):
        out = ops.rms_norm_single_round(c["x"], c["w"], c["eps"])
        assert _ulp_diff_bf16(out, c["out"]) <= 1.0
        assert (out == c["out"]).float().mean() > 0.99


def test_rms_norm_hf_bitwise():
    for c in load_golden("rms_norm_hf"):
        out = ops.rms_norm_hf(c["x"], c["w"], c["eps"])
        assert torch.equal(out, c["out"])


def test_mean_lastdim():
    for c in load_golden("mean_lastdim"):
        out = ops.mean_lastdim(c["x"])
        torch.testing.assert_close(out, c["out"], rtol=0, atol=2e-7)


def test_log_softmax():
    for c in load_golden("log_softmax"):
        out = ops.log_softmax(c["x"])
        torch.testing.assert_close(out, c["out"], rtol=0, atol=4e-6)


def test_gather_logprob_consistent_with_log_softmax():
    for c in load_golden("log_softmax"):
        rows, n = c["x"].shape
        labels = torch.arange(rows) * 7 % n
        lp = ops.gather_logprob(c["x"], labels)
        want = c["out"].gather(-1, labels[:, None]).squeeze(-1)
        torch.testing.assert_close(lp, want, rtol=0, atol=4e-6)
    lp = ops.gather_logprob(c["x"], torch.full((rows,), -100))
    assert torch.all(lp == 0)


def test_rope_bitwise():
    c = load_golden("rope")
    cos, sin, _ = ops.rope_cos_sin(c["positions"], 128, c["theta"])
    assert torch.equal(cos, c["cos"]) and torch.equal(sin, c["sin"])
    q = c["q"][0].transpose(0, 1)  # [T, heads, d]
    k = c["k"][0].transpose(0, 1)
    assert torch.equal(ops.apply_rope(q, cos, sin), c["q_out"][0].transpose(0, 1))
    assert torch.equal(ops.apply_rope(k, cos, sin), c["k_out"][0].transpose(0, 1))


def test_kv_store_exact():
    c = load_golden("kv_store")
    kc = torch.zeros_like(c["k_cache"])
    vc = torch.zeros_like(c["v_cache"])
    ops.kv_store(c["key"], c["value"], kc, vc, c["slots"])
    assert torch.equal(kc, c["k_cache"]) and torch.equal(vc, c["v_cache"])


def test_paged_attention_vs_reference_kernel_and_eager():
    for c in load_golden("paged_attention"):
        args = (c["q"], c["k_cache"], c["v_cache"], c["cu_seqlens_q"], c["seqused_k"], c["page_table"], c["scale"])
        eager = ops.paged_attention(*args).float()
        blocked = ops.paged_attention(*args, block_n=64).float()
        # reference tests' own tolerance for bf16 paged attention vs eager: 3e-3
        # (tests/batch_invariant_ops/test_triton_attention_varlen.py:415)
        torch.testing.assert_close(eager, c["out_eager_fp32"], rtol=0, atol=3e-3 + 8e-3)
        torch.testing.assert_close(blocked, c["out_triton_fp32"], rtol=0, atol=3e-3 + 8e-3)
        # fp32 eager oracle against the reference kernel's fp32 output: bf16 output rounding only
        assert (eager - c["out_triton_fp32"]).abs().max() < 0.02


def test_route_softmax_topk():
    for c in load_golden("route_softmax_topk"):
        w, idx = ops.route_softmax_topk(c["logits"], c["top_k"], True)
        # experts: exact wherever the k-th and (k+1)-th probabilities differ (bf16 logits tie often)
        probs = torch.softmax(c["logits"].float(), 1)
        srt = torch.sort(probs, descending=True).values
        distinct = (srt[:, : c["top_k"] + 1].diff(dim=1) != 0).all(dim=1)
        assert distinct.any()
        assert torch.equal(idx[distinct], c["experts"][distinct])
        # where values tie the selected *set of probabilities* still agrees
        assert torch.equal(torch.sort(probs.gather(1, idx), 1).values,
                           torch.sort(probs.gather(1, c["experts"]), 1).values)
        assert _ulp_diff_bf16(w, c["weights"]) <= 1.0


def test_route_sigmoid_group_topk():
    for c in load_golden("route_sigmoid_group_topk"):
        idx, w = ops.route_sigmoid_group_topk(c["logits"], c["bias"], c["n_group"], c["topk_group"], c["top_k"],
                                              True, c["scale"])
        # the reference uses topk(sorted=False): compare as sets, weights after a joint sort
        a = torch.sort(idx, 1)
        b = torch.sort(c["experts"], 1)
        assert torch.equal(a.values, b.values)
        torch.testing.assert_close(w.gather(1, a.indices), c["weights"].gather(1, b.indices), rtol=1e-6, atol=1e-7)


def test_moe_indices_exact():
    c = load_golden("moe_indices")
    cu, a_idx, scatter = ops.build_moe_indices(c["experts"], c["num_experts"])
    assert (cu == c["cu_seqlens"].numpy()).all()
    assert (a_idx == c["a_idx"].numpy()).all()
    assert (scatter == c["scatter_index"].numpy()).all()


def test_fused_moe_vs_naive_experts():
    c = load_golden("moe_naive")
    E = c["gate_up"].shape[0]
    I = c["gate_up"].shape[1] // 2
    fc1_1, fc1_2 = c["gate_up"][:, :I], c["gate_up"][:, I:]
    out = ops.fused_moe(E, c["weights"], c["experts"], c["hidden"], fc1_1, fc1_2, c["down"])
    out_b = ops.fused_moe_batched(E, c["weights"], c["experts"], c["hidden"], fc1_1, fc1_2, c["down"])
    assert torch.equal(out, out_b)
    # reference threshold for fused vs token-by-token MoE: 1e-3 (tests/batch_invariant_ops/test_fused_moe.py)
    # on outputs of this magnitude; the naive form keeps fp32 between steps, so allow bf16 rounding noise
    err = (out.float() - c["out_fp32"]).abs().max().item()
    assert err < 2e-3 * max(1.0, c["out_fp32"].abs().max().item())


def test_pp_indices_exact():
    table = load_golden("pp_indices")
    for (L, pp), want in table.items():
        got = [ops.get_pp_indices(L, r, pp) for r in range(pp)]
        assert got == [tuple(w) for w in want]


def test_slot_mapping_formula():
    slots = ops.slot_mapping([[3, 1], [2]], [14, 0], [4, 2], 16)
    assert slots.tolist() == [3 * 16 + 14, 3 * 16 + 15, 16, 17, 32, 33]


def test_mla_projection_and_rope_match_hf_deepseek_modules():
    """The oracle's MLA q/k/v (the restatement of modeling_deepseek_v3.py:234-261) equals the HF
    DeepseekV3 modules and helpers that the reference's forward calls, bit for bit."""
    from transformers import DeepseekV3Config
    from transformers.models.deepseek_v3 import modeling_deepseek_v3 as m

    from oracle import cpu_model
    from vexact_b200.inferencer import MLAShape, ModelShape

    torch.manual_seed(0)
    cfg = DeepseekV3Config(hidden_size=256, num_attention_heads=2, num_key_value_heads=2, kv_lora_rank=64,
                           q_lora_rank=None, qk_nope_head_dim=32, qk_rope_head_dim=64, v_head_dim=32,
                           num_hidden_layers=1, intermediate_size=128, moe_intermediate_size=64, n_routed_experts=8,
                           num_experts_per_tok=2, n_shared_experts=1, n_group=1, topk_group=1, vocab_size=64,
                           rope_theta=50000.0, first_k_dense_replace=1, rope_interleave=True)
    att = m.DeepseekV3Attention(cfg, 0).to(BF).eval()
    rot = m.DeepseekV3RotaryEmbedding(cfg)
    T = 7
    x = torch.randn(1, T, 256).to(BF)
    pos = torch.tensor([[0, 1, 5, 17, 100, 1000, 4095]])
    cos, sin = rot(x, pos)
    with torch.no_grad():
        q = att.q_proj(x).view(1, T, -1, 96).transpose(1, 2)
        q_pass, q_rot = torch.split(q, [32, 64], -1)
        ckv = att.kv_a_proj_with_mqa(x)
        k_pass, k_rot = torch.split(ckv, [64, 64], -1)
        k_pass = att.kv_b_proj(att.kv_a_layernorm(k_pass)).view(1, T, -1, 64).transpose(1, 2)
        k_pass, v = torch.split(k_pass, [32, 32], -1)
        q_rot, k_rot = m.apply_rotary_pos_emb_interleave(q_rot, k_rot.view(1, 1, T, 64), cos, sin)
        Q = torch.cat((q_pass, q_rot), -1)
        K = torch.cat((k_pass, k_rot.expand(*k_pass.shape[:-1], -1)), -1)
    shape = ModelShape("t", 1, 256, 2, 2, 96, 64, mla=MLAShape(64, 32, 64, 32), rope_theta=50000.0,
                       rms_eps=cfg.rms_norm_eps, norm_single_round=True)
    lw = dict(qkv=att.q_proj.weight.data, kv_a=att.kv_a_proj_with_mqa.weight.data,
              kv_a_norm=att.kv_a_layernorm.weight.data, kv_b=att.kv_b_proj.weight.data)
    q2, k2, v2 = cpu_model.mla_qkv(shape, lw, x[0], pos[0])
    assert torch.equal(q2, Q[0].transpose(0, 1)) and torch.equal(k2, K[0].transpose(0, 1))
    assert torch.equal(v2, v[0].transpose(0, 1))


# --------------------------------------------------------------------------------------------------------------
# The oracle against outputs of the reference's COMPILED kernels (tests/golden/ref_gpu_*.pt, written on a B200 by
# tests/golden/make_reference_gpu_golden.py; inputs rebuilt here from the same seeds, guarded by checksums).
# These pin what the interpreter fixtures above cannot: bf16 operands end to end (P really rounded to bf16 in the
# attention kernel) and the fused-MoE expert arithmetic (Triton and quack expert functions).  The oracle's GEMMs
# run through torch's CPU bf16 matmul, whose accumulation order is not the kernels', hence tolerances here; the
# CUDA kernels meet the same fixtures bit for bit where tests/test_gpu_reference_parity.py says so.
import os as _os

import pytest
import sys as _sys

from conftest import GOLDEN as _GOLDEN

_sys.path.insert(0, _GOLDEN)
import golden_inputs as _gi  # noqa: E402


def _have(name):
    return _os.path.exists(_os.path.join(_GOLDEN, name + ".pt"))


@pytest.mark.skipif(not _have("ref_gpu_matmul"), reason="fixture not generated")
def test_oracle_matmul_vs_compiled_reference():
    for fx in load_golden("ref_gpu_matmul"):
        a, w, bias = _gi.matmul_inputs(fx["case"])
        assert _gi.checksum(a, w, bias) == fx["checksum"], "seeded inputs changed"
        for got, want in ((ops.matmul(a, w.t()), fx["out"]), (ops.matmul(a, w.t(), bias), fx["out_bias"])):
            tol = 2.0 ** -7 * want.float().abs().clamp(min=0.25)       # one bf16 ulp, with a floor for cancellation
            assert bool(((got.float() - want.float()).abs() <= tol).all()), fx["case"]
            assert (got == want).float().mean() > 0.97, fx["case"]


@pytest.mark.skipif(not _have("ref_gpu_rms_norm"), reason="fixture not generated")
def test_oracle_row_ops_vs_compiled_reference():
    for fx in load_golden("ref_gpu_rms_norm"):
        x, w = _gi.rmsnorm_inputs(fx["case"])
        assert _gi.checksum(x, w) == fx["checksum"]
        got = ops.rms_norm_single_round(x, w, 1e-6)
        assert _ulp_diff_bf16(got, fx["out"]) <= 1 and (got == fx["out"]).float().mean() > 0.999, fx["case"]
    for fx in load_golden("ref_gpu_mean_dim"):
        x, _ = _gi.rmsnorm_inputs(fx["case"], seed=23)
        torch.testing.assert_close(ops.mean_lastdim(x.float()).reshape(-1), fx["out"].reshape(-1), rtol=1e-6, atol=1e-7)
    for fx in load_golden("ref_gpu_logits"):
        x, labels, cols = _gi.logits_inputs(fx["case"])
        assert _gi.checksum(x, labels) == fx["checksum"]
        torch.testing.assert_close(ops.log_softmax(x)[:, cols], fx["log_softmax_cols"], rtol=0, atol=4e-6)
        torch.testing.assert_close(ops.gather_logprob(x, labels), fx["logprob"], rtol=0, atol=4e-6)
    fx = load_golden("ref_gpu_kv_store")
    c = fx["case"]
    key, value, slots = _gi.kv_store_inputs()
    kc = torch.zeros((c["blocks"], c["page"], c["heads"], c["dk"]), dtype=torch.bfloat16)
    vc = torch.zeros((c["blocks"], c["page"], c["heads"], c["dv"]), dtype=torch.bfloat16)
    ops.kv_store(key, value, kc, vc, slots)
    assert torch.equal(kc, fx["k_cache"]) and torch.equal(vc, fx["v_cache"])


@pytest.mark.skipif(not _have("ref_gpu_paged_attention"), reason="fixture not generated")
def test_oracle_attention_vs_compiled_reference_bf16_p():
    """bf16 operands: the reference kernel really rounds P to bf16 (triton_invariant_attention.py:542); the
    blocked oracle with the reference's 64-key blocks restates exactly that."""
    for fx in load_golden("ref_gpu_paged_attention"):
        case = fx["case"]
        q, kc, vc, cu, used, table = _gi.attention_inputs(case)
        assert _gi.checksum(q, kc, vc, cu, used, table) == fx["checksum"]
        block_n = 64 if case["dk"] <= 128 else 32        # the reference's BLOCK_N choice (:648-649)
        got = ops.paged_attention(q, kc, vc, cu, used, table, case["dk"] ** -0.5, block_n=block_n)
        d = (got.float() - fx["out"].float()).abs()
        assert d.max() <= 0.04 and d.mean() <= 1e-3, (case["name"], float(d.max()), float(d.mean()))


@pytest.mark.skipif(not _have("ref_gpu_fused_moe"), reason="fixture not generated")
def test_oracle_fused_moe_vs_compiled_reference_triton_and_quack():
    """The expert arithmetic (fused_moe.py:299-344) as the reference's own Triton and quack expert functions
    computed it on bf16 operands: the oracle's restatement of the rounding points, checked against both."""
    for fx in load_golden("ref_gpu_fused_moe"):
        case = fx["case"]
        hidden, gate_up, down, router = _gi.moe_inputs(case)
        assert _gi.checksum(hidden, gate_up, down, router) == fx["checksum"]
        E, I = case["E"], case["I"]
        sel, rw = fx["selected"], fx["weights"]
        # index math, bit exact against the reference's histogram kernel + sorts
        cu, _, scat = ops.build_moe_indices(sel, E)
        assert torch.equal(torch.as_tensor(scat).reshape(-1).int(), fx["scatter_index"].reshape(-1).int()), case["name"]
        got = ops.fused_moe_batched(E, rw, sel, hidden, gate_up[:, :I], gate_up[:, I:], down)
        for tag in ("out_triton", "out_quack"):
            want = fx[tag]
            tol = 2.0 ** -6 * max(float(want.float().abs().max()), 1e-3)
            torch.testing.assert_close(got.float(), want.float(), rtol=0, atol=tol)
            assert (got == want).float().mean() > 0.90, (case["name"], tag)
