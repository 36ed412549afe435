"""This library's kernels against outputs of the reference's own COMPILED kernels.

The fixtures tests/golden/ref_gpu_*.pt were written on a B200 by tests/golden/make_reference_gpu_golden.py,
which ran the reference package (its Triton kernels, quack's grouped GEMM, flash-attn's Triton cross
entropy) on seeded inputs; tests/golden/reference_agreement_b200.json is that run's report.  The inputs
are rebuilt here from the same seeds (a checksum stored with every fixture guards the rebuild), so the
reference itself is not needed to run these tests.

Tolerances, with what the generating run measured in brackets:
  matmul (+bias), mean.dim, KV store, fused MoE (Triton and quack expert functions), MoE index math,
      log-prob of fp32 logits                       bit-exact                    [bit-exact]
  RMSNorm (single rounding)                         <= 1 bf16 ulp, >= 99.9 % identical   [1 of 131072 elements off by 1 ulp]
  log_softmax fp32                                  4e-6 absolute                [1.9e-6]
  log-prob of bf16 logits                           2e-6 absolute                [9.5e-7]
  paged attention (bf16 P, 128- vs 64-key blocks)   0.05 absolute, mean 2e-3     [max 0.031 at |out| <= 4, mean 7e-4]
  model-level per-token logprob (28-layer dense, 2-layer MoE, random init)
                                                    0.25 absolute, mean 0.08     [max 0.125, mean 0.04]
"""
import os
import sys

import pytest
import torch

from conftest import GOLDEN, load_golden

sys.path.insert(0, GOLDEN)
import golden_inputs as gi  # noqa: E402

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"


def _have(name):
    return os.path.exists(os.path.join(GOLDEN, name + ".pt"))


def _bf16_ulp_close(a, b, ulps=1):
    a, b = a.float(), b.float()
    tol = ulps * torch.maximum(a.abs(), b.abs()) * 2.0 ** -7
    return bool(((a - b).abs() <= tol + 1e-30).all())


def test_matmul_bit_exact_vs_reference_triton():
    import vexact_b200 as vb

    for fx in load_golden("ref_gpu_matmul"):
        a, w, bias = gi.matmul_inputs(fx["case"])
        assert gi.checksum(a, w, bias) == fx["checksum"], "seeded inputs changed"
        ad, wd, bd = a.to(DEV), w.to(DEV), bias.to(DEV)
        assert torch.equal(vb.matmul_persistent(ad, wd.t()).cpu(), fx["out"]), fx["case"]
        assert torch.equal(vb.matmul_persistent(ad, wd.t(), bd).cpu(), fx["out_bias"]), fx["case"]


def test_rms_norm_and_mean_vs_reference_triton():
    import vexact_b200 as vb

    for fx in load_golden("ref_gpu_rms_norm"):
        x, w = gi.rmsnorm_inputs(fx["case"])
        assert gi.checksum(x, w) == fx["checksum"]
        out = vb.batch_invariant_rms_norm(x.to(DEV), w.to(DEV), 1e-6).cpu()
        assert _bf16_ulp_close(out, fx["out"], 1), fx["case"]
        assert (out == fx["out"]).float().mean() >= 0.999, fx["case"]
    for fx in load_golden("ref_gpu_mean_dim"):
        x, _ = gi.rmsnorm_inputs(fx["case"], seed=23)
        assert gi.checksum(x) == fx["checksum"]
        assert torch.equal(vb.mean_dim(x.float().to(DEV), -1, keepdim=True).cpu(), fx["out"]), fx["case"]


def test_log_softmax_and_logprob_vs_reference():
    import vexact_b200 as vb

    for fx in load_golden("ref_gpu_logits"):
        x, labels, cols = gi.logits_inputs(fx["case"])
        assert gi.checksum(x, labels) == fx["checksum"]
        xd, ld = x.to(DEV), labels.to(DEV)
        ls = vb.log_softmax(xd, dim=-1)[:, cols.to(DEV)].cpu()
        torch.testing.assert_close(ls, fx["log_softmax_cols"], rtol=0, atol=4e-6)
        assert torch.equal(vb.logprobs_from_logits_flash_attn(xd, ld).cpu(), fx["logprob"]), fx["case"]
        lp16 = vb.logprobs_from_logits_flash_attn(xd.to(BF), ld).float().cpu()
        torch.testing.assert_close(lp16, fx["logprob_bf16_logits"], rtol=0, atol=2e-6)


def test_kv_store_bit_exact_vs_reference_triton():
    import vexact_b200 as vb

    fx = load_golden("ref_gpu_kv_store")
    c = fx["case"]
    key, value, slots = gi.kv_store_inputs()
    assert gi.checksum(key, value, slots) == fx["checksum"]
    kc = torch.zeros((c["blocks"], c["page"], c["heads"], c["dk"]), device=DEV, dtype=BF)
    vc = torch.zeros((c["blocks"], c["page"], c["heads"], c["dv"]), device=DEV, dtype=BF)
    vb.store_kvcache(key.to(DEV), value.to(DEV), kc, vc, slots.to(DEV))
    assert torch.equal(kc.cpu(), fx["k_cache"]) and torch.equal(vc.cpu(), fx["v_cache"])


def test_paged_attention_vs_reference_triton_bf16():
    """bf16 operands, so the reference kernel really rounds P to bf16 before the PV product."""
    import vexact_b200 as vb

    for fx in load_golden("ref_gpu_paged_attention"):
        case = fx["case"]
        q, kc, vc, cu, used, table = gi.attention_inputs(case)
        assert gi.checksum(q, kc, vc, cu, used, table) == fx["checksum"]
        out, _ = vb.flash_attn_varlen_func(q.to(DEV), kc.to(DEV), vc.to(DEV), cu_seqlens_q=cu.to(DEV),
                                           max_seqlen_q=max(case["q_lens"]), seqused_k=used.to(DEV),
                                           page_table=table.to(DEV), softmax_scale=case["dk"] ** -0.5, causal=True)
        d = (out.cpu().float() - fx["out"].float()).abs()
        assert d.max() <= 0.05 and d.mean() <= 2e-3, (case["name"], float(d.max()), float(d.mean()))


def test_fused_moe_bit_exact_vs_reference_triton_and_quack():
    import vexact_b200 as vb
    from vexact_b200.fused_moe import build_moe_indices

    for fx in load_golden("ref_gpu_fused_moe"):
        case = fx["case"]
        hidden, gate_up, down, router = gi.moe_inputs(case)
        assert gi.checksum(hidden, gate_up, down, router) == fx["checksum"]
        E, k, I = case["E"], case["k"], case["I"]
        hd, gud, dd = hidden.to(DEV), gate_up.to(DEV), down.to(DEV)
        sel, rw = fx["selected"].to(DEV), fx["weights"].to(DEV)
        # routing on the same logits picks the same experts (the stored ones come from torch.topk)
        logits = vb.matmul_persistent(hd, router.to(DEV).t())
        ow, osel = vb.route_softmax_topk(logits, k, True)
        assert torch.equal(osel.sort(-1).values, sel.sort(-1).values), case["name"]
        # index math against the reference's histogram kernel and sorts
        cu, _, scat = build_moe_indices(sel, E)
        assert torch.equal(scat.cpu(), fx["scatter_index"]), case["name"]
        assert torch.equal((cu[1:] - cu[:-1]).cpu(), fx["splits"]), case["name"]
        out = vb.fused_moe_forward(E, rw, sel, hd, fc2_weight=dd, fc1_1_2_weight=gud)
        split = vb.fused_moe_forward(E, rw, sel, hd, gud[:, :I].contiguous(), gud[:, I:].contiguous(), dd)
        for tag in ("out_triton", "out_quack"):
            assert tag in fx, f"the generating run could not execute the reference's {tag[4:]} path"
            assert torch.equal(out.cpu(), fx[tag]), (case["name"], tag)
            assert torch.equal(split.cpu(), fx[tag]), (case["name"], tag, "split fc1 weights")


def _stage_logprobs(model, fx, steps):
    """Feeds the reference run's tokens through the stage runner; per step the logprob of the reference's
    greedy token at every sequence's last position."""
    from vexact_b200.inferencer import StageRunner, StepInputs, allocate_kv_cache
    from vexact_b200.models import shape_from_hf_config, stage_weights_from_hf

    shape = shape_from_hf_config(model.config)
    w = stage_weights_from_hf(model, shape, device=DEV)
    kc, vc = allocate_kv_cache(shape, 0, shape.num_layers, steps.nblocks, steps.page, device=DEV)
    runner = StageRunner(w, kc, vc)
    plan = [steps.prefill()] + [steps.decode(fx["ref_tokens"][i].to(DEV), i) for i in range(fx["decode_steps"])]
    outs = []
    for st in plan:
        inp = StepInputs(input_ids=st["input_ids"], hidden_in=None, positions=st["positions"],
                         slot_mapping=st["slot_mapping"], query_start_loc=st["query_start_loc"],
                         context_lens=st["context_lens"], block_tables=st["block_tables"],
                         max_seqlen_q=st["max_seqlen_q"])
        outs.append(runner.step(inp)[2].float().clone())
    return outs


def _check_model_fixture(fx, outs):
    worst, mean = 0.0, 0.0
    for i, logits in enumerate(outs):
        lp = torch.log_softmax(logits, dim=-1)
        # the reference's own greedy token: the first decode input for step 0, its argmax afterwards
        tok = fx["ref_greedy"][i].to(DEV)
        d = (lp.gather(1, tok[:, None]).squeeze(1).cpu() - fx["ref_logprobs"][i]).abs()
        worst, mean = max(worst, float(d.max())), max(mean, float(d.mean()))
    print(f"{fx['model']}: per-token logprob delta vs the reference run: max {worst:.4f}, worst step mean {mean:.4f}")
    assert worst <= 0.25 and mean <= 0.08


@pytest.mark.skipif(not _have("ref_gpu_model_qwen3_dense"), reason="fixture not generated")
def test_dense_model_logprobs_vs_reference_run():
    transformers = pytest.importorskip("transformers")
    fx = load_golden("ref_gpu_model_qwen3_dense")
    if "ref_greedy" not in fx:
        pytest.skip("fixture predates reproducible weights")
    with torch.device(DEV):
        model = transformers.Qwen3ForCausalLM(gi.dense_model_config()).to(BF).eval()
    gi.reinit_parameters(model, seed=fx["init_seed"])
    steps = gi.Steps(fx["prompt_lens"], model.config.vocab_size, fx["page"], fx["seed"], DEV)
    _check_model_fixture(fx, _stage_logprobs(model, fx, steps))


@pytest.mark.skipif(not _have("ref_gpu_model_qwen3_moe"), reason="fixture not generated")
def test_moe_model_logprobs_vs_reference_run():
    transformers = pytest.importorskip("transformers")
    fx = load_golden("ref_gpu_model_qwen3_moe")
    if "ref_greedy" not in fx:
        pytest.skip("fixture predates reproducible weights")
    with torch.device(DEV):
        model = transformers.Qwen3MoeForCausalLM(gi.moe_model_config(2)).to(BF).eval()
    gi.reinit_parameters(model, seed=fx["init_seed"])
    steps = gi.Steps(fx["prompt_lens"], model.config.vocab_size, fx["page"], fx["seed"], DEV)
    _check_model_fixture(fx, _stage_logprobs(model, fx, steps))
