"""Runs the reference's COMPILED kernels on a B200 next to this library's kernels.

    sh tests/golden/install_reference.sh          # once, where the reference checkout exists
    python tests/golden/make_reference_gpu_golden.py --out <dir> [--sections a,b,...]

For every op of the hot path it (1) builds seeded inputs (tests/golden/golden_inputs.py), (2) runs the
reference implementation from baseline/_ref on the GPU (its Triton kernels, quack's GEMM, flash-attn's
Triton cross entropy: whatever `vexact` itself would call on this GPU), (3) runs this library on the
same inputs, (4) times both with CUDA events and (5) writes
    <out>/ref_gpu_<op>.pt        small fixtures (reference outputs + case descriptions + input checksums)
                                 that tests/test_gpu_reference_parity.py replays without the reference,
    <out>/reference_agreement.json   max-abs / mismatch-rate / logprob deltas and the timings.
Model-level sections run a stock HuggingFace module tree twice, once under the reference's
`enable_batch_invariant_mode()` + attention function + MoE patch and once under this library's, plus
the stage runner on weights loaded from the same module, and report per-token logprob deltas.

A section that cannot run records the exception text instead of numbers.  One GPU only: quack's sm100
GEMM uses thread-block clusters, so this script is a one-GPU tool and is kept out of multi-GPU runs.  Test infrastructure: nothing here is imported by vexact_b200/ or timed by bench.py.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import traceback
import types

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("VEXACT_REF", os.path.join(ROOT, "baseline", "_ref"))
for p in (HERE, ROOT, REF):
    if p not in sys.path:
        sys.path.insert(0, p)
os.environ.setdefault("VEXACT_DISABLE_MODEL_PATCH", "1")   # register_models() would import veomni (absent)

import torch  # noqa: E402

import golden_inputs as gi  # noqa: E402

BF = torch.bfloat16
DEV = "cuda"
REPORT: dict = {}


# --------------------------------------------------------------------------------------- helpers
def cuda_ms(fn, warm=3, reps=10, flush=None):
    """Median CUDA-event time of fn() in ms; `flush` (a big tensor) is rewritten between runs."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        if flush is not None:
            flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def delta(ours: torch.Tensor, ref: torch.Tensor) -> dict:
    o, r = ours.detach().float().cpu(), ref.detach().float().cpu()
    d = (o - r).abs()
    return {"max_abs": float(d.max()) if d.numel() else 0.0, "mean_abs": float(d.mean()) if d.numel() else 0.0,
            "ref_max_abs": float(r.abs().max()) if r.numel() else 0.0,
            "frac_bit_identical": float((ours.detach().cpu() == ref.detach().cpu()).float().mean()) if d.numel() else 1.0}


def section(name):
    def deco(fn):
        fn._section = name
        return fn
    return deco


def run_section(fn, out_dir):
    name = fn._section
    t0 = time.time()
    try:
        REPORT[name] = fn(out_dir)
    except Exception as e:  # record, keep going
        REPORT[name] = {"error": f"{type(e).__name__}: {e}", "traceback": traceback.format_exc()[-1500:]}
    REPORT[name]["seconds"] = round(time.time() - t0, 1)
    print(f"[{name}] {json.dumps(REPORT[name])[:600]}", flush=True)
    with open(os.path.join(out_dir, "reference_agreement.json"), "w") as f:
        json.dump(REPORT, f, indent=1)


def save(out_dir, name, obj):
    torch.save(obj, os.path.join(out_dir, name + ".pt"))


def flush_buffer():
    return torch.zeros(160 * 1024 * 1024, dtype=torch.float16, device=DEV)   # 320 MB > L2


# --------------------------------------------------------------------------------------- op level
@section("matmul")
def sec_matmul(out_dir):
    import vexact.batch_invariant_ops as rbio
    import vexact_b200 as vb

    cases, rep = [], []
    for case in gi.MATMUL_CASES:
        a, w, bias = gi.matmul_inputs(case)
        ad, wd, bd = a.to(DEV), w.to(DEV), bias.to(DEV)
        r = rbio.matmul_persistent(ad, wd.t())
        rb = rbio.matmul_persistent(ad, wd.t(), bd)
        o = vb.matmul_persistent(ad, wd.t())
        ob = vb.matmul_persistent(ad, wd.t(), bd)
        cases.append(dict(case=case, checksum=gi.checksum(a, w, bias), out=r.cpu(), out_bias=rb.cpu()))
        rep.append(dict(case=case, plain=delta(o, r), bias=delta(ob, rb)))
    save(out_dir, "ref_gpu_matmul", cases)
    # reference row invariance on this GPU (its own claim), config-1 shape
    a, w, _ = gi.matmul_inputs(dict(M=256, K=2048, N=6144), seed=12)
    ad, wd = a.to(DEV), w.to(DEV)
    full = rbio.matmul_persistent(ad, wd.t())
    inv = {m: bool(torch.equal(rbio.matmul_persistent(ad[:m], wd.t()), full[:m])) for m in (1, 7, 64)}
    ours_full = vb.matmul_persistent(ad, wd.t())
    timing = {}
    fl = flush_buffer()
    for (M, K, N, tag) in [(512, 2048, 5120, "qkv"), (512, 4096, 2048, "o"), (512, 2048, 128, "router"),
                           (512, 2048, 151936, "lm_head"), (64, 2048, 6144, "cfg1_M64"), (256, 2048, 6144, "cfg1_M256")]:
        x = torch.randn(M, K, device=DEV).to(BF)
        wt = (torch.randn(N, K, device=DEV) * 0.02).to(BF)
        timing[tag] = dict(shape=[M, K, N], ref_ms=cuda_ms(lambda: rbio.matmul_persistent(x, wt.t()), flush=fl),
                           ours_ms=cuda_ms(lambda: vb.matmul_persistent(x, wt.t()), flush=fl))
        del x, wt
    return dict(cases=rep, reference_row_invariant_M1_7_64_vs_256=inv, cfg1_M256=delta(ours_full, full), timing=timing)


@section("rmsnorm_mean_logsoftmax_logprob")
def sec_rowops(out_dir):
    import vexact.batch_invariant_ops as rbio
    import vexact.batch_invariant_ops.batch_invariant_ops as rmod
    from vexact.batch_invariant_ops.standalone_logprobs import logprobs_from_logits_flash_attn as ref_lp
    import vexact_b200 as vb

    rep = {}
    cases = []
    for case in gi.RMSNORM_CASES:
        x, w = gi.rmsnorm_inputs(case)
        xd, wd = x.to(DEV), w.to(DEV)
        r = rbio.batch_invariant_rms_norm(xd, wd, 1e-6)
        o = vb.batch_invariant_rms_norm(xd, wd, 1e-6)
        cases.append(dict(case=case, checksum=gi.checksum(x, w), out=r.cpu()))
        rep.setdefault("rms_norm", []).append(dict(case=case, **delta(o, r)))
    save(out_dir, "ref_gpu_rms_norm", cases)

    cases = []
    for case in gi.RMSNORM_CASES[:3]:
        x, _ = gi.rmsnorm_inputs(case, seed=23)
        xf = x.float().to(DEV)
        r = rbio.mean_dim(xf, -1, keepdim=True)
        o = vb.mean_dim(xf, -1, keepdim=True)
        cases.append(dict(case=case, checksum=gi.checksum(x), out=r.cpu()))
        rep.setdefault("mean_dim", []).append(dict(case=case, **delta(o, r)))
    save(out_dir, "ref_gpu_mean_dim", cases)

    cases = []
    for case in gi.LOGITS_CASES:
        x, labels, cols = gi.logits_inputs(case)
        xd, ld = x.to(DEV), labels.to(DEV)
        r = rbio.log_softmax(xd, dim=-1)
        o = vb.log_softmax(xd, dim=-1)
        rl = ref_lp(xd, ld)
        ol = vb.logprobs_from_logits_flash_attn(xd, ld)
        rl16 = ref_lp(xd.to(BF), ld)
        ol16 = vb.logprobs_from_logits_flash_attn(xd.to(BF), ld)
        cases.append(dict(case=case, checksum=gi.checksum(x, labels), log_softmax_cols=r[:, cols.to(DEV)].cpu(),
                          logprob=rl.cpu(), logprob_bf16_logits=rl16.float().cpu()))
        rep.setdefault("log_softmax", []).append(dict(case=case, **delta(o, r)))
        rep.setdefault("logprob_fp32_logits", []).append(dict(case=case, **delta(ol, rl)))
        rep.setdefault("logprob_bf16_logits", []).append(dict(case=case, **delta(ol16.float(), rl16.float())))
    save(out_dir, "ref_gpu_logits", cases)

    # timings at config-1 shapes (memory-bound row ops: achieved GB/s on algorithmic bytes)
    fl = flush_buffer()
    t = {}
    M, n, V = 4096, 2048, 151936
    x = torch.randn(M, n, device=DEV).to(BF)
    w = torch.ones(n, device=DEV, dtype=BF)
    for tag, rf, of, nbytes in [
        ("rms_norm_4096x2048", lambda: rbio.batch_invariant_rms_norm(x, w, 1e-6),
         lambda: vb.batch_invariant_rms_norm(x, w, 1e-6), 2 * M * n * 2),
        ("hf_rms_norm_4096x2048", None, lambda: vb.hf_rms_norm(x, w, 1e-6), 2 * M * n * 2),
    ]:
        e = dict(bytes=nbytes, ours_ms=cuda_ms(of, flush=fl))
        e["ours_GBps"] = nbytes / e["ours_ms"] / 1e6
        if rf is not None:
            e["ref_ms"] = cuda_ms(rf, flush=fl)
        t[tag] = e
    rows = 256
    lg = torch.randn(rows, V, device=DEV) * 2
    lab = torch.randint(0, V, (rows,), device=DEV)
    lg16 = lg.to(BF)
    for tag, rf, of, nbytes in [
        ("log_softmax_f32_256x151936", lambda: rbio.log_softmax(lg), lambda: vb.log_softmax(lg), 8 * rows * V),
        ("gather_logprob_f32_256x151936", lambda: ref_lp(lg, lab), lambda: vb.logprobs_from_logits_flash_attn(lg, lab),
         4 * rows * V),
        ("gather_logprob_bf16_256x151936", lambda: ref_lp(lg16, lab),
         lambda: vb.logprobs_from_logits_flash_attn(lg16, lab), 2 * rows * V),
    ]:
        e = dict(bytes=nbytes, ours_ms=cuda_ms(of, flush=fl), ref_ms=cuda_ms(rf, flush=fl))
        e["ours_GBps"] = nbytes / e["ours_ms"] / 1e6
        e["ref_GBps"] = nbytes / e["ref_ms"] / 1e6
        t[tag] = e
    rep["timing"] = t
    _ = rmod
    return rep


@section("kv_store")
def sec_kv_store(out_dir):
    from vexact.batch_invariant_ops.kv_cache_context import store_kvcache as ref_store
    import vexact_b200 as vb

    c = gi.KV_STORE_CASE
    key, value, slots = gi.kv_store_inputs()
    shape_k, shape_v = (c["blocks"], c["page"], c["heads"], c["dk"]), (c["blocks"], c["page"], c["heads"], c["dv"])
    outs = []
    for store in (ref_store, vb.store_kvcache):
        kc, vc = torch.zeros(shape_k, device=DEV, dtype=BF), torch.zeros(shape_v, device=DEV, dtype=BF)
        store(key.to(DEV), value.to(DEV), kc, vc, slots.to(DEV))
        outs.append((kc.cpu(), vc.cpu()))
    save(out_dir, "ref_gpu_kv_store", dict(case=c, checksum=gi.checksum(key, value, slots), k_cache=outs[0][0],
                                           v_cache=outs[0][1]))
    # timing: config-4 decode shape (512 tokens, 4 kv heads x 128) and a 2048-token prefill chunk
    t = {}
    fl = flush_buffer()
    for T in (512, 2048):
        k = torch.randn(T, 4, 128, device=DEV).to(BF)
        v = torch.randn(T, 4, 128, device=DEV).to(BF)
        kc = torch.zeros(4096, 16, 4, 128, device=DEV, dtype=BF)
        vc = torch.zeros_like(kc)
        sl = torch.randperm(4096 * 16, device=DEV)[:T].int()
        nbytes = 2 * 2 * T * 4 * 128 * 2
        e = dict(bytes=nbytes, ours_ms=cuda_ms(lambda: vb.store_kvcache(k, v, kc, vc, sl), flush=fl),
                 ref_ms=cuda_ms(lambda: ref_store(k, v, kc, vc, sl), flush=fl))
        e["ours_GBps"] = nbytes / e["ours_ms"] / 1e6
        t[f"T{T}"] = e
    return dict(k_equal=bool(torch.equal(outs[0][0], outs[1][0])), v_equal=bool(torch.equal(outs[0][1], outs[1][1])),
                timing=t)


@section("paged_attention")
def sec_attention(out_dir):
    from vexact.batch_invariant_ops.triton_invariant_attention import flash_attn_varlen_func as ref_attn
    import vexact_b200 as vb

    rep, cases = [], []
    for case in gi.ATTENTION_CASES:
        q, kc, vc, cu, used, table = gi.attention_inputs(case)
        args = [t.to(DEV) for t in (q, kc, vc, cu, used, table)]
        scale = case["dk"] ** -0.5
        kw = dict(cu_seqlens_q=args[3], max_seqlen_q=max(case["q_lens"]), seqused_k=args[4], page_table=args[5],
                  softmax_scale=scale, causal=True)
        r, _ = ref_attn(args[0], args[1], args[2], **kw)
        o, _ = vb.flash_attn_varlen_func(args[0], args[1], args[2], **kw)
        # the reference's own batched-vs-single invariance on this GPU: sequence 0 alone
        n0 = case["q_lens"][0]
        r1, _ = ref_attn(args[0][:n0], args[1], args[2], cu_seqlens_q=args[3][:2], max_seqlen_q=n0,
                         seqused_k=args[4][:1], page_table=args[5][:1], softmax_scale=scale, causal=True)
        cases.append(dict(case=case, checksum=gi.checksum(q, kc, vc, cu, used, table), out=r.cpu()))
        rep.append(dict(case=case["name"], reference_batched_equals_single=bool(torch.equal(r1, r[:n0])), **delta(o, r)))
    save(out_dir, "ref_gpu_paged_attention", cases)

    # timing: config-4 decode (512 x 2048 ctx, 32 / 4 heads, 16-token pages) and a 2048-token causal prefill
    t = {}
    S, ctx, page, hq, hkv, d = 512, 2048, 16, 32, 4, 128
    pages = ctx // page
    g = torch.Generator(device=DEV).manual_seed(0)
    kc = torch.randn(S * pages, page, hkv, d, device=DEV, generator=g).to(BF)
    vc = torch.randn(S * pages, page, hkv, d, device=DEV, generator=g).to(BF)
    table = torch.randperm(S * pages, device=DEV, generator=g).view(S, pages).int()
    q = torch.randn(S, hq, d, device=DEV, generator=g).to(BF)
    cu = torch.arange(S + 1, dtype=torch.int32, device=DEV)
    used = torch.full((S,), ctx, dtype=torch.int32, device=DEV)
    kw = dict(cu_seqlens_q=cu, max_seqlen_q=1, seqused_k=used, page_table=table, softmax_scale=d ** -0.5, causal=True)
    r, _ = ref_attn(q, kc, vc, **kw)
    o, _ = vb.flash_attn_varlen_func(q, kc, vc, **kw)
    nbytes = S * ctx * hkv * 2 * d * 2
    t["decode_cfg4"] = dict(kv_bytes=nbytes, **delta(o, r),
                            ref_ms=cuda_ms(lambda: ref_attn(q, kc, vc, **kw), warm=2, reps=5),
                            ours_ms=cuda_ms(lambda: vb.flash_attn_varlen_func(q, kc, vc, **kw), warm=2, reps=5))
    qlen = 2048
    qp = torch.randn(qlen, hq, d, device=DEV, generator=g).to(BF)
    kw = dict(cu_seqlens_q=torch.tensor([0, qlen], dtype=torch.int32, device=DEV), max_seqlen_q=qlen,
              seqused_k=torch.tensor([qlen], dtype=torch.int32, device=DEV), page_table=table[:1].contiguous(),
              softmax_scale=d ** -0.5, causal=True)
    r, _ = ref_attn(qp, kc, vc, **kw)
    o, _ = vb.flash_attn_varlen_func(qp, kc, vc, **kw)
    flops = 2.0 * (qlen * (qlen + 1) / 2) * hq * 2 * d
    e = dict(flops=flops, **delta(o, r), ref_ms=cuda_ms(lambda: ref_attn(qp, kc, vc, **kw), warm=2, reps=5),
             ours_ms=cuda_ms(lambda: vb.flash_attn_varlen_func(qp, kc, vc, **kw), warm=2, reps=5))
    e["ref_tflops"], e["ours_tflops"] = flops / e["ref_ms"] / 1e9, flops / e["ours_ms"] / 1e9
    t["prefill_2048_cfg4_heads"] = e
    return dict(cases=rep, timing=t)


def _ref_topk_route(logits, k):
    """modeling_qwen3_moe.py:128-134 in plain torch (the reference's own routing code path)."""
    w = torch.softmax(logits, dim=1, dtype=torch.float)
    w, sel = torch.topk(w, k, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return w.to(BF), sel


@section("fused_moe")
def sec_moe(out_dir):
    import vexact.batch_invariant_ops.fused_moe as rmoe
    from vexact.batch_invariant_ops.group_gemm.kernel.group_gemm import group_gemm_same_nk
    from vexact.batch_invariant_ops.group_gemm.kernel.moe import expert_histogram, moe_gather, moe_scatter
    import vexact_b200 as vb
    from vexact_b200.fused_moe import build_moe_indices

    rep, cases = [], []
    for case in gi.MOE_CASES:
        hidden, gate_up, down, router = gi.moe_inputs(case)
        E, k, I = case["E"], case["k"], case["I"]
        hd, gud, dd, rd = (t.to(DEV) for t in (hidden, gate_up, down, router))
        logits = vb.matmul_persistent(hd, rd.t())
        rw, sel = _ref_topk_route(logits, k)
        ow, osel = vb.route_softmax_topk(logits, k, True)
        fc11, fc12 = gud[:, :I].contiguous(), gud[:, I:].contiguous()
        entry = dict(case=case["name"])
        # index math: the reference's histogram kernel + sorts against this library's index kernel
        splits = expert_histogram(sel, E)
        cu_ref, aidx_ref, scat_ref = rmoe._build_moe_indices(sel, E)
        cu, aidx, scat = build_moe_indices(sel, E)
        entry["indices_bit_exact"] = bool(torch.equal(cu.cpu(), cu_ref.cpu()) and torch.equal(aidx.cpu(), aidx_ref.cpu())
                                          and torch.equal(scat.cpu(), scat_ref.cpu()))
        entry["routing_sets_equal_frac"] = float((sel.sort(-1).values == osel.sort(-1).values).all(-1).float().mean())
        # the Triton expert function (what DEVICE_MAJOR < 9 runs) and the quack one (what this GPU runs)
        fix = dict(case=case, checksum=gi.checksum(hidden, gate_up, down, router), selected=sel.cpu(),
                   weights=rw.cpu(), splits=splits.cpu(), scatter_index=scat_ref.cpu())
        for tag, fn in (("triton", rmoe.FusedMoeExpertFunction), ("quack", rmoe.QuackFusedMoeExpertFunction)):
            try:
                with torch.no_grad():
                    r = fn.apply(E, rw, sel, hd, fc11, fc12, dd)
                fix["out_" + tag] = r.cpu()
                o = vb.fused_moe_forward(E, rw, sel, hd, fc2_weight=dd, fc1_1_2_weight=gud)
                o_split = vb.fused_moe_forward(E, rw, sel, hd, fc11, fc12, dd)
                entry[tag] = delta(o, r)
                entry[tag + "_split_weights"] = delta(o_split, r)
            except Exception as e:
                entry[tag] = {"error": f"{type(e).__name__}: {e}"[:400]}
        # moe_scatter / moe_gather alone
        sc = moe_scatter(hd, scat_ref)
        y = torch.randn(sel.numel(), case["H"], device=DEV).to(BF)
        ga = moe_gather(y, scat_ref)
        fix["gather_in_seed"] = 0
        from vexact_b200 import _lib
        ours_ga = torch.empty_like(ga)
        _lib.check(_lib.load().b200_moe_unpermute_reduce(y.data_ptr(), scat_ref.contiguous().data_ptr(), None,
                                                         ours_ga.data_ptr(), hd.shape[0], k, case["H"],
                                                         _lib.current_stream()), "b200_moe_unpermute_reduce")
        entry["moe_gather"] = delta(ours_ga, ga)
        entry["moe_scatter_rows_match"] = bool(torch.equal(sc[scat_ref.flatten().long()],
                                                           hd.repeat_interleave(k, dim=0)))
        cases.append(fix)
        rep.append(entry)
        _ = group_gemm_same_nk
    save(out_dir, "ref_gpu_fused_moe", cases)
    return dict(cases=rep)


@section("moe_timing_cfg4")
def sec_moe_timing(out_dir):
    """ours vs the reference's Triton path vs quack's sm100 GEMM at the config-4 layer shape,
    uniform routing and a Zipf(1.1)-skewed one."""
    import vexact.batch_invariant_ops.fused_moe as rmoe
    from vexact.batch_invariant_ops.group_gemm.kernel.group_gemm import group_gemm_same_nk
    from quack.gemm_interface import gemm as quack_gemm
    import vexact_b200 as vb
    from vexact_b200.fused_moe import _grouped_gemm, _permute

    T, E, k, H, I = 512, 128, 8, 2048, 768
    g = torch.Generator(device=DEV).manual_seed(0)
    hidden = torch.randn(T, H, device=DEV, generator=g).to(BF)
    gate_up = (torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.02).to(BF)
    down = (torch.randn(E, H, I, device=DEV, generator=g) * 0.02).to(BF)
    router = (torch.randn(E, H, device=DEV, generator=g) * 0.02).to(BF)
    fc11, fc12 = gate_up[:, :I].contiguous(), gate_up[:, I:].contiguous()
    zipf = torch.tensor([1.0 / (i + 1) ** 1.1 for i in range(E)], device=DEV)
    bias = zipf[torch.randperm(E, device=DEV, generator=g)] * 8.0     # skewed variant: per-expert logit bias
    out = {}
    fl = flush_buffer()
    for tag, b in (("uniform", None), ("zipf", bias)):
        logits = vb.matmul_persistent(hidden, router.t()).float()
        if b is not None:
            logits = logits + b
        rw, sel = _ref_topk_route(logits, k)
        counts = torch.bincount(sel.flatten(), minlength=E)
        e = dict(rows_per_expert_max=int(counts.max()), rows_per_expert_mean=float(counts.float().mean()),
                 experts_hit=int((counts > 0).sum()))
        e["ours_ms"] = cuda_ms(lambda: vb.fused_moe_forward(E, rw, sel, hidden, fc2_weight=down, fc1_1_2_weight=gate_up),
                               flush=fl)
        for name, fn in (("triton", rmoe.FusedMoeExpertFunction), ("quack", rmoe.QuackFusedMoeExpertFunction)):
            try:
                with torch.no_grad():
                    e[name + "_ms"] = cuda_ms(lambda: fn.apply(E, rw, sel, hidden, fc11, fc12, down), flush=fl)
            except Exception as ex:
                e[name + "_error"] = f"{type(ex).__name__}: {ex}"[:300]
        # the GEMMs alone
        plan = _permute(sel, rw, hidden, E)
        e["tiles"] = int(plan["tile_count"].item())
        xp, rs = plan["x_perm"], plan["row_scale"]
        e["ours_fc1_swiglu_ms"] = cuda_ms(lambda: _grouped_gemm(xp, gate_up, rs, plan, I, mode=1), flush=fl)
        hmid = _grouped_gemm(xp, gate_up, rs, plan, I, mode=1)
        e["ours_fc2_ms"] = cuda_ms(lambda: _grouped_gemm(hmid, down, None, plan, H, mode=0), flush=fl)
        cu_ref, aidx_ref, scat_ref = rmoe._build_moe_indices(sel, E)
        cumsum_t = torch.cumsum(torch.bincount(sel.flatten(), minlength=E), 0)
        try:
            e["triton_fc1_two_gemms_ms"] = cuda_ms(lambda: (
                group_gemm_same_nk(a=xp, b=fc11, cumsum_M=cumsum_t, max_M=xp.shape[0], transpose_a=False, transpose_b=True),
                group_gemm_same_nk(a=xp, b=fc12, cumsum_M=cumsum_t, max_M=xp.shape[0], transpose_a=False, transpose_b=True)),
                flush=fl)
            e["triton_fc2_ms"] = cuda_ms(lambda: group_gemm_same_nk(a=hmid, b=down, cumsum_M=cumsum_t, max_M=xp.shape[0],
                                                                    transpose_a=False, transpose_b=True), flush=fl)
        except Exception as ex:
            e["triton_gemm_error"] = f"{type(ex).__name__}: {ex}"[:300]
        try:
            w1t, w2t, w3t = fc11.transpose(1, 2), fc12.transpose(1, 2), down.transpose(1, 2)
            e["quack_fc1_two_gemms_ms"] = cuda_ms(lambda: (
                quack_gemm(hidden, w1t, cu_seqlens_m=cu_ref, A_idx=aidx_ref),
                quack_gemm(hidden, w2t, cu_seqlens_m=cu_ref, A_idx=aidx_ref)), flush=fl)
            e["quack_fc2_ms"] = cuda_ms(lambda: quack_gemm(hmid, w3t, cu_seqlens_m=cu_ref), flush=fl)
        except Exception as ex:
            e["quack_gemm_error"] = f"{type(ex).__name__}: {ex}"[:300]
        out[tag] = e
    # many rows per expert (a 2048-token prefill chunk): the regime of quack's large tiles
    T2 = 4096
    hidden2 = torch.randn(T2, H, device=DEV, generator=g).to(BF)
    logits = vb.matmul_persistent(hidden2, router.t()).float()
    rw, sel = _ref_topk_route(logits, k)
    e = dict(tokens=T2)
    e["ours_ms"] = cuda_ms(lambda: vb.fused_moe_forward(E, rw, sel, hidden2, fc2_weight=down, fc1_1_2_weight=gate_up),
                           flush=fl, reps=5)
    for name, fn in (("triton", rmoe.FusedMoeExpertFunction), ("quack", rmoe.QuackFusedMoeExpertFunction)):
        try:
            with torch.no_grad():
                e[name + "_ms"] = cuda_ms(lambda: fn.apply(E, rw, sel, hidden2, fc11, fc12, down), flush=fl, reps=5)
        except Exception as ex:
            e[name + "_error"] = f"{type(ex).__name__}: {ex}"[:300]
    e["flops"] = 2.0 * T2 * k * 3 * H * I
    out["prefill_4096_tokens"] = e
    return out


@section("dsv3_router_flip_rate")
def sec_router(out_dir):
    """DeepSeek-V3 router: the reference multiplies fp32 operands with tl.dot (TF32 inputs), this library
    with exact fp32 FMAs.  Same seeded hidden states and weights through both, then the reference's
    routing rule on each set of logits: how often does the selected expert set differ?"""
    import vexact.batch_invariant_ops as rbio
    import vexact_b200 as vb
    from oracle import ops as oracle_ops

    T, H, E, k = 4096, 2048, 64, 6
    x = gi.randn((T, H), 71).to(DEV)
    w = gi.randn((E, H), 72, 0.02).to(DEV)
    bias = torch.zeros(E)
    ref_logits = rbio.matmul_persistent(x.float(), w.float().t())
    our_logits = vb.linear(x.float(), w.float())
    exact = (x.double() @ w.double().t()).float()
    sel_ref, _ = oracle_ops.route_sigmoid_group_topk(ref_logits.cpu(), bias, 1, 1, k, True, 2.446)
    sel_our, _ = oracle_ops.route_sigmoid_group_topk(our_logits.cpu(), bias, 1, 1, k, True, 2.446)
    sel_gpu, _ = vb.route_sigmoid_group_topk(our_logits, bias.to(DEV), 1, 1, k, True, 2.446)
    same = (sel_ref.sort(-1).values == sel_our.sort(-1).values).all(-1)
    return dict(tokens=T, reference_logits_vs_fp64=delta(ref_logits, exact), ours_logits_vs_fp64=delta(our_logits, exact),
                ours_vs_reference_logits=delta(our_logits, ref_logits), flip_rate=float(1 - same.float().mean()),
                gpu_routing_equals_oracle_on_same_logits=bool(
                    (sel_gpu.cpu().sort(-1).values == sel_our.sort(-1).values).all()))


# --------------------------------------------------------------------------------------- model level
def _install_veomni_stand_in():
    """The reference's model files call `veomni.ops.fused_moe_forward(..., fc1_1_2_weight=...)`; veomni is
    not installed.  Bind that name to the reference's own fused MoE (vexact.batch_invariant_ops.fused_moe),
    splitting the fused gate_up weight, which is the implementation the reference documents as equivalent."""
    import vexact.batch_invariant_ops.fused_moe as rmoe

    def fused_moe_forward(num_experts, routing_weights, selected_experts, hidden_states, fc1_1_weight=None,
                          fc1_2_weight=None, fc2_weight=None, fc1_1_2_weight=None):
        if fc1_1_2_weight is not None:
            half = fc1_1_2_weight.shape[1] // 2
            fc1_1_weight = fc1_1_2_weight[:, :half].contiguous()
            fc1_2_weight = fc1_1_2_weight[:, half:].contiguous()
        return rmoe.fused_moe_forward(num_experts, routing_weights, selected_experts, hidden_states, fc1_1_weight,
                                      fc1_2_weight, fc2_weight)

    pkg, ops = types.ModuleType("veomni"), types.ModuleType("veomni.ops")
    ops.fused_moe_forward = fused_moe_forward
    pkg.ops = ops
    sys.modules["veomni"], sys.modules["veomni.ops"] = pkg, ops


def _hf_step(model, ctx_mod, caches, st):
    ctx_mod.set_kv_cache_context(is_paged_attn=True, key_cache=caches[0], value_cache=caches[1],
                                 block_tables=st["block_tables"], context_lens=st["context_lens"],
                                 slot_mapping=st["slot_mapping"], query_start_loc=st["query_start_loc"],
                                 max_seqlen_q=st["max_seqlen_q"])
    with torch.inference_mode():
        out = model(input_ids=st["input_ids"][None], position_ids=st["positions"][None], use_cache=False)
    last = (st["query_start_loc"][1:] - 1).long()
    return out.logits[0, last].clone()


def _alloc_caches(layers, nblocks, page, hkv, dk, dv, fill=None):
    kc, vc = {}, {}
    for li in range(layers):
        kc[li] = torch.zeros(nblocks, page, hkv, dk, device=DEV, dtype=BF)
        vc[li] = torch.zeros(nblocks, page, hkv, dv, device=DEV, dtype=BF)
        if fill is not None:
            kc[li].copy_(fill[0][li])
            vc[li].copy_(fill[1][li])
    return kc, vc


def _logprob_of(logits, tokens):
    lp = torch.log_softmax(logits.float(), dim=-1)
    return lp.gather(1, tokens[:, None]).squeeze(1)


def _compare_logits(ours, ref, tokens):
    d = delta(ours, ref)
    lp_o, lp_r = _logprob_of(ours, tokens), _logprob_of(ref, tokens)
    dl = (lp_o - lp_r).abs()
    return dict(logits=d, logprob_delta_max=float(dl.max()), logprob_delta_mean=float(dl.mean()),
                greedy_agree=float((ours.argmax(-1) == ref.argmax(-1)).float().mean()))


ATTN_KEY = "fa-invariant"   # one of the reference's ALL_ATTENTION_FUNCTIONS keys; the function behind it is swapped


def _model_agreement(model, shape_name, heads, page, prompt_lens, decode_steps, seed, before_ref=None,
                     before_ours=None):
    """Runs the module tree under the reference's kernels, then under this library's (HF drop-in and the
    stage runner on the same weights), feeding both the reference's greedy tokens."""
    import vexact.batch_invariant_ops as rbio
    import vexact.batch_invariant_ops.kv_cache_context as rctx
    import vexact_b200 as vb
    import vexact_b200.kv_cache_context as octx
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    from vexact_b200.inferencer import StageRunner, StepInputs
    from vexact_b200.models import shape_from_hf_config, stage_weights_from_hf

    cfg = model.config
    L, (hkv, dk, dv) = cfg.num_hidden_layers, heads
    steps = gi.Steps(prompt_lens, cfg.vocab_size, page, seed, DEV)
    plan = [steps.prefill()]                                    # one packed prefill step
    res = {"model": shape_name, "sequences": steps.S, "prefill_tokens": int(sum(prompt_lens)),
           "decode_steps": decode_steps}

    def run(mode):
        if mode == "ref":
            ALL_ATTENTION_FUNCTIONS[ATTN_KEY] = rbio.triton_flash_attention_forward
            if before_ref:
                before_ref()
            rbio.enable_batch_invariant_mode()
            ctx_mod = rctx
        else:
            ALL_ATTENTION_FUNCTIONS[ATTN_KEY] = vb.flash_attention_forward
            if before_ours:
                before_ours()
            vb.enable_batch_invariant_mode()
            ctx_mod = octx
        caches = _alloc_caches(L, steps.nblocks, page, hkv, dk, dv)
        outs, toks = [], []
        try:
            lg = _hf_step(model, ctx_mod, caches, plan[0])
            outs.append(lg)
            for i in range(decode_steps):
                nxt = run.ref_tokens[i] if mode != "ref" else lg.argmax(-1)
                toks.append(nxt)
                st = steps.decode(nxt, i)
                lg = _hf_step(model, ctx_mod, caches, st)
                outs.append(lg)
        finally:
            (rbio if mode == "ref" else vb).disable_batch_invariant_mode()
            torch.use_deterministic_algorithms(False)   # both mode switches turn it on and leave it on
        if mode == "ref":
            run.ref_tokens = toks
        return outs, caches

    t0 = time.time()
    ref_outs, _ = run("ref")
    res["reference_seconds"] = round(time.time() - t0, 1)
    t0 = time.time()
    our_outs, our_caches = run("ours")
    res["ours_hf_dropin_seconds"] = round(time.time() - t0, 1)
    ref_tok = [o.argmax(-1) for o in ref_outs]
    res["hf_dropin_vs_reference"] = [_compare_logits(o, r, t) for o, r, t in zip(our_outs, ref_outs, ref_tok)]

    # the stage runner on weights loaded from the same module tree
    shape = shape_from_hf_config(cfg, shape_name)
    w = stage_weights_from_hf(model, shape, device=DEV)
    kc, vc = _alloc_caches(L, steps.nblocks, page, hkv, dk, dv)
    runner = StageRunner(w, kc, vc)
    st_outs = []
    sts = [plan[0]] + [steps.decode(run.ref_tokens[i], i) for i in range(decode_steps)]
    for st in sts:
        inp = StepInputs(input_ids=st["input_ids"], hidden_in=None, positions=st["positions"],
                         slot_mapping=st["slot_mapping"], query_start_loc=st["query_start_loc"],
                         context_lens=st["context_lens"], block_tables=st["block_tables"],
                         max_seqlen_q=st["max_seqlen_q"])
        _, _, lg = runner.step(inp)
        st_outs.append(lg.clone())
    res["stage_runner_vs_reference"] = [_compare_logits(o, r, t) for o, r, t in zip(st_outs, ref_outs, ref_tok)]
    res["stage_runner_vs_hf_dropin"] = [_compare_logits(o, r, t) for o, r, t in zip(st_outs, our_outs, ref_tok)]
    fixture = dict(model=shape_name, prompt_lens=prompt_lens, page=page, seed=seed, decode_steps=decode_steps,
                   ref_tokens=[t.cpu() for t in run.ref_tokens], ref_greedy=[t.cpu() for t in ref_tok],
                   ref_logprobs=[_logprob_of(o, t).cpu() for o, t in zip(ref_outs, ref_tok)],
                   ref_top_logits=[o.float().topk(8, dim=-1).values.cpu() for o in ref_outs])
    return res, fixture


@section("model_qwen3_dense_cfg2")
def sec_model_dense(out_dir):
    import transformers

    cfg = gi.dense_model_config()
    from vexact_b200.attention import register_attention_functions

    register_attention_functions()
    cfg._attn_implementation = ATTN_KEY
    torch.manual_seed(0)
    with torch.device(DEV):
        model = transformers.Qwen3ForCausalLM(cfg).to(BF).eval()
    gi.reinit_parameters(model, seed=100)
    g = torch.Generator().manual_seed(5)
    prompt_lens = torch.randint(16, 120, (16,), generator=g).tolist()
    res, fix = _model_agreement(model, "qwen3-1.7b-shape", (8, 128, 128), 16, prompt_lens, 4, seed=7)
    fix["init_seed"] = 100
    save(out_dir, "ref_gpu_model_qwen3_dense", fix)
    return res


@section("model_qwen3_moe_cfg4_2layers")
def sec_model_moe(out_dir):
    import transformers
    from vexact.models.qwen3_moe.modeling_qwen3_moe import apply_qwen3_moe_patches as ref_patch

    _install_veomni_stand_in()
    ref_patch()                                   # fused experts container + the reference's block forward
    import transformers.models.qwen3_moe.modeling_qwen3_moe as hfm

    ref_forward = hfm.Qwen3MoeSparseMoeBlock.forward
    cfg = gi.moe_model_config(2)
    from vexact_b200.attention import register_attention_functions
    import vexact_b200.models as om

    register_attention_functions()
    cfg._attn_implementation = ATTN_KEY
    torch.manual_seed(0)
    with torch.device(DEV):
        model = transformers.Qwen3MoeForCausalLM(cfg).to(BF).eval()
    gi.reinit_parameters(model, seed=101)          # (the reference's expert container allocates with torch.empty)
    g = torch.Generator().manual_seed(6)
    prompt_lens = torch.randint(16, 100, (24,), generator=g).tolist()

    # the same module tree runs the reference's block forward in the reference pass and this library's in ours
    def use_ref_forward():
        hfm.Qwen3MoeSparseMoeBlock.forward = ref_forward

    def use_our_forward():
        hfm.Qwen3MoeSparseMoeBlock.forward = om._qwen3_moe_block_forward

    res, fix = _model_agreement(model, "qwen3-30b-a3b-shape-2layers", (4, 128, 128), 16, prompt_lens, 4, seed=8,
                                before_ref=use_ref_forward, before_ours=use_our_forward)
    fix["init_seed"] = 101
    save(out_dir, "ref_gpu_model_qwen3_moe", fix)
    return res


@section("backward")
def sec_backward(out_dir):
    """Training-side gradients: the reference's packed attention backward (triton_invariant_attention.py:194-431)
    and its Triton fused-MoE backward (fused_moe.py:113-265) next to this library's, same bf16 inputs and
    upstream gradients.  Numbers only (max-abs / mean-abs deltas per gradient); no fixtures are stored."""
    from vexact.batch_invariant_ops.triton_invariant_attention import flash_attn_varlen_func as ref_attn
    import vexact.batch_invariant_ops.fused_moe as rmoe
    import vexact_b200 as vb

    rep = {}
    g = torch.Generator().manual_seed(7)
    q_lens, kv_lens, hq, hkv, d = [65, 129], [65, 129], 4, 2, 128
    base = [torch.randn(sum(q_lens), hq, d, generator=g).to(BF).to(DEV),
            torch.randn(sum(kv_lens), hkv, d, generator=g).to(BF).to(DEV),
            torch.randn(sum(kv_lens), hkv, d, generator=g).to(BF).to(DEV)]
    dout = torch.randn(sum(q_lens), hq, d, generator=g).to(BF).to(DEV)
    cu_q = torch.tensor([0, 65, 194], dtype=torch.int32, device=DEV)
    grads = {}
    for tag, fn in (("reference", ref_attn), ("ours", vb.flash_attn_varlen_func)):
        leaves = [t.clone().requires_grad_(True) for t in base]
        out, _ = fn(*leaves, cu_q, cu_q, max_seqlen_q=129, max_seqlen_k=129, softmax_scale=d ** -0.5, causal=True)
        out.backward(dout)
        grads[tag] = [out.detach()] + [t.grad for t in leaves]
    rep["attention"] = {n: delta(o, r) for n, o, r in zip(("out", "dq", "dk", "dv"), grads["ours"], grads["reference"])}
    REPORT["backward"] = dict(rep)                       # partial results survive a late failure
    with open(os.path.join(out_dir, "reference_agreement.json"), "w") as f:
        json.dump(REPORT, f, indent=1)

    for case in (gi.MOE_CASES[0], gi.MOE_CASES[2]):
        _backward_moe_case(case, g, rep)
    return rep


def _backward_moe_case(case, g, rep):
    import vexact.batch_invariant_ops.fused_moe as rmoe
    import vexact_b200 as vb

    try:
        hidden, gate_up, down, router = gi.moe_inputs(case)
        E, k, I = case["E"], case["k"], case["I"]
        hd, gud, dd, rd = (t.to(DEV) for t in (hidden, gate_up, down, router))
        rw, sel = _ref_topk_route(vb.matmul_persistent(hd, rd.t()), k)
        gy = torch.randn(hd.shape, generator=g).to(BF).to(DEV)
        base = dict(rw=rw, x=hd, w1=gud[:, :I].contiguous(), w2=gud[:, I:].contiguous(), w3=dd)
        grads = {}
        for tag, fn in (("reference", rmoe.FusedMoeExpertFunction.apply),
                        ("ours", vb.fused_moe.FusedMoeExpertFunction.apply)):
            lv = {n: t.clone().requires_grad_(True) for n, t in base.items()}
            out = fn(E, lv["rw"], sel, lv["x"], lv["w1"], lv["w2"], lv["w3"])
            out.backward(gy)
            grads[tag] = dict(out=out.detach(), **{n: t.grad for n, t in lv.items()})
        rep["fused_moe_" + case["name"]] = {n: delta(grads["ours"][n], grads["reference"][n]) for n in grads["ours"]}
    except Exception as e:      # keep the other numbers
        rep["fused_moe_" + case["name"]] = {"error": f"{type(e).__name__}: {e}"[:600]}


SECTIONS = [sec_matmul, sec_rowops, sec_kv_store, sec_attention, sec_moe, sec_moe_timing, sec_router, sec_model_dense,
            sec_model_moe, sec_backward]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(ROOT, "ref_gpu_out"))
    ap.add_argument("--sections", default="")
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the reference's kernels are Triton / CuTe-DSL GPU code")
    if not os.path.isdir(os.path.join(REF, "vexact")):
        raise SystemExit(f"{REF}/vexact not found: run tests/golden/install_reference.sh where the checkout exists")
    torch.cuda.set_device(0)
    import triton

    REPORT["environment"] = dict(gpu=torch.cuda.get_device_name(0), torch=torch.__version__, triton=triton.__version__,
                                 reference=REF)
    try:
        import quack

        REPORT["environment"]["quack"] = getattr(quack, "__version__", "?")
    except Exception as e:
        REPORT["environment"]["quack"] = f"unavailable: {e}"
    want = [s for s in args.sections.split(",") if s]
    for fn in SECTIONS:
        if want and fn._section not in want:
            continue
        run_section(fn, args.out)
        torch.cuda.empty_cache()
    from vexact_b200 import _lib

    REPORT["status_word"] = list(_lib.read_status())
    with open(os.path.join(args.out, "reference_agreement.json"), "w") as f:
        json.dump(REPORT, f, indent=1)
    print("done", flush=True)


if __name__ == "__main__":
    main()
