"""Generates tests/golden/*.pt from the reference itself.  Run once, in a container that has
the reference checkout (it does not travel to the GPU box; the fixtures do):

    python tests/golden/make_golden.py /path/to/vexact

How the reference is executed without a GPU:
  * its Triton kernels run under Triton's CPU interpreter (TRITON_INTERPRET=1).  The
    interpreter mishandles bf16 operands of tl.dot, so contraction kernels (matmul, paged
    attention, grouped GEMM) are fed fp32 tensors holding bf16-representable values: every
    product is then exact in fp32 and the accumulation is the kernel's own fp32
    accumulation, i.e. the arithmetic of the bf16 path; outputs are rounded to bf16 here.
    With fp32 operands the attention kernel keeps P in fp32 (its `p.to(dtype)` is a no-op),
    which the fixture records as `p_dtype = "fp32"`.
    Kernels that end in a cast to bf16 (RMSNorm) are treated the same way, because the
    interpreter's fp32->bf16 cast truncates where the compiled kernel rounds to nearest.
  * host wrappers that insist on CUDA tensors are bypassed by launching the jitted kernel
    with the same arguments the wrapper would pass.
  * model-level torch code (routing, RMSNorm, rotary embedding, layer split, block
    allocator) runs as is on CPU.
Every fixture stores its inputs next to the reference's outputs.
"""
from __future__ import annotations

import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
os.environ.setdefault("VEXACT_DISABLE_MODEL_PATCH", "1")

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("VEXACT_SRC", "")
if not os.path.isdir(REF):
    raise SystemExit("usage: pass the path of a vexact checkout (or set VEXACT_SRC)")
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, "tests"))

import torch  # noqa: E402
import triton  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
BF = torch.bfloat16


def bfvals(*shape, std=1.0, gen=None):
    """fp32 tensor whose values are exactly representable in bf16."""
    return (torch.randn(*shape, generator=gen) * std).to(BF).float()


def save(name, obj):
    torch.save(obj, os.path.join(OUT, name + ".pt"))
    print("wrote", name)


def main():
    g = torch.Generator().manual_seed(0)
    import vexact.batch_invariant_ops.batch_invariant_ops as bio

    bio.get_compute_units = lambda: 4

    # ---- matmul_persistent (batch_invariant_ops.py:159), with and without bias
    cases = []
    for (M, K, N) in [(1, 256, 384), (7, 256, 384), (33, 512, 200), (130, 192, 136)]:
        a = bfvals(M, K, gen=g)
        w = bfvals(N, K, std=0.05, gen=g)
        bias = bfvals(N, std=0.5, gen=g)
        c = bio.matmul_persistent(a, w.t())
        cb = bio.matmul_persistent(a, w.t(), bias)
        cases.append(dict(a=a.to(BF), w=w.to(BF), bias=bias.to(BF), out=c.to(BF), out_bias=cb.to(BF)))
    save("matmul", cases)

    # ---- _rms_norm_forward (:672), mean_dim (:385), log_softmax (:295)
    cases = []
    for (rows, n) in [(5, 2048), (3, 128), (2, 1000), (4, 512)]:
        x = torch.randn(rows, n, generator=g).to(BF)
        w = (1 + 0.02 * torch.randn(n, generator=g)).to(BF)
        # fp32 tensors holding the bf16 values: the kernel's final cast is then a no-op and the
        # single rounding to bf16 is done here with round-to-nearest-even (the interpreter's own
        # fp32->bf16 cast truncates, unlike the compiled kernel)
        y = bio._rms_norm_forward(x.float(), w.float(), 1e-6)
        cases.append(dict(x=x, w=w, eps=1e-6, out=y.to(BF), out_fp32=y))
    save("rms_norm_single", cases)

    cases = []
    for (rows, n) in [(6, 2048), (5, 128), (3, 777)]:
        x = torch.randn(rows, n, generator=g)
        # mean_dim asserts a CUDA tensor; launch the kernel the way the wrapper does (:456-471)
        out = torch.empty(rows)
        x3 = x.reshape(rows, n, 1)
        o2 = out.reshape(rows, 1)
        bio.mean_kernel[(rows,)](x3, o2, x3.stride(0), x3.stride(1), x3.stride(2), o2.stride(0), o2.stride(1),
                                 rows, n, 1, 1024)
        cases.append(dict(x=x, out=out))
    save("mean_lastdim", cases)

    cases = []
    for (rows, n) in [(4, 1000), (1, 151936), (3, 4097)]:
        x = torch.randn(rows, n, generator=g) * 2
        cases.append(dict(x=x, out=bio.log_softmax(x)))
    save("log_softmax", cases)

    # ---- HF eager RMSNorm and rotary embedding (what Qwen3 runs between the reference's ops)
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RMSNorm, apply_rotary_pos_emb
    cases = []
    for (rows, n) in [(5, 2048), (7, 128)]:
        x = torch.randn(rows, n, generator=g).to(BF)
        mod = Qwen3RMSNorm(n, eps=1e-6).to(BF)
        mod.weight.data = (1 + 0.02 * torch.randn(n, generator=g)).to(BF)
        cases.append(dict(x=x, w=mod.weight.data.clone(), eps=1e-6, out=mod(x)))
    save("rms_norm_hf", cases)

    from transformers import Qwen3Config
    from transformers.models.qwen3.modeling_qwen3 import Qwen3RotaryEmbedding
    cfg = Qwen3Config(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                      rope_theta=1e6, num_hidden_layers=1, intermediate_size=64, vocab_size=32)
    rot = Qwen3RotaryEmbedding(cfg)
    T = 9
    pos = torch.tensor([[0, 1, 2, 17, 100, 1023, 2047, 4096, 8191]])
    q = torch.randn(1, 2, T, 128, generator=g).to(BF)
    k = torch.randn(1, 1, T, 128, generator=g).to(BF)
    cos, sin = rot(q, pos)
    qe, ke = apply_rotary_pos_emb(q, k, cos, sin)
    save("rope", dict(q=q, k=k, positions=pos[0], theta=1e6, cos=cos[0], sin=sin[0], q_out=qe, k_out=ke))

    # ---- store_kvcache (kv_cache_context.py:294) through the kernel (:260)
    import vexact.batch_invariant_ops.kv_cache_context as kvc
    N, H, D, blocks, page = 6, 2, 128, 4, 16
    key = torch.randn(N, H, D, generator=g)
    val = torch.randn(N, H, D, generator=g)
    kc = torch.zeros(blocks, page, H, D)
    vc = torch.zeros(blocks, page, H, D)
    slots = torch.tensor([5, -1, 63, 0, 17, 32], dtype=torch.int32)
    kvc.store_kvcache(key, val, kc, vc, slots)
    save("kv_store", dict(key=key.to(BF), value=val.to(BF), slots=slots, k_cache=kc.to(BF), v_cache=vc.to(BF)))

    from types import SimpleNamespace as NS
    mgr = kvc.KVCacheManager(NS(max_cache_blocks=8, page_size=16))
    a1 = mgr.allocate_blocks(40)             # 3 blocks
    a2 = mgr.allocate_blocks(30)             # 2 blocks
    mgr.free_blocks(a1[:2])
    a3 = mgr.allocate_blocks(70, num_current_blocks=2)   # 3 more
    a4 = mgr.allocate_blocks(16 * 9)         # cannot be satisfied -> None
    save("kv_manager", dict(a1=a1, a2=a2, a3=a3, a4=a4, free=mgr.num_free_blocks(),
                            allocated=mgr.num_allocated_blocks()))

    # ---- paged attention kernel (triton_invariant_attention.py:434) launched as :651-693 does
    import vexact.batch_invariant_ops.triton_invariant_attention as tia
    from batch_invariant_ops.test_triton_attention_varlen import _eager_attention
    cases = []
    for (q_lens, kv_lens, hq, hkv, d, page) in [
        ([1, 1, 1], [5, 64, 77], 8, 1, 128, 16),       # decode, GQA 8
        ([4, 1, 9], [4, 33, 70], 4, 2, 128, 16),       # prefill / decode / chunk, GQA 2
        ([3, 1], [40, 19], 6, 1, 128, 64),             # GQA 6, page 64
    ]:
        S = len(q_lens)
        max_pages = max((kl + page - 1) // page for kl in kv_lens)
        nblocks = S * max_pages + 2
        perm = torch.randperm(nblocks, generator=g)
        kcache = bfvals(nblocks, page, hkv, d, gen=g)
        vcache = bfvals(nblocks, page, hkv, d, gen=g)
        ptab = torch.full((S, max_pages), -1, dtype=torch.int32)
        nxt = 0
        for s in range(S):
            for pg in range((kv_lens[s] + page - 1) // page):
                ptab[s, pg] = perm[nxt]
                nxt += 1
        qtot = sum(q_lens)
        q = bfvals(qtot, hq, d, gen=g)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
        used = torch.tensor(kv_lens, dtype=torch.int32)
        o = torch.empty(qtot, hq, d)
        scale = d ** -0.5
        block_m, block_n = 128, 64
        grid = (S, triton.cdiv(max_pages * page, block_m), hq)
        tia._paged_attn_fwd_block_kernel[grid](
            q, kcache, vcache, o, cu, used, ptab,
            q.stride(0), q.stride(1), q.stride(2),
            kcache.stride(0), kcache.stride(1), kcache.stride(2), kcache.stride(3),
            vcache.stride(0), vcache.stride(1), vcache.stride(2), vcache.stride(3),
            o.stride(0), o.stride(1), o.stride(2),
            ptab.stride(0), ptab.stride(1),
            scale, page, hq, hkv, d, d, True,
            BF16_OUTPUT=False, FP32_OUTPUT=True, BLOCK_M=block_m, BLOCK_N=block_n, BLOCK_D=128,
        )
        # the reference tests' own fp32 ground truth, per sequence
        eager = torch.empty(qtot, hq, d)
        for s in range(S):
            ks = torch.stack([kcache[ptab[s, p // page], p % page] for p in range(kv_lens[s])])
            vs = torch.stack([vcache[ptab[s, p // page], p % page] for p in range(kv_lens[s])])
            eager[cu[s]:cu[s + 1]] = _eager_attention(q[cu[s]:cu[s + 1]], ks, vs, scale)
        cases.append(dict(q=q.to(BF), k_cache=kcache.to(BF), v_cache=vcache.to(BF), cu_seqlens_q=cu,
                          seqused_k=used, page_table=ptab, scale=scale, p_dtype="fp32",
                          out_triton_fp32=o, out_eager_fp32=eager))
    save("paged_attention", cases)

    # ---- Qwen3-MoE routing (modeling_qwen3_moe.py:128-134), executed line for line on CPU
    import torch.nn.functional as F
    cases = []
    for (T, E, k) in [(16, 128, 8), (5, 64, 6)]:
        logits = (torch.randn(T, E, generator=g) * 0.9).to(BF)
        rw = F.softmax(logits, dim=1, dtype=torch.float)
        rw, sel = torch.topk(rw, k, dim=-1)
        rw /= rw.sum(dim=-1, keepdim=True)
        rw = rw.to(BF)
        cases.append(dict(logits=logits, top_k=k, weights=rw, experts=sel))
    save("route_softmax_topk", cases)

    # ---- DeepSeek-V3 routing (modeling_deepseek_v3.py:185-208) through the reference class
    try:
        from types import SimpleNamespace
        import vexact.models.deepseek_v3.modeling_deepseek_v3 as ds
        cases = []
        for (T, E, ng, tg, k) in [(12, 64, 8, 4, 6), (7, 64, 1, 1, 6)]:
            logits = torch.randn(T, E, generator=g)
            bias = torch.randn(E, generator=g) * 0.1
            fake = SimpleNamespace(gate=SimpleNamespace(e_score_correction_bias=bias), n_group=ng, topk_group=tg,
                                   n_routed_experts=E, norm_topk_prob=True, routed_scaling_factor=2.5, top_k=k)
            idx, w = ds.PatchDeepseekV3MoE.route_tokens_to_experts(fake, logits.clone())
            cases.append(dict(logits=logits, bias=bias, n_group=ng, topk_group=tg, top_k=k, scale=2.5,
                              experts=idx, weights=w))
        save("route_sigmoid_group_topk", cases)
    except Exception as e:
        print("deepseek routing skipped:", repr(e))

    # ---- MoE index build (fused_moe.py:280-292; the histogram is a bincount, its Triton kernel
    #      needs a GPU context) and moe_gather / moe_scatter kernels (group_gemm/kernel/moe.py)
    T, k, E, H = 12, 4, 8, 64
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    flat = sel.flatten()
    sorted_order = flat.argsort(stable=True)
    scatter_index = sorted_order.argsort().int().view(sel.shape)
    a_idx = (sorted_order // k).int()
    cu = torch.zeros(E + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.bincount(flat, minlength=E), 0).int()
    save("moe_indices", dict(experts=sel, num_experts=E, cu_seqlens=cu, a_idx=a_idx, scatter_index=scatter_index))

    # ---- naive expert arithmetic (modeling_qwen3_moe.py:76-80) for the MoE tolerance test
    I = 32
    hidden = (torch.randn(T, H, generator=g)).to(BF)
    gate_up = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(BF)
    down = (torch.randn(E, H, I, generator=g) * 0.05).to(BF)
    rw = torch.rand(T, k, generator=g)
    rw = (rw / rw.sum(-1, keepdim=True)).to(BF)
    out = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(sel[t, j])
            gu = torch.matmul(hidden[t:t + 1].float(), gate_up[e].float().t())
            gt, up = gu.chunk(2, dim=-1)
            hmid = F.silu(gt) * up
            out[t] += (torch.matmul(hidden.new_tensor(hmid).float(), down[e].float().t()) * rw[t, j].float())[0]
    save("moe_naive", dict(hidden=hidden, gate_up=gate_up, down=down, experts=sel, weights=rw, out_fp32=out))

    # ---- pipeline layer split (model_loader.py:141)
    os.environ["VEXACT_DISABLE_MODEL_PATCH"] = "1"
    try:
        from vexact.inferencer.model_loader import get_pp_indices
        table = {}
        for L in (27, 28, 48):
            for pp in (1, 2, 4, 8):
                table[(L, pp)] = [get_pp_indices(L, r, pp) for r in range(pp)]
        save("pp_indices", table)
    except Exception as e:
        print("pp_indices skipped:", repr(e))


if __name__ == "__main__":
    main()
