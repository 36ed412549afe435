"""CPU decoder-stack forward in plain torch ops.  TEST INFRASTRUCTURE / TIMED CPU BASELINE ONLY.

This is the reference's CPU-executable path for the rollout forward: the HF Qwen3 / Qwen2 /
Qwen3-MoE layer arithmetic with plain `torch.mm` (bf16), the HF RMSNorm formula, rotary
embedding, eager fp32 attention over the paged cache
(tests/batch_invariant_ops/test_triton_attention_varlen.py:52-72), the Qwen3-MoE routing
(vexact/models/qwen3_moe/modeling_qwen3_moe.py:128-134) and the per-expert loop
(modeling_qwen3_moe.py:76-80).  The reference's Triton overrides cannot run on a CPU.

Used by tests (small shapes, compared with the CUDA stage runner) and by bench.py's
`cpu_baseline` / `--impl reference` legs.  Never imported by the product package.
"""
from __future__ import annotations

import torch

from . import ops

BF = torch.bfloat16


def _linear(x, w, b=None):
    if b is not None:
        return torch.addmm(b, x, w.t())
    return torch.mm(x, w.t())


def attention_eager(q, k_cache, v_cache, cu, used, ptab, scale):
    """Eager fp32 causal attention over the paged cache, vectorised per sequence."""
    total_q, hq, d = q.shape
    hkv = k_cache.shape[2]
    g = hq // hkv
    page = k_cache.shape[1]
    out = torch.zeros((total_q, hq, v_cache.shape[-1]), dtype=q.dtype)
    for s in range(len(used)):
        q0, q1 = int(cu[s]), int(cu[s + 1])
        qlen, kvlen = q1 - q0, int(used[s])
        if qlen <= 0 or kvlen <= 0:
            continue
        npages = (kvlen + page - 1) // page
        blocks = ptab[s, :npages].long()
        k = k_cache[blocks].reshape(npages * page, hkv, -1)[:kvlen].float()
        v = v_cache[blocks].reshape(npages * page, hkv, -1)[:kvlen].float()
        k = k.permute(1, 0, 2).repeat_interleave(g, dim=0)      # [hq, kv, d]
        v = v.permute(1, 0, 2).repeat_interleave(g, dim=0)
        qs = q[q0:q1].float().permute(1, 0, 2)                   # [hq, q, d]
        sc = torch.matmul(qs, k.transpose(-1, -2)) * scale
        pos = torch.arange(kvlen - qlen, kvlen)
        mask = torch.arange(kvlen)[None, :] > pos[:, None]
        sc = sc.masked_fill(mask[None], float("-inf"))
        p = torch.softmax(sc, dim=-1).to(q.dtype).float()
        out[q0:q1] = torch.matmul(p, v).permute(1, 0, 2).to(q.dtype)
    return out


def moe_block(x, router_w, gate_up, down, top_k, norm_topk_prob):
    """Routing + per-expert loop, index_add accumulation as the eager model code does."""
    logits = _linear(x, router_w)
    rw, sel = ops.route_softmax_topk(logits, top_k, norm_topk_prob, x.dtype)
    out = torch.zeros_like(x)
    E = router_w.shape[0]
    I = gate_up.shape[1] // 2
    for e in range(E):
        tok, slot = torch.where(sel == e)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        gu = torch.mm(xe, gate_up[e].t())
        h = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        y = torch.mm(h, down[e].t()) * rw[tok, slot, None]
        out.index_add_(0, tok, y.to(out.dtype))
    return out


def _norm(shape, x, w):
    if getattr(shape, "norm_single_round", False):
        return ops.rms_norm_single_round(x, w, shape.rms_eps)   # DeepSeek-V3: batch_invariant_rms_norm
    return ops.rms_norm_hf(x, w, shape.rms_eps)


def rope_interleave(x, cos, sin):
    """transformers apply_rotary_pos_emb_interleave for x [T, heads, d]: de-interleave the pairs,
    then (x * cos) + (rotate_half(x) * sin) in bf16 arithmetic."""
    T, hds, d = x.shape
    x = x.view(T, hds, d // 2, 2).transpose(3, 2).reshape(T, hds, d)
    return ops.apply_rope(x, cos, sin)


def mla_qkv(shape, lw, xn, positions):
    """vexact/models/deepseek_v3/modeling_deepseek_v3.py:234-261 (q_lora_rank = None): returns
    query [T, heads, nope + rope], key [T, heads, nope + rope], value [T, heads, v]."""
    a = shape.mla
    T, heads = xn.shape[0], shape.num_q_heads
    q = _linear(xn, lw["qkv"]).view(T, heads, a.qk_nope + a.qk_rope)
    q_pass, q_rot = torch.split(q, [a.qk_nope, a.qk_rope], dim=-1)
    ckv = _linear(xn, lw["kv_a"])
    k_lat, k_rot = torch.split(ckv, [a.kv_lora_rank, a.qk_rope], dim=-1)
    kvb = _linear(ops.rms_norm_single_round(k_lat, lw["kv_a_norm"], shape.rms_eps), lw["kv_b"])
    kvb = kvb.view(T, heads, a.qk_nope + a.v_head)
    k_pass, v = torch.split(kvb, [a.qk_nope, a.v_head], dim=-1)
    cos, sin, _ = ops.rope_cos_sin(positions, a.qk_rope, shape.rope_theta, xn.dtype)
    q_rot = rope_interleave(q_rot.contiguous(), cos, sin)
    k_rot = rope_interleave(k_rot.reshape(T, 1, a.qk_rope).contiguous(), cos, sin).expand(T, heads, a.qk_rope)
    return torch.cat((q_pass, q_rot), dim=-1), torch.cat((k_pass, k_rot), dim=-1), v.contiguous()


def dsv3_moe_block(shape, lw, x):
    """PatchDeepseekV3MoE.forward (modeling_deepseek_v3.py:210-218): fp32 router, sigmoid group
    routing, per-expert loop (eager branch :127-143), plus the shared experts."""
    m = shape.moe
    logits = torch.nn.functional.linear(x.float(), lw["router"].float())
    idx, w = ops.route_sigmoid_group_topk(logits, lw.get("router_bias"), m.n_group, m.topk_group, m.top_k,
                                          m.norm_topk_prob, m.routed_scaling_factor)
    w = w.to(x.dtype)
    out = torch.zeros_like(x)
    I = m.intermediate
    for e in range(m.num_experts):
        tok, slot = torch.where(idx == e)
        if tok.numel() == 0:
            continue
        gu = torch.mm(x[tok], lw["experts_gate_up"][e].t())
        hmid = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        y = torch.mm(hmid, lw["experts_down"][e].t()) * w[tok, slot, None]
        out.index_add_(0, tok, y.to(out.dtype))
    if lw.get("shared_gate_up") is not None:
        si = lw["shared_gate_up"].shape[0] // 2
        gu = _linear(x, lw["shared_gate_up"])
        out = out + _linear(torch.nn.functional.silu(gu[:, :si]) * gu[:, si:], lw["shared_down"])
    return out


def layer_forward(shape, lw, h, positions, slots, k_cache, v_cache, cu, used, ptab):
    """One decoder layer; `lw` holds CPU tensors with the names of vexact_b200.inferencer.LayerWeights."""
    T = h.shape[0]
    xn = _norm(shape, h, lw["input_norm"])
    if getattr(shape, "mla", None) is not None:
        q, k, v = mla_qkv(shape, lw, xn, positions)
        scale = q.shape[-1] ** -0.5
    else:
        qkv = _linear(xn, lw["qkv"], lw.get("qkv_bias"))
        q, k, v = ops.qknorm_rope(qkv, positions, shape.num_q_heads, shape.num_kv_heads, shape.head_dim,
                                  lw.get("q_norm"), lw.get("k_norm"), shape.rope_theta, shape.rms_eps)
        scale = shape.head_dim ** -0.5
    ops.kv_store(k.contiguous(), v.contiguous(), k_cache, v_cache, slots)
    attn = attention_eager(q, k_cache, v_cache, cu, used, ptab, scale)
    h = h + _linear(attn.reshape(T, -1), lw["o"])
    xn = _norm(shape, h, lw["post_norm"])
    if lw.get("router") is not None:
        m = shape.moe
        if m.scoring == "sigmoid_group":
            delta = dsv3_moe_block(shape, lw, xn)
        else:
            delta = moe_block(xn, lw["router"], lw["experts_gate_up"], lw["experts_down"], m.top_k, m.norm_topk_prob)
    else:
        ffn = lw["gate_up"].shape[0] // 2
        gu = _linear(xn, lw["gate_up"])
        act = torch.nn.functional.silu(gu[:, :ffn]) * gu[:, ffn:]
        delta = _linear(act, lw["down"])
    return h + delta


def head_forward(shape, final_norm, lm_head, h_last):
    xn = _norm(shape, h_last, final_norm)
    logits = _linear(xn, lm_head)
    tokens = logits.argmax(-1)
    return tokens, ops.gather_logprob(logits, tokens), logits
