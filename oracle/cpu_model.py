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


def layer_forward(shape, lw, h, positions, slots, k_cache, v_cache, cu, used, ptab):
    """One decoder layer; `lw` holds CPU tensors with the names of vexact_b200.inferencer.LayerWeights."""
    T = h.shape[0]
    xn = ops.rms_norm_hf(h, lw["input_norm"], shape.rms_eps)
    qkv = _linear(xn, lw["qkv"], lw.get("qkv_bias"))
    q, k, v = ops.qknorm_rope(qkv, positions, shape.num_q_heads, shape.num_kv_heads, shape.head_dim,
                              lw.get("q_norm"), lw.get("k_norm"), shape.rope_theta, shape.rms_eps)
    ops.kv_store(k, v, k_cache, v_cache, slots)
    attn = attention_eager(q, k_cache, v_cache, cu, used, ptab, shape.head_dim ** -0.5)
    h = h + _linear(attn.reshape(T, -1), lw["o"])
    xn = ops.rms_norm_hf(h, lw["post_norm"], shape.rms_eps)
    if shape.moe is not None:
        m = shape.moe
        delta = moe_block(xn, lw["router"], lw["experts_gate_up"], lw["experts_down"], m.top_k, m.norm_topk_prob)
    else:
        gu = _linear(xn, lw["gate_up"])
        act = torch.nn.functional.silu(gu[:, :shape.ffn]) * gu[:, shape.ffn:]
        delta = _linear(act, lw["down"])
    return h + delta


def head_forward(shape, final_norm, lm_head, h_last):
    xn = ops.rms_norm_hf(h_last, final_norm, shape.rms_eps)
    logits = _linear(xn, lm_head)
    tokens = logits.argmax(-1)
    return tokens, ops.gather_logprob(logits, tokens), logits
