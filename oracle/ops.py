"""CPU oracle for the rollout-forward hot path.  TEST INFRASTRUCTURE ONLY.

Each function restates, with torch CPU tensors (bf16 rounding needs a bf16 type;
all index work is integer-exact), what the cited reference code computes.  Paths
are relative to the verl-project/vexact tree.

Pinning: every function here is checked against fixtures under tests/golden/
(tests/test_oracle_golden.py), of two kinds.  (1) tests/golden/make_golden.py ran the
reference's own Triton kernels under the Triton CPU interpreter and the reference's
torch-level model code on CPU.  (2) tests/golden/make_reference_gpu_golden.py ran the
reference's compiled kernels on a B200 with bf16 operands (ref_gpu_*.pt): its Triton GEMM,
norms, log-softmax, KV store and paged attention (P really rounded to bf16), flash-attn's
cross entropy, and the fused-MoE expert arithmetic through both of the reference's expert
functions (Triton and quack), which is what the model files' call to
`veomni.ops.fused_moe_forward` (veomni @ a4ed599, not vendored) is bound to
(vexact/models/register.py:40-57).
"""
from __future__ import annotations

import numpy as np
import torch

BF16 = torch.bfloat16


def _bf(x: torch.Tensor) -> torch.Tensor:
    """Round to bf16 and return as fp32 (a bf16 tensor materialised between two ops)."""
    return x.to(BF16).float()


# ----------------------------------------------------------------------------- matmul
def matmul(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """vexact/batch_invariant_ops/batch_invariant_ops.py:104-131: fp32 accumulation over K,
    bias added in fp32 before the cast to the output dtype."""
    acc = a.float() @ b.float()
    if bias is not None:
        acc = acc + bias.float()
    return acc.to(a.dtype)


# ----------------------------------------------------------------------------- norms
def rms_norm_single_round(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """batch_invariant_ops.py:653-669: inv = 1/sqrt(sum(x^2)/n + eps); out = (x*inv*w) rounded once."""
    xf = x.float()
    inv = 1.0 / torch.sqrt(xf.pow(2).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return (xf * inv * w.float()).to(x.dtype)


def rms_norm_hf(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """transformers Qwen3RMSNorm.forward (modeling_qwen3.py:59-64): the normalised value is cast
    to the input dtype, then multiplied by the weight (a bf16 x bf16 product)."""
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    normed = (xf * torch.rsqrt(var + eps)).to(x.dtype)
    return w * normed


def mean_lastdim(x: torch.Tensor) -> torch.Tensor:
    """batch_invariant_ops.py:365-381: sum over the reduced dim (fp32), divided by its length."""
    return (x.float().sum(-1) / x.shape[-1]).to(x.dtype)


# ----------------------------------------------------------------------------- softmax / logprob
def log_softmax(x: torch.Tensor) -> torch.Tensor:
    """batch_invariant_ops.py:251-291: x - max - log(sum(exp(x - max)))."""
    xf = x.float()
    m = xf.max(-1, keepdim=True).values
    s = torch.exp(xf - m).sum(-1, keepdim=True)
    return (xf - m - torch.log(s)).to(x.dtype)


def gather_logprob(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """flash_attn/ops/triton/cross_entropy.py:52-81 as called by
    vexact/batch_invariant_ops/standalone_logprobs.py:50: loss = lse - x[label], logprob = -loss,
    0 for ignored labels."""
    xf = logits.float()
    m = xf.max(-1, keepdim=True).values
    lse = (torch.log(torch.exp(xf - m).sum(-1, keepdim=True)) + m).squeeze(-1)
    safe = labels.clamp(min=0)
    picked = xf.gather(-1, safe.unsqueeze(-1)).squeeze(-1)
    out = picked - lse
    return torch.where(labels == ignore_index, torch.zeros_like(out), out)


# ----------------------------------------------------------------------------- paged KV
def slot_mapping(block_ids_per_req, start_pos_per_req, tokens_per_req, page_size: int) -> np.ndarray:
    """vexact/inferencer/inferencer.py:208-221: slot = block_ids[pos // page] * page + pos % page."""
    out = []
    for blocks, start, n in zip(block_ids_per_req, start_pos_per_req, tokens_per_req):
        for pos in range(start, start + n):
            out.append(blocks[pos // page_size] * page_size + pos % page_size)
    return np.asarray(out, dtype=np.int32)


def kv_store(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             slots: torch.Tensor) -> None:
    """vexact/batch_invariant_ops/kv_cache_context.py:269-276: row i -> flat slot slots[i]; -1 skips."""
    kc = k_cache.view(-1, k_cache.shape[-2] * k_cache.shape[-1])
    vc = v_cache.view(-1, v_cache.shape[-2] * v_cache.shape[-1])
    for i, s in enumerate(slots.tolist()):
        if s == -1:
            continue
        kc[s] = key[i].reshape(-1)
        vc[s] = value[i].reshape(-1)


def gather_paged(cache: torch.Tensor, page_table_row, kv_len: int) -> torch.Tensor:
    """Contiguous [kv_len, heads, dim] view of one sequence's cached tokens."""
    page = cache.shape[1]
    rows = []
    for pos in range(kv_len):
        rows.append(cache[page_table_row[pos // page], pos % page])
    return torch.stack(rows) if rows else cache.new_zeros((0,) + cache.shape[2:])


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_seqlens_q, seqused_k,
                    page_table, scale: float, block_n: int | None = None) -> torch.Tensor:
    """Causal attention of packed queries over a paged cache.

    block_n=None: the fp32 eager form the reference tests against
    (tests/batch_invariant_ops/test_triton_attention_varlen.py:52-72).
    block_n=k: the blocked online-softmax form of
    vexact/batch_invariant_ops/triton_invariant_attention.py:497-596 (base-2 exponent with
    scale*log2(e) folded in, P rounded to the activation dtype before the PV product and
    before the row sum, keys walked from 0 in blocks of k).
    """
    total_q, hq, dk = q.shape
    hkv = k_cache.shape[2]
    dv = v_cache.shape[-1]
    g = hq // hkv
    out = torch.zeros((total_q, hq, dv), dtype=q.dtype)
    cu = [int(v) for v in cu_seqlens_q]
    for s in range(len(cu) - 1):
        q0, q1 = cu[s], cu[s + 1]
        qlen, kvlen = q1 - q0, int(seqused_k[s])
        if qlen <= 0 or kvlen <= 0:
            continue
        k = gather_paged(k_cache, [int(v) for v in page_table[s]], kvlen).float()  # [kv, hkv, dk]
        v = gather_paged(v_cache, [int(v) for v in page_table[s]], kvlen).float()
        for h in range(hq):
            kh, vh = k[:, h // g], v[:, h // g]
            qh = q[q0:q1, h].float()
            pos = torch.arange(kvlen - qlen, kvlen)
            if block_n is None:
                sc = qh @ kh.T * scale
                mask = torch.arange(kvlen)[None, :] > pos[:, None]
                sc = sc.masked_fill(mask, float("-inf"))
                o = torch.softmax(sc, -1) @ vh
            else:
                qk_scale = np.float32(scale) * np.float32(1.44269504)
                m = torch.full((qlen,), float("-inf"))
                l = torch.zeros(qlen)
                acc = torch.zeros(qlen, dv)
                for n0 in range(0, kvlen, block_n):
                    n1 = min(n0 + block_n, kvlen)
                    sc = (qh @ kh[n0:n1].T) * float(qk_scale)
                    mask = torch.arange(n0, n1)[None, :] > pos[:, None]
                    sc = sc.masked_fill(mask, float("-inf"))
                    m_new = torch.maximum(m, sc.max(-1).values)
                    live = torch.isfinite(m_new)
                    m_safe = torch.where(live, m_new, torch.zeros_like(m_new))
                    p = _bf(torch.exp2(sc - m_safe[:, None]))
                    alpha = torch.where(torch.isfinite(m), torch.exp2(m - m_safe), torch.zeros_like(m))
                    acc = acc * alpha[:, None] + p @ vh[n0:n1]
                    l = l * alpha + p.sum(-1)
                    m = m_new
                o = acc / l[:, None]
            out[q0:q1, h] = o.to(q.dtype)
    return out


# ----------------------------------------------------------------------------- rotary / qk norm
def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, dtype=BF16):
    """transformers Qwen3RotaryEmbedding.forward: inv_freq = 1/theta^(2i/d) (fp32),
    freqs = pos * inv_freq, emb = cat(freqs, freqs), cos/sin cast to the activation dtype."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    freqs = positions.float()[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype), inv_freq


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """transformers apply_rotary_pos_emb in bf16 arithmetic: (x*cos) + (rotate_half(x)*sin),
    x [T, heads, d], cos/sin [T, d]."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return (x * cos[:, None, :]) + (rot * sin[:, None, :])


def qknorm_rope(qkv: torch.Tensor, positions: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int,
                q_norm_w, k_norm_w, theta: float, eps: float):
    """HF Qwen3Attention.forward between the projections and the attention call: per-head RMSNorm
    of q and k (if the model has it), then rotary embedding.  Returns q, k, v as [T, heads, d]."""
    T = qkv.shape[0]
    q, k, v = qkv.split([num_q_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * head_dim], dim=-1)
    q = q.reshape(T, num_q_heads, head_dim)
    k = k.reshape(T, num_kv_heads, head_dim)
    v = v.reshape(T, num_kv_heads, head_dim)
    if q_norm_w is not None:
        q = rms_norm_hf(q, q_norm_w, eps)
        k = rms_norm_hf(k, k_norm_w, eps)
    cos, sin, _ = rope_cos_sin(positions, head_dim, theta, qkv.dtype)
    return apply_rope(q, cos, sin), apply_rope(k, cos, sin), v


# ----------------------------------------------------------------------------- MoE routing
def route_softmax_topk(router_logits: torch.Tensor, top_k: int, norm_topk_prob: bool, out_dtype=BF16):
    """vexact/models/qwen3_moe/modeling_qwen3_moe.py:128-134.  Ties go to the lower expert index
    (a stable descending sort), which is what torch.topk does on CPU for distinct values and the
    convention of the CUDA kernel."""
    probs = torch.softmax(router_logits.float(), dim=1)
    order = torch.sort(probs, dim=-1, descending=True, stable=True)
    w = order.values[:, :top_k].clone()
    idx = order.indices[:, :top_k].clone()
    if norm_topk_prob:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.to(out_dtype), idx


def route_sigmoid_group_topk(router_logits: torch.Tensor, bias, n_group: int, topk_group: int, top_k: int,
                             norm_topk_prob: bool, scale: float):
    """vexact/models/deepseek_v3/modeling_deepseek_v3.py:185-208, selected experts listed in
    descending choice-score order with ties to the lower index."""
    s = router_logits.float().sigmoid()
    choice = s + (bias.float() if bias is not None else 0.0)
    T, E = s.shape
    gs = choice.view(T, n_group, E // n_group).topk(2, dim=-1)[0].sum(dim=-1)
    g_order = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :topk_group]
    gmask = torch.zeros_like(gs)
    gmask.scatter_(1, g_order, 1)
    smask = gmask.unsqueeze(-1).expand(-1, n_group, E // n_group).reshape(T, E)
    masked = choice.masked_fill(~smask.bool(), 0.0)
    idx = torch.sort(masked, dim=-1, descending=True, stable=True).indices[:, :top_k]
    w = s.gather(1, idx)
    if norm_topk_prob:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    return idx, w * scale


def build_moe_indices(expert_index: torch.Tensor, num_experts: int):
    """vexact/batch_invariant_ops/fused_moe.py:280-292: stable argsort by expert, inverse
    permutation, token index of each sorted row, histogram, cumulative sum.  Pure numpy ints."""
    e = expert_index.numpy().astype(np.int64)
    topk = e.shape[1]
    flat = e.reshape(-1)
    sorted_order = np.argsort(flat, kind="stable")
    scatter_index = np.empty_like(sorted_order)
    scatter_index[sorted_order] = np.arange(flat.size)
    a_idx = (sorted_order // topk).astype(np.int32)
    splits = np.bincount(flat, minlength=num_experts)
    cu = np.zeros(num_experts + 1, dtype=np.int32)
    cu[1:] = np.cumsum(splits)
    return cu, a_idx, scatter_index.astype(np.int32).reshape(e.shape)


def silu_bf16(x: torch.Tensor) -> torch.Tensor:
    """torch.ops.aten.silu on a bf16 tensor: x / (1 + exp(-x)) in fp32, one rounding."""
    xf = x.float()
    return (xf / (1.0 + torch.exp(-xf))).to(BF16)


def fused_moe(num_experts: int, routing_weights: torch.Tensor, selected_experts: torch.Tensor,
              hidden: torch.Tensor, fc1_1: torch.Tensor, fc1_2: torch.Tensor, fc2: torch.Tensor) -> torch.Tensor:
    """vexact/batch_invariant_ops/fused_moe.py:299-344 (QuackFusedMoeExpertFunction.forward):
    per-expert GEMMs with bf16 outputs, silu (bf16), gate*up (bf16), * routing weight (bf16),
    fc2 (bf16), then moe_gather: fp32 sum over the k rows of a token in k order, one cast
    (group_gemm/kernel/moe.py:111-128)."""
    T, H = hidden.shape
    k = selected_experts.shape[1]
    rw = routing_weights.to(BF16)
    x = hidden.to(BF16)
    rows = torch.zeros((T, k, H), dtype=BF16)
    for t in range(T):
        for j in range(k):
            e = int(selected_experts[t, j])
            g = matmul(x[t:t + 1], fc1_1[e].t())
            u = matmul(x[t:t + 1], fc1_2[e].t())
            act = silu_bf16(g) * u
            act = act * rw[t, j]
            rows[t, j] = matmul(act, fc2[e].t())[0]
    acc = torch.zeros((T, H), dtype=torch.float32)
    for j in range(k):
        acc = acc + rows[:, j].float()
    return acc.to(BF16)


def fused_moe_batched(num_experts: int, routing_weights, selected_experts, hidden, fc1_1, fc1_2, fc2):
    """Same arithmetic as `fused_moe`, one matmul per expert (faster for larger cases)."""
    T, H = hidden.shape
    k = selected_experts.shape[1]
    rw = routing_weights.to(BF16)
    x = hidden.to(BF16)
    rows = torch.zeros((T, k, H), dtype=BF16)
    for e in range(num_experts):
        tok, slot = torch.where(selected_experts == e)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        g = matmul(xe, fc1_1[e].t())
        u = matmul(xe, fc1_2[e].t())
        act = silu_bf16(g) * u
        act = act * rw[tok, slot].unsqueeze(-1)
        rows[tok, slot] = matmul(act, fc2[e].t())
    acc = torch.zeros((T, H), dtype=torch.float32)
    for j in range(k):
        acc = acc + rows[:, j].float()
    return acc.to(BF16)


def get_pp_indices(num_hidden_layers: int, pp_rank: int, pp_size: int) -> tuple[int, int]:
    """vexact/inferencer/model_loader.py:141-171: even split, remainder spread over the
    ranks from the second-to-last one backwards."""
    layers_per = num_hidden_layers // pp_size
    parts = [layers_per for _ in range(pp_size)]
    remaining = num_hidden_layers % pp_size
    if remaining:
        for i in range(2, remaining + 2):
            parts[-i] += 1
    start = sum(parts[:pp_rank])
    return start, start + parts[pp_rank]
