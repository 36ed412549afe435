"""Pipeline-stage forward for the rollout hot path.

Stands where the reference's `Inferencer._forward` + `TransformersForCausalLM.forward` +
`Inferencer._select_tokens` stand (vexact/inferencer/inferencer.py:352-449,
vexact/inferencer/model_loader.py:218-276, vexact/inferencer/cudagraph_utils.py:109-190):
one forward of the local decoder layers over a packed token batch with paged KV, then, on
the last stage, last-token gather, lm_head, greedy token and its log-probability.

The layer arithmetic is the HF Qwen3 / Qwen2 / Qwen3-MoE decoder layer with the reference's
operator overrides, op for op and rounding for rounding:
    h = h + o_proj(attn(rope(norm?(qkv(rmsnorm(h))))));  h = h + mlp_or_moe(rmsnorm(h))
with every matmul, norm, rope/store, attention, routing and expert GEMM a call into
libvexact_b200.so.  The whole stage forward is captured in a CUDA graph per token bucket
(static input buffers, replay per step), as the reference does.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import torch

from . import _lib
from .attention import paged_attention
from .batch_invariant_ops import add_rms_norm, batch_invariant_rms_norm, hf_rms_norm, linear, linear_f32_from_bf16
from .fused_moe import (TILE_ROWS, PendingMoE, _grouped_gemm, fused_moe_forward, route_plan_softmax_topk,
                        route_sigmoid_group_topk,
                        route_softmax_topk)
from .standalone_logprobs import greedy_token_and_logprob, lm_head_greedy
from .sampler import sample_token_and_logprob

BF = torch.bfloat16
# B200_MOE_ROUTE_PLAN=1: routing hands out the permutation itself (route -> scatter, two launches instead of
# route -> index -> scatter; same outputs bit for bit, rows of an expert's group in arrival order).  Off by
# default: inside the captured decode step it measured 0.0-0.5 % (32.04 -> 31.87-32.04 ms), within run-to-run
# noise, and the stable order is the simpler thing to reason about.
_ROUTE_PLAN = os.environ.get("B200_MOE_ROUTE_PLAN", "0") == "1"


@dataclass(frozen=True)
class MoEShape:
    num_experts: int
    top_k: int
    intermediate: int
    norm_topk_prob: bool = True
    # DeepSeek-V3 style routing (modeling_deepseek_v3.py:185-208) when scoring == "sigmoid_group"
    scoring: str = "softmax"
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    n_shared_experts: int = 0


@dataclass(frozen=True)
class MLAShape:
    """Multi-head latent attention dims (DeepSeek-V3 / Moonlight), q_lora_rank = None."""

    kv_lora_rank: int = 512
    qk_nope: int = 128
    qk_rope: int = 64
    v_head: int = 128


@dataclass(frozen=True)
class ModelShape:
    """The subset of an HF config the forward needs."""

    name: str
    num_layers: int
    hidden: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    vocab: int
    ffn: int = 0                      # dense SwiGLU width (0 for MoE layers)
    moe: Optional[MoEShape] = None
    qk_norm: bool = True
    qkv_bias: bool = False
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    mla: Optional[MLAShape] = None
    first_k_dense: int = 0            # leading layers with a dense FFN in an MoE model
    norm_single_round: bool = False   # DeepSeek-V3: every RMSNorm is batch_invariant_rms_norm

    @property
    def qkv_out(self) -> int:
        return (self.num_q_heads + 2 * self.num_kv_heads) * self.head_dim

    @property
    def k_dim(self) -> int:
        return self.mla.qk_nope + self.mla.qk_rope if self.mla else self.head_dim

    @property
    def v_dim(self) -> int:
        return self.mla.v_head if self.mla else self.head_dim

    def layer_is_moe(self, layer_idx: int) -> bool:
        return self.moe is not None and layer_idx >= self.first_k_dense


QWEN3_1P7B = ModelShape("qwen3-1.7b-shape", 28, 2048, 16, 8, 128, 151936, ffn=6144)
QWEN2_1P5B = ModelShape("qwen2-1.5b-shape", 28, 1536, 12, 2, 128, 151936, ffn=8960, qk_norm=False, qkv_bias=True)
QWEN3_30B_A3B = ModelShape("qwen3-30b-a3b-shape", 48, 2048, 32, 4, 128, 151936, moe=MoEShape(128, 8, 768))
# Moonlight-16B-A3B (DeepSeek-V3 architecture).  n_group / topk_group / scaling are not fixed by the
# benchmark description: 1 / 1 / 2.446 (Moonlight's published config) are used.
MOONLIGHT_16B_A3B = ModelShape(
    "moonlight-16b-a3b-shape", 27, 2048, 16, 16, 192, 163840, ffn=11264, qk_norm=False, rope_theta=50000.0,
    rms_eps=1e-5, mla=MLAShape(), first_k_dense=1, norm_single_round=True,
    moe=MoEShape(64, 6, 1408, True, "sigmoid_group", 1, 1, 2.446, 2))
PRESETS = {m.name: m for m in (QWEN3_1P7B, QWEN2_1P5B, QWEN3_30B_A3B, MOONLIGHT_16B_A3B)}


def get_pp_indices(num_hidden_layers: int, pp_rank: int, pp_size: int) -> tuple[int, int]:
    """Layer range of a pipeline rank; same rule as vexact/inferencer/model_loader.py:141-171."""
    per = num_hidden_layers // pp_size
    parts = [per] * pp_size
    rem = num_hidden_layers % pp_size
    for i in range(2, rem + 2):
        parts[-i] += 1
    start = sum(parts[:pp_rank])
    return start, start + parts[pp_rank]


def _randn(shape, std, device, gen):
    t = torch.empty(shape, device=device, dtype=BF)
    t.normal_(0.0, std, generator=gen)
    return t


@dataclass
class LayerWeights:
    input_norm: torch.Tensor
    qkv: torch.Tensor                  # [(hq + 2 hkv) * d, hidden]: q_proj, k_proj, v_proj stacked
    qkv_bias: Optional[torch.Tensor]
    q_norm: Optional[torch.Tensor]
    k_norm: Optional[torch.Tensor]
    o: torch.Tensor                    # [hidden, hq * d]
    post_norm: torch.Tensor
    gate_up: Optional[torch.Tensor] = None   # dense: [2 * ffn, hidden] (gate rows first)
    down: Optional[torch.Tensor] = None      # dense: [hidden, ffn]
    router: Optional[torch.Tensor] = None    # moe: [E, hidden]
    experts_gate_up: Optional[torch.Tensor] = None  # moe: [E, 2I, hidden]
    experts_down: Optional[torch.Tensor] = None     # moe: [E, hidden, I]
    router_bias: Optional[torch.Tensor] = None      # DeepSeek-V3 e_score_correction_bias [E] fp32
    router_logit_bias: Optional[torch.Tensor] = None  # softmax routing: bias of the router Linear [E] bf16
    shared_gate_up: Optional[torch.Tensor] = None   # shared experts: [2 * I * n_shared, hidden]
    shared_down: Optional[torch.Tensor] = None      # [hidden, I * n_shared]
    kv_a: Optional[torch.Tensor] = None             # MLA: kv_a_proj_with_mqa [kv_lora + rope, hidden]
    kv_a_norm: Optional[torch.Tensor] = None        # MLA: [kv_lora]
    kv_b: Optional[torch.Tensor] = None             # MLA: [heads * (nope + v), kv_lora]


@dataclass
class StageWeights:
    shape: ModelShape
    start_layer: int
    end_layer: int
    layers: list = field(default_factory=list)
    embed: Optional[torch.Tensor] = None      # first stage
    final_norm: Optional[torch.Tensor] = None  # last stage
    lm_head: Optional[torch.Tensor] = None     # last stage, [vocab, hidden]
    inv_freq: Optional[torch.Tensor] = None

    @staticmethod
    def random_init(shape: ModelShape, pp_rank: int = 0, pp_size: int = 1, device="cuda", seed: int = 0,
                    std: float = 0.02, norm_jitter: float = 0.0) -> "StageWeights":
        """Random weights ~ N(0, std) in bf16 (HF initializer_range), norm weights 1 (+ jitter)."""
        start, end = get_pp_indices(shape.num_layers, pp_rank, pp_size)
        gen = torch.Generator(device=device).manual_seed(seed * 1000 + pp_rank)
        w = StageWeights(shape, start, end)

        def norm_w(n):
            t = torch.ones(n, device=device, dtype=BF)
            if norm_jitter:
                t += _randn((n,), norm_jitter, device, gen)
            return t

        H, D = shape.hidden, shape.head_dim
        for li in range(start, end):
            if shape.mla is not None:
                a = shape.mla
                lw = LayerWeights(
                    input_norm=norm_w(H),
                    qkv=_randn((shape.num_q_heads * (a.qk_nope + a.qk_rope), H), std, device, gen),  # q_proj
                    qkv_bias=None, q_norm=None, k_norm=None,
                    o=_randn((H, shape.num_q_heads * a.v_head), std, device, gen),
                    post_norm=norm_w(H),
                    kv_a=_randn((a.kv_lora_rank + a.qk_rope, H), std, device, gen),
                    kv_a_norm=norm_w(a.kv_lora_rank),
                    kv_b=_randn((shape.num_q_heads * (a.qk_nope + a.v_head), a.kv_lora_rank), std, device, gen),
                )
            else:
                lw = LayerWeights(
                    input_norm=norm_w(H),
                    qkv=_randn((shape.qkv_out, H), std, device, gen),
                    qkv_bias=_randn((shape.qkv_out,), std, device, gen) if shape.qkv_bias else None,
                    q_norm=norm_w(D) if shape.qk_norm else None,
                    k_norm=norm_w(D) if shape.qk_norm else None,
                    o=_randn((H, shape.num_q_heads * D), std, device, gen),
                    post_norm=norm_w(H),
                )
            if shape.layer_is_moe(li):
                m = shape.moe
                lw.router = _randn((m.num_experts, H), std, device, gen)
                lw.experts_gate_up = _randn((m.num_experts, 2 * m.intermediate, H), std, device, gen)
                lw.experts_down = _randn((m.num_experts, H, m.intermediate), std, device, gen)
                if m.scoring == "sigmoid_group":
                    lw.router_bias = torch.zeros(m.num_experts, device=device, dtype=torch.float32)
                    if norm_jitter:
                        lw.router_bias.normal_(0.0, norm_jitter, generator=gen)
                if m.n_shared_experts:
                    si = m.intermediate * m.n_shared_experts
                    lw.shared_gate_up = _randn((2 * si, H), std, device, gen)
                    lw.shared_down = _randn((H, si), std, device, gen)
            else:
                lw.gate_up = _randn((2 * shape.ffn, H), std, device, gen)
                lw.down = _randn((H, shape.ffn), std, device, gen)
            w.layers.append(lw)
        if pp_rank == 0:
            w.embed = _randn((shape.vocab, H), std, device, gen)
        if pp_rank == pp_size - 1:
            w.final_norm = norm_w(H)
            w.lm_head = _randn((shape.vocab, H), std, device, gen)
        rd = shape.mla.qk_rope if shape.mla is not None else D
        w.inv_freq = (1.0 / (shape.rope_theta ** (torch.arange(0, rd, 2, dtype=torch.int64).float() / rd))).to(device)
        return w

    def num_bytes(self) -> int:
        n = 0
        for lw in self.layers:
            for t in vars(lw).values():
                if isinstance(t, torch.Tensor):
                    n += t.numel() * t.element_size()
        for t in (self.embed, self.final_norm, self.lm_head):
            if t is not None:
                n += t.numel() * t.element_size()
        return n


@dataclass
class StepInputs:
    """Device-side inputs of one stage forward (the fields of the reference's InputBuffers /
    GenerationContext that the kernels read, vexact/core/runtime_data.py:68-134)."""

    input_ids: Optional[torch.Tensor]        # [T] int64 (first stage)
    hidden_in: Optional[torch.Tensor]        # [T, H] bf16 (later stages)
    positions: torch.Tensor                  # [T] int64
    slot_mapping: torch.Tensor               # [T] int32, -1 = padded token
    query_start_loc: torch.Tensor            # [S + 1] int32
    context_lens: torch.Tensor               # [S] int32
    block_tables: torch.Tensor               # [S, max_blocks] int32
    max_seqlen_q: int
    seq_order: Optional[torch.Tensor] = None  # [S] int32, sequences by descending context (attention balance)


def _gather_rows(src: torch.Tensor, ids: Optional[torch.Tensor] = None,
                 query_start_loc: Optional[torch.Tensor] = None) -> torch.Tensor:
    """src[ids] (the embedding lookup) or each sequence's last-token row src[query_start_loc[1:] - 1]
    (inferencer.py:403-404; a zero-length padding sequence reads row 0), one kernel either way."""
    if src.dim() != 2 or src.dtype != BF or src.stride(1) != 1:
        raise ValueError("row gather expects a 2-D bf16 matrix with contiguous rows")
    if ids is not None:
        ids = ids.reshape(-1)
        if ids.dtype != torch.int64 or not ids.is_contiguous():
            ids = ids.to(torch.int64).contiguous()
        T = ids.numel()
    else:
        if query_start_loc.dtype != torch.int32 or not query_start_loc.is_contiguous():
            query_start_loc = query_start_loc.to(torch.int32).contiguous()
        T = query_start_loc.numel() - 1
    out = torch.empty((T, src.shape[1]), device=src.device, dtype=BF)
    _lib.check(_lib.load().b200_gather_rows(src.data_ptr(), src.shape[0], src.stride(0), _lib.ptr(ids),
                                            _lib.ptr(query_start_loc) if ids is None else None, out.data_ptr(), T,
                                            src.shape[1], _lib.current_stream()), "b200_gather_rows")
    return out


class StageRunner:
    """Runs the local layers of one pipeline stage; optionally through a captured CUDA graph."""

    def __init__(self, weights: StageWeights, key_cache: dict, value_cache: dict, pp_rank: int = 0,
                 pp_size: int = 1):
        self.w = weights
        self.shape = weights.shape
        self.key_cache = key_cache
        self.value_cache = value_cache
        self.pp_rank, self.pp_size = pp_rank, pp_size
        self.is_first = pp_rank == 0
        self.is_last = pp_rank == pp_size - 1
        self._graphs: dict = {}
        self._dense_tiles: dict = {}
        # None = greedy; else dict(temperature=..., top_k=..., top_p=...) applied to every request
        self.sampling: Optional[dict] = None
        # greedy decoding without the [num_seqs, vocab] logits: lm_head and token selection fused
        # (`select_tokens` then returns None for the logits)
        self.fused_head = False

    # -- dense MLP through the grouped-GEMM kernel's fused SwiGLU epilogue (one group)
    def _dense_plan(self, T: int, device):
        plan = self._dense_tiles.get(T)
        if plan is None:
            tile = TILE_ROWS
            rows = [(0, r, min(tile, T - r), 0) for r in range(0, T, tile)]
            plan = dict(tile_table=torch.tensor(rows, dtype=torch.int32, device=device),
                        tile_count=torch.tensor([len(rows)], dtype=torch.int32, device=device),
                        max_tiles=len(rows), tile_rows=tile)
            self._dense_tiles[T] = plan
        return plan

    def prepare(self, T: int, device="cuda") -> None:
        """Build host-constructed constants for a token count (call before graph capture)."""
        self._dense_plan(T, device)

    def _norm(self, x, w):
        s = self.shape
        return batch_invariant_rms_norm(x, w, s.rms_eps) if s.norm_single_round else hf_rms_norm(x, w, s.rms_eps)

    def _add_norm(self, x, residual, w):
        if isinstance(x, PendingMoE):   # the MoE's top-k sum joins the residual add and the norm
            return x.add_norm(residual, w, self.shape.rms_eps, hf=not self.shape.norm_single_round)
        return add_rms_norm(x, residual, w, self.shape.rms_eps, hf=not self.shape.norm_single_round)

    def _attention_block(self, lw: LayerWeights, layer_idx: int, xn: torch.Tensor, inp: StepInputs) -> torch.Tensor:
        s = self.shape
        T = xn.shape[0]
        kc, vc = self.key_cache[layer_idx], self.value_cache[layer_idx]
        if s.mla is not None:
            return self._mla_block(lw, kc, vc, xn, inp)
        qkv = linear(xn, lw.qkv, lw.qkv_bias)
        q = torch.empty((T, s.num_q_heads, s.head_dim), device=xn.device, dtype=BF)
        _lib.check(
            _lib.load().b200_qknorm_rope_store(
                qkv.data_ptr(), qkv.stride(0), inp.positions.data_ptr(), inp.slot_mapping.data_ptr(),
                _lib.ptr(lw.q_norm), _lib.ptr(lw.k_norm), self.w.inv_freq.data_ptr(), q.data_ptr(), kc.data_ptr(),
                vc.data_ptr(), T, s.num_q_heads, s.num_kv_heads, s.head_dim, kc.shape[0] * kc.shape[1],
                float(s.rms_eps), _lib.current_stream()),
            "b200_qknorm_rope_store",
        )
        attn = paged_attention(q, kc, vc, inp.query_start_loc, inp.context_lens, inp.block_tables,
                               s.head_dim ** -0.5, inp.max_seqlen_q, seq_order=inp.seq_order)
        return linear(attn.view(T, s.num_q_heads * s.head_dim), lw.o)

    def _mla_block(self, lw: LayerWeights, kc, vc, xn: torch.Tensor, inp: StepInputs) -> torch.Tensor:
        """deepseek_v3_attention_forward (modeling_deepseek_v3.py:225-283), q_lora_rank = None."""
        s, a = self.shape, self.shape.mla
        T, heads = xn.shape[0], s.num_q_heads
        q_in = linear(xn, lw.qkv)                                   # q_proj: [T, heads * (nope + rope)]
        ckv = linear(xn, lw.kv_a)                                   # [T, kv_lora + rope]
        k_lat = batch_invariant_rms_norm(ckv[:, :a.kv_lora_rank], lw.kv_a_norm, s.rms_eps)
        kvb = linear(k_lat, lw.kv_b)                                # [T, heads * (nope + v)]
        k_rot = ckv[:, a.kv_lora_rank:]
        q = torch.empty((T, heads, a.qk_nope + a.qk_rope), device=xn.device, dtype=BF)
        _lib.check(
            _lib.load().b200_mla_rope_store(
                q_in.data_ptr(), q_in.stride(0), kvb.data_ptr(), kvb.stride(0), k_rot.data_ptr(), k_rot.stride(0),
                inp.positions.data_ptr(), inp.slot_mapping.data_ptr(), self.w.inv_freq.data_ptr(), q.data_ptr(),
                kc.data_ptr(), vc.data_ptr(), T, heads, a.qk_nope, a.qk_rope, a.v_head, kc.shape[0] * kc.shape[1],
                _lib.current_stream()),
            "b200_mla_rope_store",
        )
        attn = paged_attention(q, kc, vc, inp.query_start_loc, inp.context_lens, inp.block_tables,
                               (a.qk_nope + a.qk_rope) ** -0.5, inp.max_seqlen_q, seq_order=inp.seq_order)
        return linear(attn.view(T, heads * a.v_head), lw.o)

    # Above this many tokens the fused SwiGLU epilogue (two of the four epilogue warps do the
    # activation math of a whole 128 x 256 tile) costs more than it saves: two plain GEMMs and the
    # elementwise kernel are used instead.  Both routes round at the same points, so a token's result
    # is the same bits either way (tests/test_gpu_model.py).
    DENSE_FUSED_MAX_TOKENS = 64

    def _dense_mlp(self, xn, gate_up, down, width):
        T = xn.shape[0]
        if T <= self.DENSE_FUSED_MAX_TOKENS:
            plan = self._dense_plan(T, xn.device)
            act = _grouped_gemm(xn, gate_up.view(1, 2 * width, self.shape.hidden), None, plan, width, mode=1)
        else:
            g = linear(xn, gate_up[:width])
            u = linear(xn, gate_up[width:])
            act = torch.empty_like(g)
            _lib.check(_lib.load().b200_swiglu_scale(g.data_ptr(), u.data_ptr(), None, act.data_ptr(), T, width,
                                                     _lib.current_stream()), "b200_swiglu_scale")
        return linear(act, down)

    def _mlp_block(self, lw: LayerWeights, xn: torch.Tensor) -> torch.Tensor:
        s = self.shape
        if lw.router is None:
            return self._dense_mlp(xn, lw.gate_up, lw.down, s.ffn)
        m = s.moe
        if m.scoring == "sigmoid_group":
            # PatchDeepseekV3TopkRouter: F.linear in fp32, then route_tokens_to_experts; experts + shared experts
            logits = linear_f32_from_bf16(xn, lw.router)
            sel, rw = route_sigmoid_group_topk(logits, lw.router_bias, m.n_group, m.topk_group, m.top_k,
                                               m.norm_topk_prob, m.routed_scaling_factor)
            shared = None
            if lw.shared_gate_up is not None:
                shared = self._dense_mlp(xn, lw.shared_gate_up, lw.shared_down, m.intermediate * m.n_shared_experts)
            return fused_moe_forward(m.num_experts, rw, sel, xn, fc2_weight=lw.experts_down,
                                     fc1_1_2_weight=lw.experts_gate_up, addend=shared, defer_reduce=True)
        logits = linear(xn, lw.router, lw.router_logit_bias)   # (aten::addmm when the router Linear has a bias)
        if _ROUTE_PLAN:   # routing and the permutation plan in one launch
            rw, sel, plan = route_plan_softmax_topk(logits, m.top_k, m.norm_topk_prob, m.num_experts)
            return fused_moe_forward(m.num_experts, rw, sel, xn, fc2_weight=lw.experts_down,
                                     fc1_1_2_weight=lw.experts_gate_up, defer_reduce=True, plan=plan)
        rw, sel = route_softmax_topk(logits, m.top_k, m.norm_topk_prob)
        return fused_moe_forward(m.num_experts, rw, sel, xn, fc2_weight=lw.experts_down,
                                 fc1_1_2_weight=lw.experts_gate_up, defer_reduce=True)

    def forward(self, inp: StepInputs) -> torch.Tensor:
        """Hidden states after the local layers ([T, H]); the residual stream is complete."""
        if self.is_first:
            h = _gather_rows(self.w.embed, ids=inp.input_ids)
        else:
            h = inp.hidden_in
        delta = None
        for li, lw in zip(range(self.w.start_layer, self.w.end_layer), self.w.layers):
            if delta is None:
                xn = self._norm(h, lw.input_norm)
            else:
                h, xn = self._add_norm(delta, h, lw.input_norm)
            attn_out = self._attention_block(lw, li, xn, inp)
            h, xn2 = self._add_norm(attn_out, h, lw.post_norm)
            delta = self._mlp_block(lw, xn2)
        if delta is not None:
            h = delta.finish_add(h) if isinstance(delta, PendingMoE) else h + delta
        return h

    def last_token_logits(self, h: torch.Tensor, inp: StepInputs) -> torch.Tensor:
        """Last stage: each sequence's last-token row -> final norm -> lm_head.  [num_seqs, vocab].
        (The reference runs lm_head over every packed token and gathers afterwards,
        model_loader.py:267-268 + inferencer.py:403-404; the GEMM is row-invariant, so gathering first
        gives the same rows.)"""
        return linear(self.last_token_hidden(h, inp), self.w.lm_head)

    def last_token_hidden(self, h: torch.Tensor, inp: StepInputs) -> torch.Tensor:
        return self._norm(_gather_rows(h, query_start_loc=inp.query_start_loc), self.w.final_norm)

    def select_tokens(self, h: torch.Tensor, inp: StepInputs):
        """Last stage: last-token logits -> greedy (or sampled) token + its logprob."""
        if self.fused_head and self.sampling is None:
            tokens, logprobs = lm_head_greedy(self.last_token_hidden(h, inp), self.w.lm_head)
            return tokens, logprobs, None
        logits = self.last_token_logits(h, inp)
        if self.sampling is None:
            tokens, logprobs = greedy_token_and_logprob(logits)
        else:   # temperature / top-k / top-p sampling (reference: sampler.py:32-87), one kernel
            tokens, logprobs = sample_token_and_logprob(logits, **self.sampling)
        return tokens, logprobs, logits

    def step(self, inp: StepInputs):
        h = self.forward(inp)
        if self.is_last:
            return self.select_tokens(h, inp)
        return h

    # -- CUDA graph capture over static buffers (cudagraph_utils.py:109-190)
    def capture(self, inp: StepInputs, warmup: int = 2):
        """Capture `step` for these (static) input tensors; returns (graph, outputs)."""
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.step(inp)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.step(inp)
        return graph, out


def allocate_kv_cache(shape: ModelShape, start_layer: int, end_layer: int, num_blocks: int, page_size: int,
                      device="cuda", fill_std: float = 0.0, seed: int = 0):
    """Per-layer K / V caches [blocks, page, kv_heads, head_dim] for the local layers only."""
    kc, vc = {}, {}
    gen = torch.Generator(device=device).manual_seed(seed + 17)
    for li in range(start_layer, end_layer):
        for store in (kc, vc):
            dim = shape.k_dim if store is kc else shape.v_dim
            t = torch.zeros((num_blocks, page_size, shape.num_kv_heads, dim), device=device, dtype=BF)
            if fill_std:
                t.normal_(0.0, fill_std, generator=gen)
            store[li] = t
    return kc, vc


# ------------------------------------------------------------------------------------------------
# The reference's entry points over the stage runner: model-forward keywords, Inferencer.infer
# ------------------------------------------------------------------------------------------------
@dataclass
class StageOutput:
    """What the reference reads off the HF model output (`hidden_states`, `logits`) plus
    `last_logits`: the lm_head rows of each sequence's last token, computed inside the forward so that
    they are part of the captured graph."""

    hidden_states: Optional[torch.Tensor] = None   # [1, T, H]
    logits: Optional[torch.Tensor] = None          # never materialised for all tokens here
    last_logits: Optional[torch.Tensor] = None     # [num_seqs, vocab] (last stage)
    greedy_tokens: Optional[torch.Tensor] = None   # [num_seqs] int64 (last stage, fused head)
    greedy_logprobs: Optional[torch.Tensor] = None  # [num_seqs] fp32


class StageModel:
    """The native stage behind the forward keywords the reference's `Inferencer` and `CudaGraphManager`
    use for an HF module (`TransformersForCausalLM.forward`, model_loader.py:225):
    `model(input_ids=[1, T], intermediate_tensors=[1, T, H], position_ids=[1, T], **forward_kwargs)`.
    Attention metadata and the KV caches come from the thread-local KV-cache context, as for HF."""

    def __init__(self, weights: StageWeights, pp_rank: int = 0, pp_size: int = 1, fused_greedy: bool = False):
        """fused_greedy: the last stage returns greedy tokens + log-probabilities from the fused lm_head
        instead of last-token logits (for deployments that only decode greedily and never return logits)."""
        self.runner = StageRunner(weights, {}, {}, pp_rank, pp_size)
        self.fused_greedy = fused_greedy
        self.config = None
        self.layer_ids = range(weights.start_layer, weights.end_layer)

    def eval(self):
        return self

    def forward(self, input_ids=None, intermediate_tensors=None, position_ids=None, **_unused) -> StageOutput:
        from .kv_cache_context import get_kv_cache_context

        ctx = get_kv_cache_context()
        if ctx is None or not ctx.is_paged_attn:
            raise ValueError("a paged KV-cache context is required (set_kv_cache_context(is_paged_attn=True, ...))")
        r = self.runner
        r.key_cache, r.value_cache = ctx.key_cache, ctx.value_cache
        T = position_ids.shape[-1]
        inp = StepInputs(
            input_ids=input_ids.reshape(-1) if r.is_first else None,
            hidden_in=None if r.is_first else intermediate_tensors.reshape(T, -1),
            positions=position_ids.reshape(-1), slot_mapping=ctx.slot_mapping, query_start_loc=ctx.query_start_loc,
            context_lens=ctx.context_lens, block_tables=ctx.block_tables,
            max_seqlen_q=int(ctx.max_seqlen_q) if ctx.max_seqlen_q else T)
        r.prepare(T, position_ids.device)
        h = r.forward(inp)
        out = StageOutput(hidden_states=h[None])
        if r.is_last:
            if self.fused_greedy:
                out.greedy_tokens, out.greedy_logprobs = lm_head_greedy(r.last_token_hidden(h, inp), r.w.lm_head)
            else:
                out.last_logits = r.last_token_logits(h, inp)
        return out

    __call__ = forward


class PPMissingLayer(torch.nn.Module):
    """Stands in for a module that lives on another pipeline rank: hands its first argument on
    (model_loader.py:205-215)."""

    attention_type = "full_attention"

    def forward(self, *args, **kwargs):
        return args[0] if args else next(iter(kwargs.values()))


class HFModel:
    """An HF `*ForCausalLM` module behind the same forward keywords: the module runs on this library's
    operators through `enable_batch_invariant_mode()`, the registered attention function and
    `register_models()`.  The reference's wrapper for this is `TransformersForCausalLM` (model_loader.py:218-282)
    and its pipeline plan `ModelCreator._apply_pp` (:346-400): with `pp_info` of more than one rank the decoder
    layers outside `get_pp_indices(...)` become `PPMissingLayer`s, the embedding stays on the first rank (and on
    the last one when the word embeddings are tied), the final norm and lm_head on the last; later ranks take the
    previous rank's hidden states as `inputs_embeds`."""

    def __init__(self, hf_model, pp_info=None):
        self.hf_model = hf_model
        self.config = hf_model.config
        self.pp_rank = 0 if pp_info is None else pp_info.pp_rank
        self.pp_size = 1 if pp_info is None else pp_info.pp_size
        s0, s1 = get_pp_indices(self.config.num_hidden_layers, self.pp_rank, self.pp_size)
        self.layer_ids = list(range(s0, s1))       # the layers whose KV cache this rank keeps
        if self.pp_size > 1:
            self._apply_pp()

    def _apply_pp(self):
        base = self.hf_model.model
        first, last = self.pp_rank == 0, self.pp_rank == self.pp_size - 1
        if not (first or (getattr(self.config, "tie_word_embeddings", False) and last)):
            base.embed_tokens = PPMissingLayer()
        s0, s1 = get_pp_indices(self.config.num_hidden_layers, self.pp_rank, self.pp_size)
        for i in range(len(base.layers)):
            if not (s0 <= i < s1):
                base.layers[i] = PPMissingLayer()
        if not last:
            base.norm = PPMissingLayer()
            self.hf_model.lm_head = PPMissingLayer()

    def eval(self):
        self.hf_model.eval()
        return self

    def forward(self, input_ids=None, intermediate_tensors=None, position_ids=None, **_unused) -> StageOutput:
        if self.pp_rank > 0:
            assert intermediate_tensors is not None, "a later pipeline rank runs on the previous rank's hidden states"
            out = self.hf_model.model(input_ids=None, inputs_embeds=intermediate_tensors, position_ids=position_ids,
                                      use_cache=False, return_dict=True)
        else:
            assert input_ids is not None
            out = self.hf_model.model(input_ids=input_ids, position_ids=position_ids, use_cache=False,
                                      return_dict=True)
        hidden = out.last_hidden_state
        if self.pp_rank != self.pp_size - 1:
            return StageOutput(hidden_states=hidden, logits=None)
        return StageOutput(hidden_states=hidden, logits=self.hf_model.lm_head(hidden))

    __call__ = forward


class TransformersForCausalLM(torch.nn.Module):
    """The reference's wrapper class under its own name and constructor (model_loader.py:218-276): the HF base
    model and the lm_head as two modules plus the pipeline position.  Ranks after the first run on the previous
    rank's hidden states (`intermediate_tensors` become `inputs_embeds`), ranks before the last return the hidden
    states and no logits, the last rank applies the lm_head to the positions `logits_to_keep` selects (0 = all).
    The pipeline slicing of the module tree is the caller's (the reference's `ModelCreator._apply_pp`, or
    `HFModel(hf_model, pp_info)` here, which does both)."""

    def __init__(self, model: torch.nn.Module, lm_head: torch.nn.Module, pp_info):
        super().__init__()
        self.model = model
        self.lm_head = lm_head
        self._pp_info = pp_info

    def forward(self, input_ids=None, intermediate_tensors=None, inputs_embeds=None, attention_mask=None,
                position_ids=None, use_cache=None, output_hidden_states=None, logits_to_keep=0, **kwargs):
        from transformers.modeling_outputs import CausalLMOutputWithPast

        if self._pp_info.pp_rank > 0:
            assert intermediate_tensors is not None
            input_ids, inputs_embeds = None, intermediate_tensors
        else:
            assert input_ids is not None
            inputs_embeds = None
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, inputs_embeds=inputs_embeds,
                         use_cache=use_cache, position_ids=position_ids, output_hidden_states=output_hidden_states,
                         **kwargs)
        if self._pp_info.pp_rank != self._pp_info.pp_size - 1:
            return CausalLMOutputWithPast(loss=None, logits=None, past_key_values=None,
                                          hidden_states=out.last_hidden_state, attentions=None)
        keep = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep
        logits = self.lm_head(out.last_hidden_state[:, keep, :])
        return CausalLMOutputWithPast(loss=None, logits=logits, past_key_values=None, hidden_states=out.hidden_states,
                                      attentions=None)


class Inferencer:
    """One forward + token selection per scheduler step, with the pipeline send / receive choreography.

    Same constructor, `infer(requests, recv_infer_out)` contract and helper names as the reference class
    (vexact/inferencer/inferencer.py:58-449).  `model` is a `StageModel` or an HF module running on this
    library's operators; `config` carries `.model` (hf_config, max_model_len, enforce_eager,
    use_fp32_logits), `.cache` (page_size, max_cache_blocks) and `.scheduler` (max_num_seqs,
    max_num_batched_tokens).  Requests are the scheduler's objects: `input_ids_list`, `tokens_this_step`,
    `num_computed_tokens`, `block_ids`, `generated_tokens`, `generation_config`.

    What differs inside: the first rank builds the step's buffers on the device from per-request
    counters (`b200_prepare_step`) instead of per-token host loops, block lists are uploaded as deltas
    for requests that stay in their row, and token selection is one kernel."""

    def __init__(self, model, config, pp_info, pp_messager, device, enable_batch_invariant: bool = True) -> None:
        from .batch_invariant_ops import enable_batch_invariant_mode, is_batch_invariant_mode_enabled
        from .cudagraph_utils import CudaGraphManager
        from .kv_cache_context import KVCacheStore
        from .runtime_data import InputBuffers
        from .step_inputs import StepBuffers

        self.model = model
        self.device = torch.device(device)
        self._pp_info = pp_info
        self._pp_messager = pp_messager
        self.cache_config = config.cache
        self.forward_kwargs = dict(use_cache=False, return_dict=True, output_hidden_states=True, use_fused_lce=False)
        self.use_fp32_logits = bool(getattr(config.model, "use_fp32_logits", False))
        self.page_size = self.cache_config.page_size
        hf_config = config.model.hf_config
        self.cache_store = KVCacheStore(hf_config, self.cache_config, self.device,
                                        layer_ids=getattr(model, "layer_ids", None))
        if enable_batch_invariant and not is_batch_invariant_mode_enabled():
            enable_batch_invariant_mode()
        self.input_buffers = InputBuffers(
            device=self.device, max_num_seqs=config.scheduler.max_num_seqs,
            max_num_batched_tokens=config.scheduler.max_num_batched_tokens,
            max_blocks_per_req=(config.model.max_model_len + self.page_size - 1) // self.page_size,
            hidden_size=hf_config.hidden_size)
        # first rank: the static buffers are written by the step kernel (same tensors, no extra copy)
        self._step_buffers = None
        if pp_info.is_first_rank:
            self._step_buffers = StepBuffers(self.device, config.scheduler.max_num_seqs,
                                             config.scheduler.max_num_batched_tokens,
                                             self.input_buffers.max_blocks_per_req, self.page_size,
                                             buffers=self.input_buffers)
        self._rows: list = []          # per batch row: (request_id, blocks uploaded so far)
        self._cudagraph_mgr: Optional[CudaGraphManager] = None
        if not getattr(config.model, "enforce_eager", False):
            if getattr(config.model, "attn_impl", "fa-invariant") == "flex":
                raise RuntimeError("Cuda graph is enabled but flex attention is not supported for CUDA graph replay.")
            self._cudagraph_mgr = CudaGraphManager(
                model=self.model, device=self.device, cache_store=self.cache_store,
                max_size=config.scheduler.max_num_batched_tokens, cache_config=self.cache_config,
                forward_kwargs=self.forward_kwargs, input_buffers=self.input_buffers)
            self._cudagraph_mgr.capture_graphs()

    # ------------------------------------------------------------------ one scheduler step
    def infer(self, requests, recv_infer_out: bool = False):
        """| pp rank | gen_ctx | forward | infer_out | gen_ctx |
           | first   | build   | yes     | recv      | send    |
           | middle  | recv    | yes     | -         | send    |
           | last    | recv    | yes     | send      | -       |"""
        from .kv_cache_context import set_kv_cache_context
        from .runtime_data import GenerationContext, InferencerOutput

        pp, gen_ctx, outputs = self._pp_info, None, None
        if pp.is_first_rank:
            if len(requests) > 0:
                gen_ctx = self._prepare_gen_ctx(requests)
        else:
            gen_ctx = self._pp_messager.recv_gen_ctx()
            set_kv_cache_context(is_paged_attn=True, key_cache=self.cache_store.key_cache,
                                 value_cache=self.cache_store.value_cache, block_tables=gen_ctx.block_tables,
                                 context_lens=gen_ctx.context_lens, slot_mapping=gen_ctx.slot_mapping,
                                 query_start_loc=gen_ctx.query_start_loc, max_seqlen_q=gen_ctx.max_seqlen_q)
        if gen_ctx is not None:
            outputs = self._forward(gen_ctx)
        final_output = None
        if pp.is_last_rank and gen_ctx is not None:
            token_ids, logits, logprobs = self._select_tokens(gen_ctx.generation_configs, gen_ctx.tokens_generated,
                                                              outputs, gen_ctx)
            final_output = InferencerOutput(token_ids=token_ids, logits=logits, logprobs=logprobs)
            if pp.is_first_rank:
                return final_output
            self._pp_messager.send_infer_out(final_output)
            final_output = None
        if pp.is_first_rank and recv_infer_out:
            final_output = self._pp_messager.recv_infer_out()
        if not pp.is_last_rank and gen_ctx is not None:
            num_tokens = gen_ctx.batch_position_ids.shape[1]
            self._pp_messager.send_gen_ctx(GenerationContext(
                batch_input_ids=None, intermediate_tensors=outputs.hidden_states[:, :num_tokens, :],
                query_start_loc=gen_ctx.query_start_loc, batch_position_ids=gen_ctx.batch_position_ids,
                block_tables=gen_ctx.block_tables, context_lens=gen_ctx.context_lens,
                slot_mapping=gen_ctx.slot_mapping, max_seqlen_q=gen_ctx.max_seqlen_q,
                generation_configs=gen_ctx.generation_configs, tokens_generated=gen_ctx.tokens_generated))
        return final_output

    # ------------------------------------------------------------------ first rank: requests -> buffers
    def _upload_block_lists(self, requests) -> None:
        """Keep `request_blocks[row]` equal to each request's block list, uploading only what changed:
        a request that kept its row since the last step sends the blocks it gained."""
        sb = self._step_buffers
        rows, cols, vals = [], [], []
        for row, req in enumerate(requests):
            blocks = req.block_ids
            known = self._rows[row] if row < len(self._rows) else None
            rid = getattr(req, "request_id", id(req))
            if known is not None and known[0] == rid and known[1] <= len(blocks):
                for c in range(known[1], len(blocks)):
                    rows.append(row)
                    cols.append(c)
                    vals.append(blocks[c])
            else:
                sb.set_request_blocks(row, blocks)
            if row < len(self._rows):
                self._rows[row] = (rid, len(blocks))
            else:
                self._rows.append((rid, len(blocks)))
        del self._rows[len(requests):]
        for i in range(0, len(rows), sb.max_num_seqs * 2):
            j = i + sb.max_num_seqs * 2
            sb.append_blocks(rows[i:j], cols[i:j], vals[i:j])

    def _prepare_gen_ctx(self, requests):
        from .kv_cache_context import set_kv_cache_context
        from .runtime_data import GenerationContext

        sb = self._step_buffers
        num_seqs = len(requests)
        computed = [int(r.num_computed_tokens) for r in requests]
        this_step = [int(r.tokens_this_step) for r in requests]
        total = sum(this_step)
        chunks = {}
        for row, req in enumerate(requests):
            start = computed[row] - this_step[row]
            assert start >= 0
            if start < len(req.input_ids_list):       # prefill, or re-prefill after a preemption
                chunks[row] = req.input_ids_list[start:computed[row]]
            else:                                      # decode: the last generated token
                chunks[row] = [req.generated_tokens[-1]]
        self._upload_block_lists(requests)
        max_q = max(this_step) if this_step else 0
        desc = self._cudagraph_mgr.dispatch(num_seqs, total, max_q) if self._cudagraph_mgr else None
        if self._cudagraph_mgr and desc is None:
            raise RuntimeError(f"Cuda graph is enabled but no captured descriptor can cover {num_seqs} sequences "
                               f"and {total} tokens. Available descriptors: {list(self._cudagraph_mgr.graphs)}")
        self._graph_desc = desc
        graph_seqs, cap_tokens = (desc.num_seqs, desc.num_tokens) if desc else (num_seqs, total)
        inp = sb.prepare(computed, this_step, chunks, graph_seqs, cap_tokens)
        # the (padded) static views are what the forward reads; the context handed on holds the real sizes
        set_kv_cache_context(is_paged_attn=True, key_cache=self.cache_store.key_cache,
                             value_cache=self.cache_store.value_cache, block_tables=inp.block_tables,
                             context_lens=inp.context_lens, slot_mapping=inp.slot_mapping,
                             query_start_loc=inp.query_start_loc, max_seqlen_q=max_q)
        return GenerationContext(
            batch_input_ids=sb.input_ids[:, :total], intermediate_tensors=None,
            query_start_loc=sb.query_start_loc[: num_seqs + 1], batch_position_ids=sb.position_ids[:, :total],
            block_tables=sb.request_blocks[:num_seqs], context_lens=sb.context_lens[:num_seqs],
            slot_mapping=sb.slot_mapping[:total], max_seqlen_q=max_q,
            generation_configs=[r.generation_config for r in requests],
            tokens_generated=[len(r.generated_tokens) for r in requests])

    # ------------------------------------------------------------------ later ranks: ctx -> static buffers
    def _prepare_input_buffers_from_gen_ctx(self, gen_ctx, graph_desc) -> None:
        from .kv_cache_context import set_kv_cache_context

        buf = self.input_buffers
        cap, gseqs = graph_desc.num_tokens, graph_desc.num_seqs
        num_seqs = gen_ctx.context_lens.size(0)
        total = gen_ctx.batch_position_ids.size(1)
        if total > cap:
            raise ValueError(f"total_tokens exceeds capture_tokens: {total} > {cap}")
        if gseqs < num_seqs:
            raise ValueError(f"graph_num_seqs cannot be smaller than num_seqs: {gseqs} < {num_seqs}")
        if not self._pp_info.is_first_rank:
            # (the first rank's step kernel has already written the padded buffers in place)
            buf.input_ids.gpu[:, :cap].zero_()
            buf.position_ids.gpu[:, :cap].zero_()
            buf.intermediate_tensors.gpu[:, total:cap, :].zero_()
            buf.block_tables.gpu[:gseqs].zero_()
            buf.context_lens.gpu[:gseqs].zero_()
            buf.slot_mapping.gpu[:cap].fill_(-1)
            buf.block_tables.gpu[:num_seqs, : gen_ctx.block_tables.shape[1]].copy_(gen_ctx.block_tables)
            buf.context_lens.gpu[:num_seqs].copy_(gen_ctx.context_lens)
            buf.slot_mapping.gpu[:total].copy_(gen_ctx.slot_mapping)
            buf.query_start_loc.gpu[: num_seqs + 1].copy_(gen_ctx.query_start_loc)
            if gseqs > num_seqs:      # padded requests: zero-length, placed after the real tokens
                buf.query_start_loc.gpu[num_seqs + 1: gseqs + 1] = total
            if gen_ctx.batch_input_ids is not None:
                buf.input_ids.gpu[:, :total].copy_(gen_ctx.batch_input_ids)
            buf.position_ids.gpu[:, :total].copy_(gen_ctx.batch_position_ids)
            if gen_ctx.intermediate_tensors is not None:
                buf.intermediate_tensors.gpu[:, :total, :].copy_(gen_ctx.intermediate_tensors)
        block_tables, context_lens, slot_mapping, query_start_loc = buf.get_kv_context_tensors(gseqs, cap)
        set_kv_cache_context(is_paged_attn=True, key_cache=self.cache_store.key_cache,
                             value_cache=self.cache_store.value_cache, block_tables=block_tables,
                             context_lens=context_lens, slot_mapping=slot_mapping, query_start_loc=query_start_loc,
                             max_seqlen_q=gen_ctx.max_seqlen_q)

    @torch.inference_mode()
    def _forward(self, gen_ctx):
        if self._cudagraph_mgr:
            total = (gen_ctx.batch_input_ids if gen_ctx.batch_input_ids is not None
                     else gen_ctx.intermediate_tensors).size(1)
            num_seqs = gen_ctx.context_lens.size(0)
            desc = getattr(self, "_graph_desc", None) if self._pp_info.is_first_rank else None
            if desc is None:
                desc = self._cudagraph_mgr.dispatch(num_seqs, total, gen_ctx.max_seqlen_q)
            if desc is None:
                raise RuntimeError(f"Cuda graph is enabled but no captured descriptor can cover {num_seqs} sequences "
                                   f"and {total} tokens. Available descriptors: {list(self._cudagraph_mgr.graphs)}")
            self._prepare_input_buffers_from_gen_ctx(gen_ctx, desc)
            return self._forward_cudagraph(desc)
        return self._forward_eager(gen_ctx)

    @torch.inference_mode()
    def _forward_cudagraph(self, graph_key):
        with torch.cuda.nvtx.range("model_forward_cudagraph"):
            return self._cudagraph_mgr.replay(graph_key)

    @torch.inference_mode()
    def _forward_eager(self, gen_ctx):
        with torch.cuda.nvtx.range("model_forward_eager"):
            return self.model(input_ids=gen_ctx.batch_input_ids, intermediate_tensors=gen_ctx.intermediate_tensors,
                              position_ids=gen_ctx.batch_position_ids, **self.forward_kwargs)

    # ------------------------------------------------------------------ last rank: logits -> tokens
    @torch.inference_mode()
    def _select_tokens(self, gen_configs, tokens_generated, outputs, gen_ctx):
        num_seqs = gen_ctx.context_lens.size(0)
        last_logits = getattr(outputs, "last_logits", None)
        if getattr(outputs, "greedy_tokens", None) is not None:
            # fused head: tokens and log-probabilities came out of the forward; nothing else is available
            ref = gen_configs[0]
            if any(g.do_sample and (g.temperature or 0) > 0 for g in gen_configs) or getattr(ref, "output_logits", False):
                raise RuntimeError("the model was built with fused_greedy: sampling and output_logits need logits")
            logprobs = outputs.greedy_logprobs[:num_seqs]
            if not any(getattr(g, "output_scores", False) for g in gen_configs):
                logprobs = torch.empty(0, device=self.device)
            return outputs.greedy_tokens[:num_seqs], torch.empty(0, device=self.device), logprobs
        if last_logits is not None:
            batched_logits = last_logits[:num_seqs]
        else:   # an HF module: logits of every packed token, gather the last one of each request
            last = (gen_ctx.query_start_loc[1:] - 1).to(dtype=torch.long)
            batched_logits = outputs.logits[0, last, :]
        ref = gen_configs[0]
        uniform = all((g.do_sample == ref.do_sample and g.temperature == ref.temperature and g.top_k == ref.top_k
                       and g.top_p == ref.top_p) for g in gen_configs)
        assert uniform
        scored = self.use_fp32_logits and batched_logits.dtype != torch.float32
        sample_logits = batched_logits.float() if scored else batched_logits
        assert ref.top_p is not None, "top_p must be set (use 1.0 to disable)"
        do_sample = bool(ref.do_sample) and (ref.temperature or 0) > 0 and float(ref.top_p) > 0
        if do_sample:
            noise = None
            seeds = [getattr(g, "seed", None) for g in gen_configs]
            if any(s is not None for s in seeds):     # vLLM-style: RNG keyed by request seed and token position
                if not all(s is not None for s in seeds):
                    raise ValueError("Seeded sampling requires every request in the batch to set seed.")
                from .sampler import seeded_exponential_noise
                seed_t = torch.tensor([int(s) for s in seeds], dtype=torch.int64).to(self.device, non_blocking=True)
                noise = seeded_exponential_noise(seed_t, gen_ctx.context_lens.to(torch.long) - 1,
                                                 sample_logits.shape[-1])
            tokens, logprobs = sample_token_and_logprob(sample_logits, float(ref.temperature), ref.top_k,
                                                        float(ref.top_p), True, noise)
        else:
            tokens, logprobs = greedy_token_and_logprob(sample_logits)
        logits = batched_logits.detach() if getattr(ref, "output_logits", False) else torch.empty(0, device=self.device)
        want = [i for i, g in enumerate(gen_configs) if getattr(g, "output_scores", False)]
        if not want:
            logprobs = torch.empty(0, device=self.device)
        elif len(want) != len(gen_configs):
            logprobs = logprobs.index_select(0, torch.tensor(want, dtype=torch.long).to(self.device, non_blocking=True))
        return tokens, logits, logprobs
