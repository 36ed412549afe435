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

from dataclasses import dataclass, field
from typing import Optional

import torch

from . import _lib
from .attention import paged_attention
from .batch_invariant_ops import add_rms_norm, batch_invariant_rms_norm, hf_rms_norm, linear
from .fused_moe import (TILE_ROWS, PendingMoE, _grouped_gemm, fused_moe_forward, route_sigmoid_group_topk,
                        route_softmax_topk)
from .standalone_logprobs import greedy_token_and_logprob
from .sampler import sample_token_and_logprob

BF = torch.bfloat16


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
            logits = linear(xn.float(), lw.router.float())
            sel, rw = route_sigmoid_group_topk(logits, lw.router_bias, m.n_group, m.topk_group, m.top_k,
                                               m.norm_topk_prob, m.routed_scaling_factor)
            shared = None
            if lw.shared_gate_up is not None:
                shared = self._dense_mlp(xn, lw.shared_gate_up, lw.shared_down, m.intermediate * m.n_shared_experts)
            return fused_moe_forward(m.num_experts, rw, sel, xn, fc2_weight=lw.experts_down,
                                     fc1_1_2_weight=lw.experts_gate_up, addend=shared, defer_reduce=True)
        logits = linear(xn, lw.router)
        rw, sel = route_softmax_topk(logits, m.top_k, m.norm_topk_prob)
        return fused_moe_forward(m.num_experts, rw, sel, xn, fc2_weight=lw.experts_down,
                                 fc1_1_2_weight=lw.experts_gate_up, defer_reduce=True)

    def forward(self, inp: StepInputs) -> torch.Tensor:
        """Hidden states after the local layers ([T, H]); the residual stream is complete."""
        if self.is_first:
            h = self.w.embed.index_select(0, inp.input_ids)
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
            h = h + (delta.finish() if isinstance(delta, PendingMoE) else delta)
        return h

    def select_tokens(self, h: torch.Tensor, inp: StepInputs):
        """Last stage: last-token rows -> final norm -> lm_head -> greedy token + its logprob."""
        s = self.shape
        last = (inp.query_start_loc[1:] - 1).to(torch.long)
        rows = h.index_select(0, last.clamp(min=0))
        xn = self._norm(rows, self.w.final_norm)
        logits = linear(xn, self.w.lm_head)
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
