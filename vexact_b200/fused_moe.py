"""Fused MoE forward: routing, permutation, grouped GEMMs, top-k reduction.

Mirror of vexact/batch_invariant_ops/fused_moe.py:459 (`fused_moe_forward`, split
fc1 signature) extended with the keyword form the model files use
(`fc1_1_2_weight`, modeling_qwen3_moe.py:89-100, modeling_deepseek_v3.py:148-160),
plus the two routing functions of the model definitions.

Pipeline (all on the caller's stream, scratch from torch's caching allocator):
  b200_moe_permute        stable sort positions, cu_seqlens, tile table, row gather
  b200_moe_grouped_gemm   fc1 with fused SwiGLU * routing weight (fused gate_up weights), or
                          two plain grouped GEMMs + b200_swiglu_scale (split weights)
  b200_moe_grouped_gemm   fc2
  b200_moe_unpermute_reduce  fp32 sum of a token's k rows in k order, one cast
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import _lib

TILE_ROWS = 64  # largest token tile of the grouped GEMM (rows of one expert per tile)
FUSED_SWIGLU_MAX_ROWS_PER_EXPERT = 64  # mean rows per expert up to which fc1 keeps its fused SwiGLU epilogue


def max_token_tiles(num_rows: int, num_experts: int, tile_rows: int = TILE_ROWS) -> int:
    """Upper bound on expert token tiles: every expert may add one partial tile."""
    return min(num_rows, num_experts) + num_rows // tile_rows


def route_softmax_topk(router_logits: torch.Tensor, top_k: int, norm_topk_prob: bool = True,
                       out_dtype: torch.dtype = torch.bfloat16):
    """softmax(fp32) -> top-k -> renormalise -> cast (modeling_qwen3_moe.py:128-134).

    Returns (routing_weights [T, k] out_dtype, selected_experts [T, k] int64), experts in
    descending weight order, ties to the lower index.
    """
    if not router_logits.is_cuda:
        raise ValueError("router_logits must be a CUDA tensor")
    T, E = router_logits.shape
    x = router_logits if router_logits.stride(-1) == 1 else router_logits.contiguous()
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise NotImplementedError(f"router logits dtype {x.dtype}")
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise NotImplementedError(f"routing weight dtype {out_dtype}")
    w = torch.empty((T, top_k), device=x.device, dtype=out_dtype)
    idx = torch.empty((T, top_k), device=x.device, dtype=torch.int64)
    _lib.check(
        _lib.load().b200_moe_route_softmax_topk(
            x.data_ptr(), 0 if x.dtype == torch.float32 else 1, x.stride(0),
            w.data_ptr() if out_dtype == torch.bfloat16 else None,
            w.data_ptr() if out_dtype == torch.float32 else None,
            None, idx.data_ptr(), T, E, top_k, 1 if norm_topk_prob else 0, _lib.current_stream()),
        "b200_moe_route_softmax_topk",
    )
    return w, idx


_PLAN_COUNTERS: dict = {}      # device index -> the 257 zeroed int32 counters of the routing-plan kernel


def route_plan_softmax_topk(router_logits: torch.Tensor, top_k: int, norm_topk_prob: bool, num_experts: int):
    """`route_softmax_topk` that also plans the expert permutation in the same launch.

    Returns (routing_weights [T, k] bf16, selected_experts [T, k] int64, plan); pass `plan` to
    `fused_moe_forward(..., plan=plan)`.  The plan orders rows inside an expert's group by arrival (an atomic
    counter), not by token; no MoE output depends on that order.  The counters live in one array per device,
    so calls on one device must not overlap (they do not on one stream)."""
    if not router_logits.is_cuda:
        raise ValueError("router_logits must be a CUDA tensor")
    T, E = router_logits.shape
    if E != num_experts:
        raise ValueError("router logits do not have one column per expert")
    x = router_logits if router_logits.stride(-1) == 1 else router_logits.contiguous()
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise NotImplementedError(f"router logits dtype {x.dtype}")
    dev = x.device
    counters = _PLAN_COUNTERS.get(dev.index)
    if counters is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("make the first routing-plan call on a device outside graph capture")
        counters = torch.zeros(257, device=dev, dtype=torch.int32)
        _PLAN_COUNTERS[dev.index] = counters
    n = T * top_k
    max_tiles = max(1, max_token_tiles(n, num_experts))
    w = torch.empty((T, top_k), device=dev, dtype=torch.bfloat16)
    idx = torch.empty((T, top_k), device=dev, dtype=torch.int64)
    rank = torch.empty(n, device=dev, dtype=torch.int32)
    cu_seqlens = torch.empty(num_experts + 1, device=dev, dtype=torch.int32)
    tile_table = torch.empty((max_tiles, 4), device=dev, dtype=torch.int32)
    tile_count = torch.empty(1, device=dev, dtype=torch.int32)
    _lib.check(
        _lib.load().b200_moe_route_plan_softmax_topk(
            x.data_ptr(), 0 if x.dtype == torch.float32 else 1, x.stride(0), w.data_ptr(), idx.data_ptr(),
            rank.data_ptr(), counters.data_ptr(), cu_seqlens.data_ptr(), tile_table.data_ptr(), tile_count.data_ptr(),
            T, E, top_k, 1 if norm_topk_prob else 0, TILE_ROWS, max_tiles, _lib.current_stream()),
        "b200_moe_route_plan_softmax_topk",
    )
    plan = dict(rank=rank, cu_seqlens=cu_seqlens, tile_table=tile_table, tile_count=tile_count, max_tiles=max_tiles)
    return w, idx, plan


def _scatter_ranked(plan: dict, expert_index: torch.Tensor, routing_weights: torch.Tensor, x: torch.Tensor,
                    num_experts: int) -> dict:
    """Expert-sorted copy of x, row scales and scatter_index for a plan of `route_plan_softmax_topk`."""
    T, k = expert_index.shape
    n, H = T * k, x.shape[-1]
    x_perm = torch.empty((n, H), device=x.device, dtype=torch.bfloat16)
    row_scale = torch.empty(n, device=x.device, dtype=torch.bfloat16)
    scatter_index = torch.empty(n, device=x.device, dtype=torch.int32)
    _lib.check(
        _lib.load().b200_moe_scatter_ranked(
            x.data_ptr(), x.stride(0), expert_index.data_ptr(), routing_weights.data_ptr(), plan["rank"].data_ptr(),
            plan["cu_seqlens"].data_ptr(), scatter_index.data_ptr(), x_perm.data_ptr(), row_scale.data_ptr(), T, k,
            num_experts, H, _lib.current_stream()),
        "b200_moe_scatter_ranked",
    )
    return dict(scatter_index=scatter_index, cu_seqlens=plan["cu_seqlens"], tile_table=plan["tile_table"],
                tile_count=plan["tile_count"], x_perm=x_perm, row_scale=row_scale, max_tiles=plan["max_tiles"])


def route_sigmoid_group_topk(router_logits: torch.Tensor, e_score_correction_bias: Optional[torch.Tensor],
                             n_group: int, topk_group: int, top_k: int, norm_topk_prob: bool,
                             routed_scaling_factor: float):
    """DeepSeek-V3 routing (modeling_deepseek_v3.py:185-208).  Returns (indices int64, weights fp32)."""
    if not router_logits.is_cuda:
        raise ValueError("router_logits must be a CUDA tensor")
    x = router_logits.float()
    x = x if x.stride(-1) == 1 else x.contiguous()
    T, E = x.shape
    bias = None if e_score_correction_bias is None else e_score_correction_bias.float().contiguous()
    w = torch.empty((T, top_k), device=x.device, dtype=torch.float32)
    idx = torch.empty((T, top_k), device=x.device, dtype=torch.int64)
    _lib.check(
        _lib.load().b200_moe_route_sigmoid_group_topk(
            x.data_ptr(), x.stride(0), _lib.ptr(bias), w.data_ptr(), None, idx.data_ptr(), T, E, n_group,
            topk_group, top_k, 1 if norm_topk_prob else 0, float(routed_scaling_factor), _lib.current_stream()),
        "b200_moe_route_sigmoid_group_topk",
    )
    return idx, w


def build_moe_indices(expert_index: torch.Tensor, num_experts: int):
    """(cu_seqlens_m [E+1], A_idx [T*k], scatter_index [T, k]) as fused_moe.py:268 returns them."""
    T, k = expert_index.shape
    plan = _permute(expert_index, None, None, num_experts, gather=True)
    return plan["cu_seqlens"], plan["gather_index"], plan["scatter_index"].view(T, k)


def _gather_default() -> bool:
    """B200_MOE_GATHER=1: fc1 reads its activation rows through the gather index and no permuted copy of the
    activations is made (16 MB less scratch at 512 tokens x top-8 x 2048).  Off by default: one TMA gather moves
    four rows, so a 64-row stage takes 32 TMA instructions instead of 2, and the decode-shaped fc1 measured
    209 us against 126 us over the permuted copy plus 7 us for making it."""
    return os.environ.get("B200_MOE_GATHER", "0") == "1"


def _permute(expert_index: torch.Tensor, routing_weights: Optional[torch.Tensor],
             hidden_states: Optional[torch.Tensor], num_experts: int, gather: bool = False):
    """Index arrays + token-tile table of one routing.  gather=False also writes the expert-sorted copy of the
    activations (`x_perm`); gather=True writes `gather_index` (sorted row -> token) instead, in one launch."""
    dev = expert_index.device
    T, k = expert_index.shape
    n = T * k
    if expert_index.dtype not in (torch.int32, torch.int64):
        expert_index = expert_index.to(torch.int64)
    expert_index = expert_index.contiguous()
    max_tiles = max(1, max_token_tiles(n, num_experts))
    scatter_index = torch.empty(n, device=dev, dtype=torch.int32)
    cu_seqlens = torch.empty(num_experts + 1, device=dev, dtype=torch.int32)
    tile_table = torch.empty((max_tiles, 4), device=dev, dtype=torch.int32)
    tile_count = torch.empty(1, device=dev, dtype=torch.int32)
    x_perm = row_scale = None
    if gather:
        gather_index = torch.empty(n, device=dev, dtype=torch.int32)
        if routing_weights is not None:
            row_scale = torch.empty(n, device=dev, dtype=torch.bfloat16)
        _lib.check(
            _lib.load().b200_moe_permute_index(
                expert_index.data_ptr(), 0 if expert_index.dtype == torch.int32 else 1, _lib.ptr(routing_weights),
                scatter_index.data_ptr(), cu_seqlens.data_ptr(), gather_index.data_ptr(), _lib.ptr(row_scale),
                tile_table.data_ptr(), tile_count.data_ptr(), T, k, num_experts, TILE_ROWS, max_tiles,
                _lib.current_stream()),
            "b200_moe_permute_index",
        )
        return dict(scatter_index=scatter_index, cu_seqlens=cu_seqlens, tile_table=tile_table, tile_count=tile_count,
                    x_perm=None, x=hidden_states, gather_index=gather_index, row_scale=row_scale,
                    max_tiles=max_tiles)
    H = 8
    x_stride = 8
    if hidden_states is not None:
        H = hidden_states.shape[-1]
        x_stride = hidden_states.stride(0)
        x_perm = torch.empty((n, H), device=dev, dtype=torch.bfloat16)
        if routing_weights is not None:
            row_scale = torch.empty(n, device=dev, dtype=torch.bfloat16)
    _lib.check(
        _lib.load().b200_moe_permute(
            expert_index.data_ptr(), 0 if expert_index.dtype == torch.int32 else 1, _lib.ptr(routing_weights),
            _lib.ptr(hidden_states), x_stride, scatter_index.data_ptr(), cu_seqlens.data_ptr(),
            _lib.ptr(x_perm), _lib.ptr(row_scale), tile_table.data_ptr(), tile_count.data_ptr(), T, k,
            num_experts, H, TILE_ROWS, max_tiles, _lib.current_stream()),
        "b200_moe_permute",
    )
    return dict(scatter_index=scatter_index, cu_seqlens=cu_seqlens, tile_table=tile_table,
                tile_count=tile_count, x_perm=x_perm, row_scale=row_scale, max_tiles=max_tiles)


def _grouped_gemm_fc1(w, row_scale, plan, n_out, mode):
    """The first grouped GEMM of the MoE: over the permuted copy, or gathering rows of the unpermuted input."""
    if plan.get("gather_index") is None:
        return _grouped_gemm(plan["x_perm"], w, row_scale, plan, n_out, mode)
    x, idx = plan["x"], plan["gather_index"]
    out = torch.empty((idx.numel(), n_out), device=x.device, dtype=torch.bfloat16)
    _lib.check(
        _lib.load().b200_moe_grouped_gemm_gather(
            x.data_ptr(), x.shape[0], x.stride(0), idx.data_ptr(), w.data_ptr(), _lib.ptr(row_scale), out.data_ptr(),
            plan["tile_table"].data_ptr(), plan["tile_count"].data_ptr(), w.shape[0], n_out, x.shape[1],
            out.stride(0), plan["max_tiles"], plan.get("tile_rows", TILE_ROWS), mode, _lib.current_stream()),
        "b200_moe_grouped_gemm_gather",
    )
    return out


def _grouped_gemm(x, w, row_scale, plan, n_out, mode):
    rows, K = x.shape
    out = torch.empty((rows, n_out), device=x.device, dtype=torch.bfloat16)
    _lib.check(
        _lib.load().b200_moe_grouped_gemm(
            x.data_ptr(), w.data_ptr(), _lib.ptr(row_scale), out.data_ptr(), plan["tile_table"].data_ptr(),
            plan["tile_count"].data_ptr(), rows, w.shape[0], n_out, K, out.stride(0), plan["max_tiles"],
            plan.get("tile_rows", TILE_ROWS), mode, _lib.current_stream()),
        "b200_moe_grouped_gemm",
    )
    return out


class PendingMoE:
    """Expert outputs still in expert-sorted order: the top-k sum has not run yet, so that it can be
    fused with the residual add and RMSNorm that follow (`add_norm`) or run on its own (`finish`)."""

    def __init__(self, y, scatter_index, addend, T, k, H, shape):
        self.y, self.scatter_index, self.addend = y, scatter_index, addend
        self.T, self.k, self.H, self.shape = T, k, H, shape

    def finish(self) -> torch.Tensor:
        out = torch.empty((self.T, self.H), device=self.y.device, dtype=torch.bfloat16)
        _lib.check(
            _lib.load().b200_moe_unpermute_reduce(self.y.data_ptr(), self.scatter_index.data_ptr(),
                                                  _lib.ptr(self.addend), out.data_ptr(), self.T, self.k, self.H,
                                                  _lib.current_stream()),
            "b200_moe_unpermute_reduce",
        )
        return out.reshape(self.shape)

    def finish_add(self, residual: torch.Tensor) -> torch.Tensor:
        """residual + moe output (each a bf16 tensor, as `residual + finish()` computes it) in the top-k sum's
        own launch; with a shared-expert addend pending the two steps stay separate."""
        if self.addend is not None:
            return residual + self.finish()
        out = torch.empty((self.T, self.H), device=self.y.device, dtype=torch.bfloat16)
        r = residual.reshape(self.T, self.H).contiguous()
        _lib.check(
            _lib.load().b200_moe_unpermute_reduce(self.y.data_ptr(), self.scatter_index.data_ptr(), r.data_ptr(),
                                                  out.data_ptr(), self.T, self.k, self.H, _lib.current_stream()),
            "b200_moe_unpermute_reduce",
        )
        return out.reshape(residual.shape)

    def add_norm(self, residual: torch.Tensor, weight: torch.Tensor, eps: float, hf: bool = True):
        """(residual + moe output, rmsnorm of that sum): `finish()` + `add_rms_norm` in one launch."""
        # the fused kernel reproduces the one-CTA-per-row norm kernel, which serves rows of 1025..8192 elements
        if self.H % 8 != 0 or self.H > 8192 or self.H <= 1024:
            from .batch_invariant_ops import add_rms_norm
            return add_rms_norm(self.finish(), residual, weight, eps, hf)
        r = residual.reshape(self.T, self.H).contiguous()
        w = weight.to(torch.bfloat16).contiguous()
        s = torch.empty_like(r)
        out = torch.empty_like(r)
        _lib.check(
            _lib.load().b200_moe_unpermute_add_rmsnorm(
                self.y.data_ptr(), self.scatter_index.data_ptr(), _lib.ptr(self.addend), r.data_ptr(), w.data_ptr(),
                s.data_ptr(), out.data_ptr(), self.T, self.k, self.H, float(eps), 1 if hf else 0,
                _lib.current_stream()),
            "b200_moe_unpermute_add_rmsnorm",
        )
        return s.reshape(residual.shape), out.reshape(residual.shape)


def fused_moe_forward(
    num_experts: int,
    routing_weights: torch.Tensor,
    selected_experts: torch.Tensor,
    hidden_states: torch.Tensor,
    fc1_1_weight: Optional[torch.Tensor] = None,
    fc1_2_weight: Optional[torch.Tensor] = None,
    fc2_weight: Optional[torch.Tensor] = None,
    fc1_1_2_weight: Optional[torch.Tensor] = None,
    addend: Optional[torch.Tensor] = None,
    defer_reduce: bool = False,
    plan: Optional[dict] = None,
):
    """sum_k w_k * fc2_e(silu(fc1_1_e x) * fc1_2_e x) for the selected experts e of each token.

    With defer_reduce the call stops before the top-k sum and returns a `PendingMoE`.

    Weights: fc1_1 / fc1_2 [E, I, H] (split) or fc1_1_2 [E, 2I, H] (gate rows first), fc2 [E, H, I].
    The routing weight multiplies the activation before fc2 and every intermediate is a bf16
    tensor, as in fused_moe.py:319-342.  `addend` [T, H] is added to the result as a separate
    bf16 add (the shared-expert output of DeepSeek-V3).
    """
    if not hidden_states.is_cuda:
        raise ValueError("hidden_states must be a CUDA tensor")
    if fc2_weight is None:
        raise ValueError("fc2_weight is required")
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (
            routing_weights, hidden_states, fc1_1_weight, fc1_2_weight, fc2_weight, fc1_1_2_weight, addend)):
        # the training side: through the autograd Function, as the reference's fused_moe_forward does (fused_moe.py:459)
        if defer_reduce or plan is not None:
            raise NotImplementedError("defer_reduce / plan are inference-only forms")
        if fc1_1_2_weight is not None:
            I = fc1_1_2_weight.shape[1] // 2
            fc1_1_weight, fc1_2_weight = fc1_1_2_weight[:, :I].contiguous(), fc1_1_2_weight[:, I:].contiguous()
        out = FusedMoeExpertFunction.apply(num_experts, routing_weights.bfloat16(), selected_experts,
                                           hidden_states.bfloat16(), fc1_1_weight, fc1_2_weight, fc2_weight)
        return out if addend is None else out + addend.to(torch.bfloat16).reshape(out.shape)
    routing_weights = routing_weights.to(torch.bfloat16).contiguous()
    orig_shape = hidden_states.shape
    x = hidden_states.to(torch.bfloat16).reshape(-1, orig_shape[-1])
    if x.stride(-1) != 1:
        x = x.contiguous()
    T, H = x.shape
    k = selected_experts.shape[-1]
    selected_experts = selected_experts.reshape(T, k)
    if plan is not None:      # made by route_plan_softmax_topk together with the routing
        if selected_experts.dtype != torch.int64 or not selected_experts.is_contiguous():
            raise ValueError("a routing plan goes with the int64 expert indices its routing call returned")
        plan = _scatter_ranked(plan, selected_experts, routing_weights.reshape(T, k), x, num_experts)
    else:
        plan = _permute(selected_experts, routing_weights.reshape(T, k), x, num_experts, gather=_gather_default())
    if fc1_1_2_weight is not None:
        assert fc1_1_2_weight.dtype == torch.bfloat16 and fc1_1_2_weight.is_contiguous()
        I = fc1_1_2_weight.shape[1] // 2
        if T * k > FUSED_SWIGLU_MAX_ROWS_PER_EXPERT * num_experts:
            # many rows per expert (prefill): the fused SwiGLU epilogue, where two of the four epilogue
            # warps do a tile's activation math, would bound the kernel; one plain grouped GEMM over the
            # gate and up rows plus the elementwise kernel rounds at the same points (same bits)
            gu = _grouped_gemm_fc1(fc1_1_2_weight, None, plan, 2 * I, mode=0)
            h = torch.empty((gu.shape[0], I), device=gu.device, dtype=torch.bfloat16)
            _lib.check(
                _lib.load().b200_swiglu_scale_strided(gu.data_ptr(), gu.data_ptr() + I * gu.element_size(),
                                                      plan["row_scale"].data_ptr(), h.data_ptr(), gu.shape[0], I,
                                                      gu.stride(0), _lib.current_stream()),
                "b200_swiglu_scale_strided",
            )
        else:
            h = _grouped_gemm_fc1(fc1_1_2_weight, plan["row_scale"], plan, I, mode=1)
    else:
        if fc1_1_weight is None or fc1_2_weight is None:
            raise ValueError("pass fc1_1_weight and fc1_2_weight, or fc1_1_2_weight")
        fc1_1_weight = fc1_1_weight.to(torch.bfloat16).contiguous()
        fc1_2_weight = fc1_2_weight.to(torch.bfloat16).contiguous()
        I = fc1_1_weight.shape[1]
        g = _grouped_gemm_fc1(fc1_1_weight, None, plan, I, mode=0)
        u = _grouped_gemm_fc1(fc1_2_weight, None, plan, I, mode=0)
        h = torch.empty_like(g)
        _lib.check(
            _lib.load().b200_swiglu_scale(g.data_ptr(), u.data_ptr(), plan["row_scale"].data_ptr(), h.data_ptr(),
                                          g.shape[0], I, _lib.current_stream()),
            "b200_swiglu_scale",
        )
    fc2_weight = fc2_weight if (fc2_weight.dtype == torch.bfloat16 and fc2_weight.is_contiguous()) \
        else fc2_weight.to(torch.bfloat16).contiguous()
    y = _grouped_gemm(h, fc2_weight, None, plan, H, mode=0)
    if addend is not None:
        addend = addend.to(torch.bfloat16).reshape(T, H).contiguous()
    pending = PendingMoE(y, plan["scatter_index"], addend, T, k, H, orig_shape)
    return pending if defer_reduce else pending.finish()


class FusedMoeExpertFunction(torch.autograd.Function):
    """The reference's entry class (fused_moe.py:22; `QuackFusedMoeExpertFunction` :295 on sm_90 and newer) with
    its positional arguments.

    Forward: the fused pipeline above.  Backward: the reference's chain (fused_moe.py:113-265) over this
    library's operators: the forward's intermediates are recomputed step by step from the saved inputs (scatter,
    two plain grouped GEMMs, SwiGLU in torch as there), then scatter of the output gradient, three dgrad grouped
    GEMMs, three ragged-K weight gradients, the elementwise steps in torch exactly as the reference writes them, and
    the top-k sum back to tokens.  Correct against autograd of the fp32 formula; the two backward GEMM forms are
    not tuned (`group_gemm.py`)."""

    @staticmethod
    def forward(ctx, num_experts, gate_weights, expert_index, hidden_states, fc1_1_weight, fc1_2_weight, fc2_weight):
        ctx.num_experts = num_experts
        ctx.save_for_backward(gate_weights, expert_index, hidden_states, fc1_1_weight, fc1_2_weight, fc2_weight)
        return fused_moe_forward(num_experts, gate_weights, expert_index, hidden_states, fc1_1_weight, fc1_2_weight,
                                 fc2_weight)

    @staticmethod
    def backward(ctx, grad_output):
        from . import group_gemm as gg

        gate_weights, expert_index, hidden_states, w1, w2, w3 = ctx.saved_tensors
        E = ctx.num_experts
        bf = torch.bfloat16
        H = grad_output.shape[-1]
        grad_output = grad_output.reshape(-1, H).to(bf).contiguous()
        x = hidden_states.reshape(-1, H).to(bf).contiguous()
        T = x.shape[0]
        experts = expert_index.reshape(T, -1)
        k = experts.shape[1]
        w1b, w2b, w3b = (w.to(bf).contiguous() for w in (w1, w2, w3))

        # forward intermediates again, one operator at a time (same rounding points as fused_moe.py:36-99)
        cu, _, scatter_index = build_moe_indices(experts, E)
        ends = cu[1:]                                   # inclusive row count per expert
        rows = T * k
        sorted_pos = scatter_index.flatten().long()
        xs = gg.moe_scatter(x, scatter_index)           # [rows, H], expert-sorted
        gate = gg.group_gemm_same_nk(xs, w1b, ends, rows, transpose_b=True)
        up = gg.group_gemm_same_nk(xs, w2b, ends, rows, transpose_b=True)
        gate_act = torch.ops.aten.silu(gate)
        act = gate_act * up
        row_w = torch.empty((rows, 1), dtype=bf, device=x.device)
        row_w[sorted_pos] = gate_weights.to(bf).reshape(-1, 1)
        hidden_in = act * row_w                         # what fc2 consumed

        need = ctx.needs_input_grad

        def wgrad(g_rows, inputs, like, original):
            return gg.group_gemm_same_mn(g_rows, inputs, torch.empty_like(like), ends, rows, transpose_a=True,
                                         transpose_b=False).to(original.dtype)

        # through the top-k sum and fc2
        g_y = gg.moe_scatter(grad_output, scatter_index)
        g_hidden_in = gg.group_gemm_same_nk(g_y, w3b, ends, rows, transpose_b=False)
        grad_w3 = wgrad(g_y, hidden_in, w3b, w3) if need[6] else None
        # the routing weight multiplies act row by row
        g_act = g_hidden_in * row_w
        grad_gate = None
        if need[1]:
            per_row = torch.sum(act * g_hidden_in, dim=-1)
            grad_gate = per_row[sorted_pos].reshape(gate_weights.shape).to(gate_weights.dtype)
        # SwiGLU: act = silu(gate) * up
        g_up = gate_act * g_act
        g_gate = torch.ops.aten.silu_backward(g_act * up, gate)
        grad_w1 = wgrad(g_gate, xs, w1b, w1) if need[4] else None
        grad_w2 = wgrad(g_up, xs, w2b, w2) if need[5] else None
        grad_hidden = None
        if need[3]:
            g_xs = (gg.group_gemm_same_nk(g_gate, w1b, ends, rows, transpose_b=False)
                    + gg.group_gemm_same_nk(g_up, w2b, ends, rows, transpose_b=False))
            grad_hidden = gg.moe_gather(g_xs, scatter_index).reshape(hidden_states.shape).to(hidden_states.dtype)
        return None, grad_gate, None, grad_hidden, grad_w1, grad_w2, grad_w3


QuackFusedMoeExpertFunction = FusedMoeExpertFunction
_build_moe_indices = build_moe_indices
