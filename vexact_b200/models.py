"""Model-definition hooks: stock HuggingFace decoder modules running on the B200 kernels.

Stands where `vexact/models/` stands in the reference:
  * `apply_qwen3_moe_patches`   (vexact/models/qwen3_moe/modeling_qwen3_moe.py:119 `moe_block_forward`,
                                 :291 `apply_qwen3_moe_patches`)
  * `apply_deepseek_v3_patches` (vexact/models/deepseek_v3/modeling_deepseek_v3.py:185
                                 `route_tokens_to_experts`, :210 MoE forward, :409 deterministic rotary
                                 embedding, :505 `_patch_rms_norm_batch_invariant`)
  * `register_models`           (vexact/models/register.py:23)
and where the weight side of `vexact/inferencer/model_loader.py` stands:
  * `shape_from_hf_config`, `stage_weights_from_hf`: an HF module tree / state dict -> the stage
    runner's weight container, with the reference's pipeline split (`get_pp_indices`, :141).

The HF modules keep their parameters and their forward signatures.  A patched forward only replaces
the arithmetic between them by calls into libvexact_b200.so: routing, the fused experts (fused
`gate_up_proj` layout, `fc1_1_2_weight` form of `fused_moe_forward`), RMSNorm and the rotary table.
The attention projections stay `nn.Linear` (aten::mm under `enable_batch_invariant_mode()`), and
attention itself is the function registered under the reference's `ALL_ATTENTION_FUNCTIONS` keys.
The installed transformers (5.x) already stores experts as stacked `gate_up_proj [E, 2I, H]` /
`down_proj [E, H, I]`, so no module is re-created and no checkpoint key is renamed.
"""
from __future__ import annotations

import os
from typing import Iterable, Mapping, Optional, Union

import torch
import torch.nn.functional as F

from . import batch_invariant_ops as bio
from .fused_moe import fused_moe_forward, route_sigmoid_group_topk, route_softmax_topk

_PATCHED = {"qwen3_moe": False, "deepseek_v3": False}
_REGISTERED = False


# ----------------------------------------------------------------------------- Qwen3-MoE
def _qwen3_moe_block_forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
    """router Linear -> softmax(fp32) -> top-k -> renormalise -> cast -> fused experts."""
    lead = hidden_states.shape[:-1]
    x = hidden_states.reshape(-1, hidden_states.shape[-1])
    gate = self.gate
    top_k = getattr(self, "top_k", None) or gate.top_k
    norm = getattr(self, "norm_topk_prob", None)
    if norm is None:
        norm = gate.norm_topk_prob
    logits = F.linear(x, gate.weight)                      # aten::mm -> b200_gemm_bf16 under the mode switch
    weights, experts = route_softmax_topk(logits, int(top_k), bool(norm), out_dtype=x.dtype)
    num_experts = self.experts.gate_up_proj.shape[0]
    out = fused_moe_forward(num_experts, weights, experts, x, fc2_weight=self.experts.down_proj,
                            fc1_1_2_weight=self.experts.gate_up_proj)
    return out.reshape(*lead, -1)


def apply_qwen3_moe_patches() -> None:
    """Route `Qwen3MoeSparseMoeBlock.forward` through the B200 routing and fused-expert kernels."""
    if _PATCHED["qwen3_moe"]:
        return
    from transformers.models.qwen3_moe.modeling_qwen3_moe import Qwen3MoeSparseMoeBlock

    Qwen3MoeSparseMoeBlock.forward = _qwen3_moe_block_forward
    _PATCHED["qwen3_moe"] = True


# ----------------------------------------------------------------------------- DeepSeek-V3
def _deepseek_v3_moe_forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
    """fp32 router logits -> sigmoid / bias / group-limited top-k -> fused experts + shared experts."""
    lead = hidden_states.shape[:-1]
    x = hidden_states.reshape(-1, hidden_states.shape[-1])
    logits = bio.linear_f32_from_bf16(x, self.gate.weight)            # F.linear in fp32 (the router module's casts)
    experts, weights = route_sigmoid_group_topk(logits, self.gate.e_score_correction_bias, self.n_group,
                                                self.topk_group, self.top_k, bool(self.norm_topk_prob),
                                                float(self.routed_scaling_factor))
    shared = self.shared_experts(hidden_states).reshape(x.shape)       # HF MLP: three aten::mm + SiLU * up
    out = fused_moe_forward(self.experts.gate_up_proj.shape[0], weights.to(x.dtype), experts, x,
                            fc2_weight=self.experts.down_proj, fc1_1_2_weight=self.experts.gate_up_proj,
                            addend=shared)
    return out.reshape(*lead, -1)


def _deepseek_v3_rms_norm_forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
    return bio.batch_invariant_rms_norm(hidden_states, self.weight, self.variance_epsilon)


def _make_rotary_forward():
    from transformers.models.deepseek_v3.modeling_deepseek_v3 import dynamic_rope_update

    @torch.no_grad()
    @dynamic_rope_update
    def rotary_forward(self, x, position_ids):
        """cos / sin of position x inverse frequency without a library GEMM: the K = 1 batched product
        is one exact fp32 multiply per element (`triton_bmm` in the reference), so the table cannot
        depend on which cuBLAS algorithm a first call happens to pick."""
        inv = self.inv_freq[None, :, None].float().expand(position_ids.shape[0], -1, 1).to(x.device)
        pos = position_ids[:, None, :].float()
        freqs = bio.triton_bmm(inv.contiguous(), pos.contiguous()).transpose(1, 2)
        emb = torch.cat((freqs, freqs), dim=-1)
        return ((emb.cos() * self.attention_scaling).to(x.dtype), (emb.sin() * self.attention_scaling).to(x.dtype))

    return rotary_forward


def apply_deepseek_v3_patches() -> None:
    """DeepSeek-V3 / Moonlight: MoE block, RMSNorm and rotary table on the B200 kernels.

    `DeepseekV3Attention.forward` is left as transformers ships it: it already hands the attention
    function full-width keys (qk_nope + qk_rope) and unpadded values for the attention keys this
    library registers, which is the form the reference's replacement forward produces."""
    if _PATCHED["deepseek_v3"]:
        return
    import transformers.models.deepseek_v3.modeling_deepseek_v3 as hf

    hf.DeepseekV3MoE.forward = _deepseek_v3_moe_forward
    hf.DeepseekV3RMSNorm.forward = _deepseek_v3_rms_norm_forward
    hf.DeepseekV3RotaryEmbedding.forward = _make_rotary_forward()
    _PATCHED["deepseek_v3"] = True


def register_models() -> None:
    """Apply the patches once and register the attention function under the reference's keys.
    `VEXACT_DISABLE_MODEL_PATCH=1` skips the model patches, as in the reference."""
    global _REGISTERED
    if _REGISTERED:
        return
    from .attention import register_attention_functions

    register_attention_functions()
    if os.getenv("VEXACT_DISABLE_MODEL_PATCH", "0") != "1":
        apply_qwen3_moe_patches()
        apply_deepseek_v3_patches()
    _REGISTERED = True


# ----------------------------------------------------------------------------- weights
def shape_from_hf_config(cfg, name: Optional[str] = None):
    """The `ModelShape` of a Qwen3 / Qwen2 / Qwen3-MoE / DeepSeek-V3 HF config."""
    from .inferencer import MLAShape, ModelShape, MoEShape

    mt = cfg.model_type
    rope_theta = getattr(cfg, "rope_theta", None)
    if rope_theta is None:
        rope_theta = (getattr(cfg, "rope_parameters", None) or {}).get("rope_theta", 1e6)
    common = dict(num_layers=cfg.num_hidden_layers, hidden=cfg.hidden_size, num_q_heads=cfg.num_attention_heads,
                  vocab=cfg.vocab_size, rope_theta=float(rope_theta), rms_eps=float(cfg.rms_norm_eps))
    if mt in ("qwen3", "qwen2"):
        hd = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        return ModelShape(name or mt, num_kv_heads=cfg.num_key_value_heads, head_dim=hd, ffn=cfg.intermediate_size,
                          qk_norm=mt == "qwen3", qkv_bias=mt == "qwen2" or bool(getattr(cfg, "attention_bias", False)),
                          **common)
    if mt == "qwen3_moe":
        hd = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        if getattr(cfg, "mlp_only_layers", None) or getattr(cfg, "decoder_sparse_step", 1) != 1:
            raise NotImplementedError("Qwen3-MoE configs that mix dense and sparse layers are not supported")
        return ModelShape(name or mt, num_kv_heads=cfg.num_key_value_heads, head_dim=hd,
                          moe=MoEShape(cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size,
                                       bool(cfg.norm_topk_prob)), **common)
    if mt == "deepseek_v3":
        if cfg.q_lora_rank is not None:
            raise NotImplementedError("q_lora_rank is not supported by the stage runner (Moonlight uses None)")
        mla = MLAShape(cfg.kv_lora_rank, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim)
        return ModelShape(name or mt, num_kv_heads=cfg.num_attention_heads, head_dim=mla.qk_nope + mla.qk_rope,
                          ffn=cfg.intermediate_size, qk_norm=False, mla=mla, first_k_dense=cfg.first_k_dense_replace,
                          norm_single_round=True,
                          moe=MoEShape(cfg.n_routed_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size,
                                       bool(cfg.norm_topk_prob), "sigmoid_group", cfg.n_group, cfg.topk_group,
                                       float(cfg.routed_scaling_factor), cfg.n_shared_experts), **common)
    raise NotImplementedError(f"model_type {mt!r}")


def _inv_freq(shape, device):
    rd = shape.mla.qk_rope if shape.mla is not None else shape.head_dim
    return (1.0 / (shape.rope_theta ** (torch.arange(0, rd, 2, dtype=torch.int64).float() / rd))).to(device)


def stage_weights_from_hf(source: Union[torch.nn.Module, Mapping[str, torch.Tensor], Iterable], shape=None,
                          pp_rank: int = 0, pp_size: int = 1, device="cuda"):
    """Build the stage runner's weights for one pipeline rank from HF parameters.

    `source` is an HF `*ForCausalLM` module, a state dict, or an iterator of (name, tensor) pairs as the
    reference's `load_weights_from_weight_iterator` consumes (model_loader.py:87).  Names are the HF
    checkpoint names (`model.layers.N.self_attn.q_proj.weight`, ...).  Experts may come stacked
    (`mlp.experts.gate_up_proj`) or one tensor per expert and projection
    (`mlp.experts.E.gate_proj.weight`), which are fused here the way the reference's loader fuses them
    (modeling_qwen3_moe.py:193, modeling_deepseek_v3.py:330).  Only this rank's layers are kept.
    Projection weights that HF keeps as separate tensors (q, k, v; gate, up) are concatenated once.
    """
    from .inferencer import LayerWeights, StageWeights, get_pp_indices

    if isinstance(source, torch.nn.Module):
        if shape is None:
            shape = shape_from_hf_config(source.config)
        tie = bool(getattr(source.config, "tie_word_embeddings", False))
        items = dict(source.state_dict())
    else:
        items = dict(source.items()) if isinstance(source, Mapping) else dict(source)
        tie = "lm_head.weight" not in items
    if shape is None:
        raise ValueError("pass the ModelShape when loading from a bare state dict")
    start, end = get_pp_indices(shape.num_layers, pp_rank, pp_size)
    BF = torch.bfloat16

    def get(name, dtype=BF, required=True):
        t = items.get(name)
        if t is None:
            if required:
                raise KeyError(f"missing parameter {name}")
            return None
        return t.detach().to(device=device, dtype=dtype).contiguous()

    def cat(names, dtype=BF):
        return torch.cat([get(n, dtype) for n in names]).contiguous()

    def experts(prefix, m):
        gu, dn = items.get(prefix + "gate_up_proj"), items.get(prefix + "down_proj")
        if gu is not None and dn is not None:
            return get(prefix + "gate_up_proj"), get(prefix + "down_proj")
        gate_up = torch.empty((m.num_experts, 2 * m.intermediate, shape.hidden), device=device, dtype=BF)
        down = torch.empty((m.num_experts, shape.hidden, m.intermediate), device=device, dtype=BF)
        for e in range(m.num_experts):
            fused = items.get(f"{prefix}{e}.gate_up_proj.weight")
            if fused is not None:
                gate_up[e].copy_(fused)
            else:
                gate_up[e, :m.intermediate].copy_(items[f"{prefix}{e}.gate_proj.weight"])
                gate_up[e, m.intermediate:].copy_(items[f"{prefix}{e}.up_proj.weight"])
            down[e].copy_(items[f"{prefix}{e}.down_proj.weight"])
        return gate_up, down

    w = StageWeights(shape, start, end)
    for li in range(start, end):
        p = f"model.layers.{li}."
        a = p + "self_attn."
        if shape.mla is not None:
            lw = LayerWeights(input_norm=get(p + "input_layernorm.weight"), qkv=get(a + "q_proj.weight"), qkv_bias=None,
                              q_norm=None, k_norm=None, o=get(a + "o_proj.weight"),
                              post_norm=get(p + "post_attention_layernorm.weight"),
                              kv_a=get(a + "kv_a_proj_with_mqa.weight"), kv_a_norm=get(a + "kv_a_layernorm.weight"),
                              kv_b=get(a + "kv_b_proj.weight"))
        else:
            lw = LayerWeights(
                input_norm=get(p + "input_layernorm.weight"),
                qkv=cat([a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight"]),
                qkv_bias=cat([a + "q_proj.bias", a + "k_proj.bias", a + "v_proj.bias"]) if shape.qkv_bias else None,
                q_norm=get(a + "q_norm.weight") if shape.qk_norm else None,
                k_norm=get(a + "k_norm.weight") if shape.qk_norm else None,
                o=get(a + "o_proj.weight"), post_norm=get(p + "post_attention_layernorm.weight"))
        m = p + "mlp."
        if shape.layer_is_moe(li):
            moe = shape.moe
            lw.router = get(m + "gate.weight")
            lw.experts_gate_up, lw.experts_down = experts(m + "experts.", moe)
            if moe.scoring == "sigmoid_group":
                lw.router_bias = get(m + "gate.e_score_correction_bias", torch.float32)
            if moe.n_shared_experts:
                lw.shared_gate_up = cat([m + "shared_experts.gate_proj.weight", m + "shared_experts.up_proj.weight"])
                lw.shared_down = get(m + "shared_experts.down_proj.weight")
        else:
            lw.gate_up = cat([m + "gate_proj.weight", m + "up_proj.weight"])
            lw.down = get(m + "down_proj.weight")
        w.layers.append(lw)
    if pp_rank == 0:
        w.embed = get("model.embed_tokens.weight")
    if pp_rank == pp_size - 1:
        w.final_norm = get("model.norm.weight")
        w.lm_head = get("model.embed_tokens.weight") if tie else get("lm_head.weight")
    w.inv_freq = _inv_freq(shape, device)
    return w
