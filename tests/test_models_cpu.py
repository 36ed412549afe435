"""Host logic of the model-definition hooks (no GPU): HF config -> ModelShape, HF parameters ->
stage weights with the reference's pipeline split, per-expert checkpoints fused like the reference's
loaders fuse them (modeling_qwen3_moe.py:193, modeling_deepseek_v3.py:330)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def _moe_cfg():
    return transformers.Qwen3MoeConfig(hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                                       num_hidden_layers=4, vocab_size=128, num_experts=8, num_experts_per_tok=2,
                                       moe_intermediate_size=32, norm_topk_prob=True, tie_word_embeddings=False,
                                       intermediate_size=96, decoder_sparse_step=1, mlp_only_layers=[])


def test_shape_from_hf_configs():
    from vexact_b200.models import shape_from_hf_config

    s = shape_from_hf_config(_moe_cfg())
    assert (s.num_layers, s.hidden, s.num_q_heads, s.num_kv_heads, s.head_dim) == (4, 64, 4, 2, 16)
    assert (s.moe.num_experts, s.moe.top_k, s.moe.intermediate, s.moe.scoring) == (8, 2, 32, "softmax")
    d = transformers.Qwen2Config(hidden_size=64, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2,
                                 vocab_size=128, intermediate_size=96)
    s = shape_from_hf_config(d)
    assert s.qkv_bias and not s.qk_norm and s.ffn == 96 and s.head_dim == 16
    v3 = transformers.DeepseekV3Config(hidden_size=64, num_attention_heads=4, num_key_value_heads=4, num_hidden_layers=3,
                                       vocab_size=128, intermediate_size=96, moe_intermediate_size=32, n_routed_experts=8,
                                       num_experts_per_tok=2, n_shared_experts=2, kv_lora_rank=32, q_lora_rank=None,
                                       qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, first_k_dense_replace=1,
                                       n_group=2, topk_group=1, routed_scaling_factor=2.5, norm_topk_prob=True)
    s = shape_from_hf_config(v3)
    assert s.mla.kv_lora_rank == 32 and s.k_dim == 24 and s.v_dim == 16 and s.first_k_dense == 1
    assert s.moe.scoring == "sigmoid_group" and s.moe.n_group == 2 and s.moe.n_shared_experts == 2
    assert s.norm_single_round and not s.layer_is_moe(0) and s.layer_is_moe(1)


def test_stage_weights_from_hf_module_and_split_checkpoint():
    from vexact_b200.inferencer import get_pp_indices
    from vexact_b200.models import stage_weights_from_hf

    torch.manual_seed(0)
    model = transformers.Qwen3MoeForCausalLM(_moe_cfg()).to(torch.bfloat16)
    for p in model.parameters():
        p.data.normal_(0, 0.05)
    sd = model.state_dict()
    for rank in range(2):
        w = stage_weights_from_hf(model, pp_rank=rank, pp_size=2, device="cpu")
        assert (w.start_layer, w.end_layer) == get_pp_indices(4, rank, 2) and len(w.layers) == 2
        assert (w.embed is not None) == (rank == 0) and (w.lm_head is not None) == (rank == 1)
        li = w.start_layer
        lw = w.layers[0]
        pre = f"model.layers.{li}."
        assert torch.equal(lw.qkv, torch.cat([sd[pre + f"self_attn.{n}_proj.weight"] for n in "qkv"]))
        assert torch.equal(lw.experts_gate_up, sd[pre + "mlp.experts.gate_up_proj"])
        assert torch.equal(lw.router, sd[pre + "mlp.gate.weight"])
        assert lw.gate_up is None and lw.q_norm is not None
    assert torch.equal(w.lm_head, sd["lm_head.weight"])

    # a checkpoint that stores one tensor per expert and projection
    split = {k: v for k, v in sd.items() if ".experts." not in k}
    I = 32
    for li in range(4):
        gu, dn = sd[f"model.layers.{li}.mlp.experts.gate_up_proj"], sd[f"model.layers.{li}.mlp.experts.down_proj"]
        for e in range(8):
            split[f"model.layers.{li}.mlp.experts.{e}.gate_proj.weight"] = gu[e, :I].clone()
            split[f"model.layers.{li}.mlp.experts.{e}.up_proj.weight"] = gu[e, I:].clone()
            split[f"model.layers.{li}.mlp.experts.{e}.down_proj.weight"] = dn[e].clone()
    from vexact_b200.models import shape_from_hf_config

    w2 = stage_weights_from_hf(iter(split.items()), shape_from_hf_config(model.config), device="cpu")
    w1 = stage_weights_from_hf(model, device="cpu")
    for a, b in zip(w1.layers, w2.layers):
        assert torch.equal(a.experts_gate_up, b.experts_gate_up) and torch.equal(a.experts_down, b.experts_down)


def test_patches_keep_parameter_names():
    """The patched blocks keep the HF module tree (so checkpoints and weight sync see the same names)."""
    import transformers.models.deepseek_v3.modeling_deepseek_v3 as v3
    import transformers.models.qwen3_moe.modeling_qwen3_moe as q3
    from vexact_b200 import models

    saved = [(q3.Qwen3MoeSparseMoeBlock, "forward"), (v3.DeepseekV3MoE, "forward"), (v3.DeepseekV3RMSNorm, "forward"),
             (v3.DeepseekV3RotaryEmbedding, "forward")]
    saved = [(c, a, getattr(c, a)) for c, a in saved]
    before = set(transformers.Qwen3MoeForCausalLM(_moe_cfg()).state_dict())
    try:
        models.apply_qwen3_moe_patches()
        models.apply_deepseek_v3_patches()
        assert q3.Qwen3MoeSparseMoeBlock.forward is models._qwen3_moe_block_forward
        after = set(transformers.Qwen3MoeForCausalLM(_moe_cfg()).state_dict())
    finally:    # the patched forwards call CUDA kernels: put the stock ones back for the CPU tests that follow
        for c, a, f in saved:
            setattr(c, a, f)
        models._PATCHED.update(qwen3_moe=False, deepseek_v3=False)
    assert before == after
    assert {"model.layers.0.mlp.gate.weight", "model.layers.0.mlp.experts.gate_up_proj",
            "model.layers.0.mlp.experts.down_proj"} <= after
