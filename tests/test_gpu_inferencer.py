"""The reference-shaped entry points on the GPU: `Inferencer.infer(requests)` over `InputBuffers`,
`CudaGraphManager` buckets and `PPMessager`-shaped hand-off (reference: tests/test_inferencer.py:180-297
single-process pipeline ranks, :301-595 CUDA graph vs eager bitwise)."""
from types import SimpleNamespace as NS

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"


def _shape():
    from vexact_b200.inferencer import ModelShape, MoEShape

    return ModelShape("tiny-moe", 4, 512, 8, 2, 128, 1024, moe=MoEShape(16, 4, 128))


def _config(shape, eager):
    from vexact_b200.config import CacheConfig, EngineConfig, ModelConfig, SchedulerConfig

    hf = NS(num_key_value_heads=shape.num_kv_heads, head_dim=shape.head_dim, hidden_size=shape.hidden,
            num_attention_heads=shape.num_q_heads, num_hidden_layers=shape.num_layers)
    return EngineConfig(model=ModelConfig(hf_config=hf, max_model_len=256, enforce_eager=eager),
                        cache=CacheConfig(page_size=16, max_cache_blocks=64),
                        scheduler=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=32))


def _requests(shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    cfg = NS(do_sample=False, temperature=1.0, top_k=None, top_p=1.0, output_scores=True, output_logits=True, seed=None)
    reqs, next_block = [], 0
    for i, n in enumerate([5, 9, 3]):
        ids = torch.randint(0, shape.vocab, (n,), generator=g).tolist()
        reqs.append(NS(request_id=f"r{i}", input_ids_list=ids, tokens_this_step=n, num_computed_tokens=n,
                       block_ids=[next_block], generated_tokens=[], generation_config=cfg))
        next_block += 2          # leave room for a second block per request
    return reqs


def _advance(reqs, tokens):
    """What the scheduler does between steps: append the token, plan one decode token, grow the block list."""
    for r, t in zip(reqs, tokens.tolist()):
        r.generated_tokens.append(int(t))
        r.tokens_this_step = 1
        r.num_computed_tokens += 1
        if (r.num_computed_tokens + 15) // 16 > len(r.block_ids):
            r.block_ids.append(r.block_ids[-1] + 1)


class _Loopback:
    """In-process stand-in for the messager between two single-process pipeline ranks."""

    def __init__(self):
        self.ctx, self.out = [], []

    def send_gen_ctx(self, c):
        import dataclasses
        self.ctx.append(dataclasses.replace(c, intermediate_tensors=c.intermediate_tensors.clone()))

    def recv_gen_ctx(self):
        return self.ctx.pop(0)

    def send_infer_out(self, o):
        self.out.append(o)

    def recv_infer_out(self):
        return self.out.pop(0)


def _run(inferencers, steps=4):
    """Drive prefill + decode steps through a chain of single-process pipeline ranks."""
    shape = _shape()
    reqs = _requests(shape)
    history = []
    for _ in range(steps):
        out = None
        for k, inf in enumerate(inferencers):
            res = inf.infer(reqs if k == 0 else [], recv_infer_out=False)
            if res is not None:
                out = res
        if out is None:                       # multi-rank chain: the last rank handed its output to the loopback
            out = inferencers[0]._pp_messager.recv_infer_out()
        history.append((out.token_ids.clone(), out.logprobs.clone(), out.logits.clone()))
        _advance(reqs, out.token_ids)
    torch.cuda.synchronize()
    return history


def _make(shape, weights_for, pp_size, eager, messager=None):
    from vexact_b200.config import PPInfo
    from vexact_b200.inferencer import Inferencer, StageModel

    out = []
    for r in range(pp_size):
        model = StageModel(weights_for(r, pp_size), r, pp_size)
        out.append(Inferencer(model, _config(shape, eager), PPInfo(pp_size, r), messager, torch.device(DEV),
                              enable_batch_invariant=False))
    return out


def test_bucket_graph_replay_equals_eager_and_pipeline_split_bitwise():
    from vexact_b200 import _lib
    from vexact_b200.cudagraph_utils import CudaGraphManager
    from vexact_b200.inferencer import StageWeights, get_pp_indices

    shape = _shape()
    full = StageWeights.random_init(shape, device=DEV, seed=5, std=0.05)

    def weights_for(rank, pp):
        s0, s1 = get_pp_indices(shape.num_layers, rank, pp)
        return StageWeights(shape, s0, s1, layers=full.layers[s0:s1], embed=full.embed if rank == 0 else None,
                            final_norm=full.final_norm if rank == pp - 1 else None,
                            lm_head=full.lm_head if rank == pp - 1 else None, inv_freq=full.inv_freq)

    assert CudaGraphManager.build_capture_sizes(32) == [1, 2, 4, 8, 16, 32]
    eager = _run(_make(shape, weights_for, 1, eager=True))
    graph_inf = _make(shape, weights_for, 1, eager=False)
    mgr = graph_inf[0]._cudagraph_mgr
    # prefill of 17 tokens / 3 sequences -> the 32-token bucket (8 sequences); decode of 3 -> the 4-sequence decode graph
    d = mgr.dispatch(3, 17, 9)
    assert (d.num_tokens, d.num_seqs, d.decode) == (32, 8, False)
    d = mgr.dispatch(3, 3, 1)
    assert (d.num_tokens, d.num_seqs, d.decode) == (4, 4, True)
    assert mgr.dispatch(9, 9, 1) is None or mgr.dispatch(9, 9, 1).num_seqs >= 9
    graph = _run(graph_inf)
    lo = _Loopback()
    split = _run(_make(shape, weights_for, 2, eager=False, messager=lo))
    for step, (a, b, c) in enumerate(zip(eager, graph, split)):
        for x, y, z, what in zip(a, b, c, ("tokens", "logprobs", "logits")):
            assert torch.equal(x, y), f"step {step}: padded-bucket graph replay differs from eager in {what}"
            assert torch.equal(x, z), f"step {step}: two pipeline ranks differ from one in {what}"
    assert _lib.read_status()[0] == 0


def test_hf_module_through_the_inferencer_matches_stage_model():
    """A stock HF Qwen3-MoE module (patched by apply_qwen3_moe_patches) and the native stage on weights loaded from
    it go through the same Inferencer and agree within the bf16 tolerance of the HF drop-in test."""
    transformers = pytest.importorskip("transformers")
    import vexact_b200 as vb
    from vexact_b200.config import PPInfo
    from vexact_b200.inferencer import HFModel, Inferencer, StageModel
    from vexact_b200.attention import register_attention_functions
    from vexact_b200.models import apply_qwen3_moe_patches, shape_from_hf_config, stage_weights_from_hf

    register_attention_functions()
    apply_qwen3_moe_patches()
    cfg = transformers.Qwen3MoeConfig(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                                      num_hidden_layers=2, vocab_size=1024, num_experts=16, num_experts_per_tok=4,
                                      moe_intermediate_size=128, norm_topk_prob=True, tie_word_embeddings=False,
                                      intermediate_size=256, decoder_sparse_step=1, mlp_only_layers=[],
                                      rope_theta=1e6, rms_norm_eps=1e-6, max_position_embeddings=4096)
    cfg._attn_implementation = "fa-invariant"
    with torch.device(DEV):
        model = transformers.Qwen3MoeForCausalLM(cfg).to(BF).eval()
    g = torch.Generator(device=DEV).manual_seed(3)
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            p.normal_(0.0, 0.05, generator=g)
            if "norm" in name:
                p.add_(1.0)
    shape = shape_from_hf_config(cfg)
    econf = _config(shape, eager=True)
    econf.model.hf_config = cfg
    try:
        hf_inf = Inferencer(HFModel(model), econf, PPInfo(1, 0), None, torch.device(DEV), enable_batch_invariant=True)
        hf = _run([hf_inf], steps=3)
    finally:
        vb.disable_batch_invariant_mode()
        torch.use_deterministic_algorithms(False)
    st_inf = Inferencer(StageModel(stage_weights_from_hf(model, shape, device=DEV)), econf, PPInfo(1, 0), None,
                        torch.device(DEV), enable_batch_invariant=False)
    st = _run([st_inf], steps=3)
    # step 0 sees identical inputs on both sides; later steps feed each side's own greedy tokens
    d = (hf[0][2].float() - st[0][2].float()).abs().max().item()
    print(f"HF module vs native stage through the Inferencer: max |dlogit| = {d:.4f}")
    assert d < 0.08
    assert (hf[0][1] - st[0][1]).abs().max().item() < 0.05 or not torch.equal(hf[0][0], st[0][0])


def test_hf_module_split_over_two_pipeline_ranks_equals_one_rank_bitwise():
    """`HFModel(hf_model, pp_info)` slices a stock HF module tree the way the reference's `_apply_pp` does
    (missing layers pass their input on, embedding on the first rank, norm + lm_head on the last); two such ranks
    chained in one process give the single-rank bits (reference: tests/test_inferencer.py:180-297)."""
    transformers = pytest.importorskip("transformers")
    import copy

    import vexact_b200 as vb
    from vexact_b200.attention import register_attention_functions
    from vexact_b200.config import PPInfo
    from vexact_b200.inferencer import HFModel, Inferencer
    from vexact_b200.models import shape_from_hf_config

    register_attention_functions()
    cfg = transformers.Qwen3Config(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                                   num_hidden_layers=4, vocab_size=1024, intermediate_size=768,
                                   tie_word_embeddings=False, rope_theta=1e6, rms_norm_eps=1e-6,
                                   max_position_embeddings=4096)
    cfg._attn_implementation = "fa-invariant"
    with torch.device(DEV):
        model = transformers.Qwen3ForCausalLM(cfg).to(BF).eval()
    g = torch.Generator(device=DEV).manual_seed(9)
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            p.normal_(0.0, 0.05, generator=g)
            if "norm" in name:
                p.add_(1.0)
    shape = shape_from_hf_config(cfg)
    econf = _config(shape, eager=True)
    econf.model.hf_config = cfg
    try:
        one = _run([Inferencer(HFModel(copy.deepcopy(model)), econf, PPInfo(1, 0), None, torch.device(DEV),
                               enable_batch_invariant=True)], steps=3)
        lo = _Loopback()
        ranks = [Inferencer(HFModel(copy.deepcopy(model), PPInfo(2, r)), econf, PPInfo(2, r), lo, torch.device(DEV),
                            enable_batch_invariant=True) for r in range(2)]
        assert ranks[0].model.layer_ids == [0, 1] and ranks[1].model.layer_ids == [2, 3]
        two = _run(ranks, steps=3)
        # the same module replayed from captured bucket graphs (reference: tests/test_inferencer.py:301-595)
        gconf = _config(shape, eager=False)
        gconf.model.hf_config = cfg
        graph = _run([Inferencer(HFModel(copy.deepcopy(model)), gconf, PPInfo(1, 0), None, torch.device(DEV),
                                 enable_batch_invariant=True)], steps=3)
        # the reference's own wrapper class and constructor (model_loader.py:218): base model + lm_head + position
        from vexact_b200.inferencer import TransformersForCausalLM
        m = copy.deepcopy(model)
        wrapped = _run([Inferencer(TransformersForCausalLM(m.model, m.lm_head, PPInfo(1, 0)), gconf, PPInfo(1, 0), None,
                                   torch.device(DEV), enable_batch_invariant=True)], steps=3)
    finally:
        vb.disable_batch_invariant_mode()
        torch.use_deterministic_algorithms(False)
    for step, (a, b, c, d) in enumerate(zip(one, two, graph, wrapped)):
        for x, y, z, w, what in zip(a, b, c, d, ("tokens", "logprobs", "logits")):
            assert torch.equal(x, y), f"step {step}: two HF pipeline ranks differ from one in {what}"
            assert torch.equal(x, z), f"step {step}: the HF module replayed from a bucket graph differs from eager in {what}"
            assert torch.equal(x, w), f"step {step}: TransformersForCausalLM differs from HFModel in {what}"


def test_attn_impl_flex_gives_the_other_keys_bits_and_refuses_graphs():
    """`attn_impl="flex"` (reference inferencer.py:52, :108-109): a stock HF module whose attention key is `flex`
    runs the paged kernel like the other three keys (same bits through the Inferencer, eager), and asking for
    CUDA graphs with it raises the reference's RuntimeError."""
    transformers = pytest.importorskip("transformers")
    import copy

    import vexact_b200 as vb
    from vexact_b200.attention import register_attention_functions
    from vexact_b200.config import PPInfo
    from vexact_b200.inferencer import HFModel, Inferencer
    from vexact_b200.models import shape_from_hf_config

    register_attention_functions()
    cfg = transformers.Qwen3Config(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                                   num_hidden_layers=2, vocab_size=1024, intermediate_size=768,
                                   tie_word_embeddings=False, rope_theta=1e6, rms_norm_eps=1e-6,
                                   max_position_embeddings=4096)
    outs = {}
    try:
        for key in ("triton-invariant", "flex"):
            c = copy.deepcopy(cfg)
            c._attn_implementation = key
            with torch.device(DEV):
                model = transformers.Qwen3ForCausalLM(c).to(BF).eval()
            g = torch.Generator(device=DEV).manual_seed(13)
            with torch.no_grad():
                for name, p in sorted(model.named_parameters()):
                    p.normal_(0.0, 0.05, generator=g)
                    if "norm" in name:
                        p.add_(1.0)
            shape = shape_from_hf_config(c)
            econf = _config(shape, eager=True)
            econf.model.hf_config = c
            econf.model.attn_impl = key
            outs[key] = _run([Inferencer(HFModel(model), econf, PPInfo(1, 0), None, torch.device(DEV),
                                         enable_batch_invariant=True)], steps=2)
        gconf = _config(shape, eager=False)
        gconf.model.hf_config = c
        gconf.model.attn_impl = "flex"
        with pytest.raises(RuntimeError, match="flex attention is not supported for CUDA graph"):
            Inferencer(HFModel(model), gconf, PPInfo(1, 0), None, torch.device(DEV), enable_batch_invariant=True)
    finally:
        vb.disable_batch_invariant_mode()
        torch.use_deterministic_algorithms(False)
    for a, b in zip(outs["triton-invariant"], outs["flex"]):
        for x, y in zip(a, b):
            assert torch.equal(x, y)


@pytest.mark.parametrize("moe", [False, True, "deepseek_v3", "qwen2"])
def test_rollout_steps_equal_one_shot_prefill_of_the_same_sequences_bitwise(moe):
    """What the engine promises the trainer (reference: tests/scripts/verify_logits_vs_native_hf.py with
    --rtol 0 --atol 0): the logits a request got at decode step k, batched with other requests and running on
    cached keys, are the bits a fresh forward over its whole sequence (prompt + the k tokens generated so far)
    gives at the last position.  Stock HF module under the mode switch, three requests, three decode steps."""
    transformers = pytest.importorskip("transformers")
    import vexact_b200 as vb
    from vexact_b200.attention import register_attention_functions
    from vexact_b200.config import PPInfo
    from vexact_b200.inferencer import HFModel, Inferencer
    from vexact_b200.models import shape_from_hf_config

    register_attention_functions()
    if moe == "deepseek_v3":   # MLA (keys 192 wide, values 128) + sigmoid-group routing + shared experts, patched
        from vexact_b200.models import apply_deepseek_v3_patches

        apply_deepseek_v3_patches()
        cfg = transformers.DeepseekV3Config(hidden_size=512, num_attention_heads=4, num_key_value_heads=4,
                                            num_hidden_layers=2, vocab_size=1024, intermediate_size=256,
                                            moe_intermediate_size=128, n_routed_experts=16, num_experts_per_tok=4,
                                            n_shared_experts=1, kv_lora_rank=64, q_lora_rank=None,
                                            qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                                            first_k_dense_replace=1, n_group=2, topk_group=1,
                                            routed_scaling_factor=2.5, norm_topk_prob=True, tie_word_embeddings=False,
                                            rms_norm_eps=1e-6, max_position_embeddings=4096)
        cls = transformers.DeepseekV3ForCausalLM
    elif moe == "qwen2":       # q/k/v projections with a bias (aten::addmm), no q/k norm
        cfg = transformers.Qwen2Config(hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
                                       num_hidden_layers=3, vocab_size=1024, intermediate_size=768,
                                       tie_word_embeddings=False, rope_theta=1e6, rms_norm_eps=1e-6,
                                       max_position_embeddings=4096)
        cls = transformers.Qwen2ForCausalLM
    elif moe:    # the MoE block runs through apply_qwen3_moe_patches(): routing kernel + fused MoE
        from vexact_b200.models import apply_qwen3_moe_patches

        apply_qwen3_moe_patches()
        cfg = transformers.Qwen3MoeConfig(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                                          num_hidden_layers=2, vocab_size=1024, num_experts=16, num_experts_per_tok=4,
                                          moe_intermediate_size=128, norm_topk_prob=True, tie_word_embeddings=False,
                                          intermediate_size=256, decoder_sparse_step=1, mlp_only_layers=[],
                                          rope_theta=1e6, rms_norm_eps=1e-6, max_position_embeddings=4096)
        cls = transformers.Qwen3MoeForCausalLM
    else:
        cfg = transformers.Qwen3Config(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                                       num_hidden_layers=3, vocab_size=1024, intermediate_size=768,
                                       tie_word_embeddings=False, rope_theta=1e6, rms_norm_eps=1e-6,
                                       max_position_embeddings=4096)
        cls = transformers.Qwen3ForCausalLM
    cfg._attn_implementation = "fa-invariant"
    with torch.device(DEV):
        model = cls(cfg).to(BF).eval()
    g = torch.Generator(device=DEV).manual_seed(13)
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            p.normal_(0.0, 0.05, generator=g)
            if "norm" in name:
                p.add_(1.0)
    shape = shape_from_hf_config(cfg)
    econf = _config(shape, eager=True)
    econf.model.hf_config = cfg
    steps = 4
    try:
        rollout = _run([Inferencer(HFModel(model), econf, PPInfo(1, 0), None, torch.device(DEV),
                                   enable_batch_invariant=True)], steps=steps)
        prompts = [r.input_ids_list for r in _requests(shape)]
        for k in range(1, steps):
            # every request's sequence so far, as one fresh prefill (a new inferencer: empty cache)
            reqs = _requests(shape)
            for i, r in enumerate(reqs):
                ids = prompts[i] + [int(rollout[j][0][i]) for j in range(k)]
                r.input_ids_list, r.tokens_this_step, r.num_computed_tokens = ids, len(ids), len(ids)
            fresh = Inferencer(HFModel(model), econf, PPInfo(1, 0), None, torch.device(DEV),
                               enable_batch_invariant=True)
            out = fresh.infer(reqs, recv_infer_out=False)
            assert torch.equal(out.logits, rollout[k][2]), f"decode step {k}: logits differ from the one-shot forward"
            assert torch.equal(out.logprobs, rollout[k][1]) and torch.equal(out.token_ids, rollout[k][0])
        # chunked prefill (reference: scripts/run_batch_invariant_tests.sh, "random prompts + chunked prefill"):
        # request 1's nine prompt tokens arrive as 4 + 5 while the other two requests prefill and then decode
        reqs = _requests(shape)
        reqs[1].tokens_this_step, reqs[1].num_computed_tokens = 4, 4
        chunked = Inferencer(HFModel(model), econf, PPInfo(1, 0), None, torch.device(DEV), enable_batch_invariant=True)
        first = chunked.infer(reqs, recv_infer_out=False)
        assert torch.equal(first.logits[0], rollout[0][2][0]) and torch.equal(first.logits[2], rollout[0][2][2])
        for i in (0, 2):                                   # requests 0 and 2 go on to their first decode step
            r = reqs[i]
            r.generated_tokens.append(int(first.token_ids[i]))
            r.tokens_this_step, r.num_computed_tokens = 1, r.num_computed_tokens + 1
        reqs[1].tokens_this_step, reqs[1].num_computed_tokens = 5, 9
        second = chunked.infer(reqs, recv_infer_out=False)
        assert torch.equal(second.logits[1], rollout[0][2][1]), "a prompt prefilled in two chunks differs from one shot"
        assert torch.equal(second.logits[0], rollout[1][2][0]) and torch.equal(second.logits[2], rollout[1][2][2])
    finally:
        vb.disable_batch_invariant_mode()
        torch.use_deterministic_algorithms(False)
