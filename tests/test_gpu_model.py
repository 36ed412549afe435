"""GPU parity at the stage level: the decoder-stack runner vs the CPU torch model, batch /
graph / pipeline-split invariance (reference: tests/test_inferencer.py:180-297 single-process
PP ranks, :301-595 CUDA graph vs eager; tests/test_generation_regression.py PP=1 vs PP=2)."""
import dataclasses

import pytest
import torch

from oracle import cpu_model, ops

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _tiny(moe):
    from vexact_b200.inferencer import MLAShape, ModelShape, MoEShape

    if moe == "dsv3":   # DeepSeek-V3 / Moonlight layout: MLA, dense first layer, sigmoid-group routing, shared expert
        return ModelShape("tiny-dsv3", 3, 512, 4, 4, 192, 1024, ffn=256, qk_norm=False, rope_theta=50000.0,
                          mla=MLAShape(128, 128, 64, 128), first_k_dense=1, norm_single_round=True,
                          moe=MoEShape(8, 2, 128, True, "sigmoid_group", 2, 1, 2.5, 1))
    if moe:
        return ModelShape("tiny-moe", 4, 512, 8, 2, 128, 1024, moe=MoEShape(16, 4, 128))
    return ModelShape("tiny-dense", 4, 512, 4, 2, 128, 1024, ffn=768, qk_norm=False, qkv_bias=True)


def _cpu_layer(lw):
    return {k: v.cpu() for k, v in vars(lw).items() if isinstance(v, torch.Tensor)}


def _inputs(shape, q_lens, ctx_lens, page, device, seed=0):
    from vexact_b200.inferencer import StepInputs

    g = torch.Generator().manual_seed(seed)
    S = len(q_lens)
    pages = max((c + page - 1) // page for c in ctx_lens)
    ptab = torch.randperm(S * pages, generator=g).view(S, pages).to(torch.int32)
    ids, pos, slots = [], [], []
    for s in range(S):
        for p in range(ctx_lens[s] - q_lens[s], ctx_lens[s]):
            ids.append(int(torch.randint(0, shape.vocab, (1,), generator=g)))
            pos.append(p)
            slots.append(int(ptab[s, p // page]) * page + p % page)
    cu = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32)
    host = dict(input_ids=torch.tensor(ids), positions=torch.tensor(pos), slot_mapping=torch.tensor(slots, dtype=torch.int32),
                query_start_loc=cu, context_lens=torch.tensor(ctx_lens, dtype=torch.int32), block_tables=ptab)
    dev = {k: v.to(device) for k, v in host.items()}
    inp = StepInputs(input_ids=dev["input_ids"], hidden_in=None, positions=dev["positions"],
                     slot_mapping=dev["slot_mapping"], query_start_loc=dev["query_start_loc"],
                     context_lens=dev["context_lens"], block_tables=dev["block_tables"], max_seqlen_q=max(q_lens))
    return host, inp, S * pages


@pytest.mark.parametrize("moe", [False, True, "dsv3"])
def test_stage_forward_vs_cpu_model_and_invariance(moe):
    from vexact_b200.inferencer import StageRunner, StageWeights, allocate_kv_cache

    dev = torch.device("cuda")
    shape = _tiny(moe)
    w = StageWeights.random_init(shape, device=dev, seed=1, std=0.05, norm_jitter=0.05)
    page = 16
    q_lens, ctx_lens = [5, 1, 20, 1], [5, 1, 20, 1]          # a prefill step (no cached tokens yet)
    host, inp, nblocks = _inputs(shape, q_lens, ctx_lens, page, dev)
    kc, vc = allocate_kv_cache(shape, 0, shape.num_layers, nblocks, page, device=dev)
    runner = StageRunner(w, kc, vc)
    tokens, logprobs, logits = runner.step(inp)

    # CPU model with the same weights, teacher-forced layer by layer: each CPU layer gets the GPU
    # runner's own input to that layer (single-layer stages chained as pipeline ranks), so errors do
    # not compound and a routing flip (bf16 router logits tie often) stays confined to its layer.
    last = (host["query_start_loc"][1:] - 1).long()
    h_gpu = w.embed.index_select(0, inp.input_ids)
    worst_tok_frac = 0.0
    for li, lw in enumerate(w.layers):
        ws = StageWeights(shape, li, li + 1, layers=[lw], inv_freq=w.inv_freq)
        kcl, vcl = allocate_kv_cache(shape, li, li + 1, nblocks, page, device=dev)
        rr = StageRunner(ws, kcl, vcl, pp_rank=1, pp_size=3)       # a middle stage: hidden in, hidden out
        h_next = rr.step(dataclasses.replace(inp, hidden_in=h_gpu))
        kc_c = torch.zeros_like(kcl[li]).cpu()
        vc_c = torch.zeros_like(vcl[li]).cpu()
        h_cpu = cpu_model.layer_forward(shape, _cpu_layer(lw), h_gpu.cpu(), host["positions"], host["slot_mapping"],
                                        kc_c, vc_c, host["query_start_loc"], host["context_lens"],
                                        host["block_tables"])
        # K/V cache rows are roped projections of the same input: one bf16 ulp
        torch.testing.assert_close(kcl[li].cpu().float(), kc_c.float(), rtol=2 ** -6, atol=5e-2)
        torch.testing.assert_close(vcl[li].cpu().float(), vc_c.float(), rtol=2 ** -6, atol=5e-2)
        assert torch.equal(kcl[li], kc[li]) and torch.equal(vcl[li], vc[li])   # same bits as the 4-layer run
        err = (h_next.cpu().float() - h_cpu.float()).abs().amax(dim=1)
        scale_ = h_cpu.float().abs().amax().item()
        bad = (err > 2 ** -5 * scale_).float().mean().item()
        worst_tok_frac = max(worst_tok_frac, bad)
        h_gpu = h_next
    # dense: every token within tolerance; MoE: tokens whose expert choice flipped may differ
    print(f"moe={moe}: worst per-layer fraction of tokens beyond 2^-5 of max|h| = {worst_tok_frac:.3f}")
    assert worst_tok_frac <= (0.15 if moe else 0.0)
    tok_c, lp_c, logits_c = cpu_model.head_forward(shape, w.final_norm.cpu(), w.lm_head.cpu(), h_gpu.cpu()[last])
    assert torch.equal(runner.select_tokens(h_gpu, inp)[2], logits)            # chained stages == one stage
    dlogit = (logits.cpu().float() - logits_c.float()).abs().max().item()
    dlp = (logprobs.cpu() - ops.gather_logprob(logits_c, tokens.cpu())).abs().max().item()
    print(f"moe={moe}: head on the same hidden: max |dlogit| = {dlogit:.4f}, max |dlogprob| = {dlp:.4f}")
    assert dlogit < 0.07 and dlp < 0.05

    # decode step for every sequence, batched vs one by one: bitwise
    ctx2 = [c + 1 for c in ctx_lens]
    host2, inp2, _ = _inputs(shape, [1, 1, 1, 1], ctx2, page, dev)
    inp2 = dataclasses.replace(inp2, block_tables=inp.block_tables)
    inp2.slot_mapping.copy_(torch.tensor([int(inp.block_tables[s, (ctx2[s] - 1) // page]) * page + (ctx2[s] - 1) % page
                                          for s in range(4)], dtype=torch.int32))
    snap = ({i: t.clone() for i, t in kc.items()}, {i: t.clone() for i, t in vc.items()})
    tok_b, lp_b, logit_b = runner.step(inp2)
    for s in range(4):
        for i in kc:
            kc[i].copy_(snap[0][i])
            vc[i].copy_(snap[1][i])
        one = dataclasses.replace(
            inp2, input_ids=inp2.input_ids[s:s + 1], positions=inp2.positions[s:s + 1],
            slot_mapping=inp2.slot_mapping[s:s + 1], query_start_loc=torch.tensor([0, 1], dtype=torch.int32, device=dev),
            context_lens=inp2.context_lens[s:s + 1], block_tables=inp2.block_tables[s:s + 1].contiguous())
        t1, l1, g1 = runner.step(one)
        assert torch.equal(g1[0], logit_b[s]) and torch.equal(l1[0], lp_b[s]) and t1[0] == tok_b[s]


def test_cuda_graph_equals_eager_and_pp_split_equals_single_stage():
    from vexact_b200.inferencer import StageRunner, StageWeights, allocate_kv_cache, get_pp_indices

    dev = torch.device("cuda")
    shape = _tiny(True)
    page = 16
    host, inp, nblocks = _inputs(shape, [3, 1, 7], [3, 1, 7], page, dev, seed=2)
    w = StageWeights.random_init(shape, device=dev, seed=3, std=0.05)
    kc, vc = allocate_kv_cache(shape, 0, shape.num_layers, nblocks, page, device=dev)
    runner = StageRunner(w, kc, vc)
    tok, lp, logits = [t.clone() for t in runner.step(inp)]
    graph, out = runner.capture(inp)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out[2], logits) and torch.equal(out[1], lp) and torch.equal(out[0], tok)

    # two pipeline stages run back to back in one process, each with its own layers' KV
    stage_out = None
    for r in range(2):
        s0, s1 = get_pp_indices(shape.num_layers, r, 2)
        ws = StageWeights(shape, s0, s1, layers=w.layers[s0:s1], embed=w.embed if r == 0 else None,
                          final_norm=w.final_norm if r == 1 else None, lm_head=w.lm_head if r == 1 else None,
                          inv_freq=w.inv_freq)
        kcs, vcs = allocate_kv_cache(shape, s0, s1, nblocks, page, device=dev)
        rr = StageRunner(ws, kcs, vcs, pp_rank=r, pp_size=2)
        stage_out = rr.step(dataclasses.replace(inp, hidden_in=stage_out))
    assert torch.equal(stage_out[2], logits) and torch.equal(stage_out[0], tok)


def test_hf_dropin_attention_and_aten_overrides():
    """A stock HF Qwen3 model under enable_batch_invariant_mode() with the attention function
    registered under the reference's key runs on these kernels and agrees with the stage runner."""
    transformers = pytest.importorskip("transformers")
    import vexact_b200 as vb
    from vexact_b200.attention import register_attention_functions
    from vexact_b200.inferencer import ModelShape, StageRunner, StageWeights, allocate_kv_cache

    dev = torch.device("cuda")
    cfg = transformers.Qwen3Config(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                                   intermediate_size=768, num_hidden_layers=2, vocab_size=1024, rope_theta=1e6,
                                   rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)
    register_attention_functions()
    cfg._attn_implementation = "fa-invariant"
    torch.manual_seed(0)
    model = transformers.Qwen3ForCausalLM(cfg).to(BF).to(dev).eval()
    shape = ModelShape("hf-tiny", 2, 512, 4, 2, 128, 1024, ffn=768)
    w = StageWeights(shape, 0, 2)
    from vexact_b200.inferencer import LayerWeights

    for layer in model.model.layers:
        a, m = layer.self_attn, layer.mlp
        w.layers.append(LayerWeights(
            input_norm=layer.input_layernorm.weight.data, post_norm=layer.post_attention_layernorm.weight.data,
            qkv=torch.cat([a.q_proj.weight.data, a.k_proj.weight.data, a.v_proj.weight.data]).contiguous(),
            qkv_bias=None, q_norm=a.q_norm.weight.data, k_norm=a.k_norm.weight.data, o=a.o_proj.weight.data,
            gate_up=torch.cat([m.gate_proj.weight.data, m.up_proj.weight.data]).contiguous(), down=m.down_proj.weight.data))
    w.embed, w.final_norm, w.lm_head = model.model.embed_tokens.weight.data, model.model.norm.weight.data, model.lm_head.weight.data
    w.inv_freq = (1.0 / (1e6 ** (torch.arange(0, 128, 2, dtype=torch.int64).float() / 128))).to(dev)
    page = 16
    host, inp, nblocks = _inputs(shape, [6, 1, 9], [6, 1, 9], page, dev, seed=4)
    kc, vc = allocate_kv_cache(shape, 0, 2, nblocks, page, device=dev)
    _, _, logits = StageRunner(w, kc, vc).step(inp)

    kc2, vc2 = allocate_kv_cache(shape, 0, 2, nblocks, page, device=dev)
    vb.set_kv_cache_context(is_paged_attn=True, key_cache=kc2, value_cache=vc2, block_tables=inp.block_tables,
                            context_lens=inp.context_lens, slot_mapping=inp.slot_mapping,
                            query_start_loc=inp.query_start_loc, max_seqlen_q=inp.max_seqlen_q)
    with torch.inference_mode(), vb.set_batch_invariant_mode(True):
        out = model(input_ids=inp.input_ids[None], position_ids=inp.positions[None], use_cache=False)
    last = (inp.query_start_loc[1:] - 1).long()
    hf_logits = out.logits[0, last]
    d = (hf_logits.float() - logits.float()).abs().max().item()
    print(f"HF drop-in vs stage runner: max |dlogit| = {d:.5f}")
    assert d < 0.06
    for li in kc:
        # the HF module normalises through the aten::mean.dim override (another summation tree)
        # (rope adds two rounded products that may cancel: absolute tolerance of ~2 ulp of the inputs)
        torch.testing.assert_close(vc[li].float(), vc2[li].float(), rtol=2 ** -6, atol=5e-2)
        torch.testing.assert_close(kc[li].float(), kc2[li].float(), rtol=2 ** -6, atol=5e-2)


@pytest.mark.gpu
def test_dense_mlp_routes_agree_bitwise():
    """The dense MLP runs fused (few tokens) or as two GEMMs + an elementwise kernel (many tokens):
    a token must get the same bits on both routes."""
    from vexact_b200.inferencer import QWEN3_1P7B, ModelShape, StageRunner, StageWeights, allocate_kv_cache

    shape = ModelShape(**{**QWEN3_1P7B.__dict__, "num_layers": 1})
    w = StageWeights.random_init(shape, 0, 1, device="cuda", seed=3)
    kc, vc = allocate_kv_cache(shape, 0, 1, 4, 16, device="cuda")
    r = StageRunner(w, kc, vc, 0, 1)
    g = torch.Generator().manual_seed(12)
    x = torch.randn(300, shape.hidden, generator=g).bfloat16().cuda()
    lw = w.layers[0]
    big = r._dense_mlp(x, lw.gate_up, lw.down, shape.ffn)                 # 300 tokens: split route
    small = r._dense_mlp(x[:64], lw.gate_up, lw.down, shape.ffn)         # 64 tokens: fused route
    one = r._dense_mlp(x[17:18], lw.gate_up, lw.down, shape.ffn)
    assert torch.equal(big[:64], small) and torch.equal(big[17:18], one)
