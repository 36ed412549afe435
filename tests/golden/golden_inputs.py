"""Seeded input builders shared by the GPU-side fixture generator (make_reference_gpu_golden.py)
and the tests that replay its fixtures (tests/test_gpu_reference_parity.py).

A fixture made on the GPU box stores the reference's OUTPUTS plus the case description; the inputs
are rebuilt from the description with CPU generators (identical bits on every machine with the same
torch), and a checksum stored with the fixture guards against a generator that ever changes.
"""
from __future__ import annotations

import torch

BF = torch.bfloat16


def randn(shape, seed: int, std: float = 1.0, dtype=BF) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def checksum(*tensors) -> int:
    """Order-sensitive checksum over the raw 32-bit words of the tensors (three strided sums each)."""
    total = 0
    for t in tensors:
        b = t.detach().cpu().contiguous().view(torch.uint8).flatten()
        pad = (-b.numel()) % 4
        if pad:
            b = torch.cat([b, torch.zeros(pad, dtype=torch.uint8)])
        v = b.view(torch.int32)
        s1, s2, s3 = (int(x.sum(dtype=torch.int64)) for x in (v, v[::3], v[1::5]))
        total = (total * 1000003 + s1 * 31 + s2 * 17 + s3) % (1 << 61)
    return total


# ---- op-level cases -------------------------------------------------------------------------------
MATMUL_CASES = [  # (M, K, N, with_bias)
    dict(M=1, K=2048, N=768), dict(M=7, K=2048, N=768), dict(M=64, K=2048, N=768), dict(M=256, K=2048, N=768),
    dict(M=33, K=512, N=200), dict(M=300, K=1536, N=256),
]


def matmul_inputs(case, seed=11):
    a = randn((case["M"], case["K"]), seed)
    w = randn((case["N"], case["K"]), seed + 1, 0.02)
    bias = randn((case["N"],), seed + 2, 0.5)
    return a, w, bias


RMSNORM_CASES = [dict(rows=5, n=2048), dict(rows=3, n=128), dict(rows=4, n=512), dict(rows=64, n=2048)]


def rmsnorm_inputs(case, seed=21):
    x = randn((case["rows"], case["n"]), seed)
    w = (1 + 0.02 * torch.randn(case["n"], generator=torch.Generator().manual_seed(seed + 1))).to(BF)
    return x, w


LOGITS_CASES = [dict(rows=4, n=151936), dict(rows=3, n=4097), dict(rows=2, n=1000)]


def logits_inputs(case, seed=31):
    x = randn((case["rows"], case["n"]), seed, 2.0, torch.float32)
    g = torch.Generator().manual_seed(seed + 1)
    labels = torch.randint(0, case["n"], (case["rows"],), generator=g)
    cols = torch.randperm(case["n"], generator=g)[:2048].sort().values   # the columns a fixture keeps
    return x, labels, cols


ATTENTION_CASES = [
    # decode, GQA 2, 16-token pages
    dict(name="decode_gqa2_page16", hq=16, hkv=8, dk=128, dv=128, page=16, q_lens=[1, 1, 1, 1], ctx=[300, 17, 128, 1]),
    # prefill + chunk + decode mixed, GQA 8, 16-token pages (the config-4 head shape)
    dict(name="mixed_gqa8_page16", hq=32, hkv=4, dk=128, dv=128, page=16, q_lens=[130, 40, 1, 7], ctx=[130, 200, 257, 7]),
    # the reference's default page size
    dict(name="prefill_page256", hq=16, hkv=8, dk=128, dv=128, page=256, q_lens=[300, 1], ctx=[300, 513]),
    # MLA dims
    dict(name="mla_192_128", hq=4, hkv=4, dk=192, dv=128, page=16, q_lens=[33, 1, 1], ctx=[33, 100, 64]),
]


def attention_inputs(case, seed=41):
    g = torch.Generator().manual_seed(seed)
    S = len(case["ctx"])
    page = case["page"]
    pages = max((c + page - 1) // page for c in case["ctx"])
    nblocks = S * pages + 1
    kc = randn((nblocks, page, case["hkv"], case["dk"]), seed + 1)
    vc = randn((nblocks, page, case["hkv"], case["dv"]), seed + 2)
    table = torch.randperm(S * pages, generator=g).view(S, pages).to(torch.int32)
    q = randn((sum(case["q_lens"]), case["hq"], case["dk"]), seed + 3)
    cu = torch.tensor([0] + torch.tensor(case["q_lens"]).cumsum(0).tolist(), dtype=torch.int32)
    used = torch.tensor(case["ctx"], dtype=torch.int32)
    return q, kc, vc, cu, used, table


MOE_CASES = [
    dict(name="small", T=64, E=16, k=4, H=512, I=256),
    dict(name="ragged", T=37, E=32, k=6, H=1024, I=384),
    dict(name="cfg4_width", T=96, E=32, k=8, H=2048, I=768),
]


def moe_inputs(case, seed=51):
    T, E, k, H, I = (case[x] for x in ("T", "E", "k", "H", "I"))
    hidden = randn((T, H), seed)
    gate_up = randn((E, 2 * I, H), seed + 1, 0.02)
    down = randn((E, H, I), seed + 2, 0.02)
    router = randn((E, H), seed + 3, 0.02)
    return hidden, gate_up, down, router


KV_STORE_CASE = dict(T=9, heads=2, dk=192, dv=128, blocks=5, page=16)


def kv_store_inputs(case=KV_STORE_CASE, seed=61):
    g = torch.Generator().manual_seed(seed)
    key = randn((case["T"], case["heads"], case["dk"]), seed + 1)
    value = randn((case["T"], case["heads"], case["dv"]), seed + 2)
    slots = torch.randperm(case["blocks"] * case["page"], generator=g)[:case["T"]].to(torch.int32)
    slots[3] = -1
    return key, value, slots


def reinit_parameters(model, seed: int, std: float = 0.02) -> None:
    """Overwrite every parameter of an HF module from one seeded device generator, in name order, so that
    the weights depend only on (names, shapes, seed) and not on which class constructed the module or on
    how its constructor consumed random numbers.  Norm weights become 1 + N(0, std), the rest N(0, std)."""
    dev = next(model.parameters()).device
    g = torch.Generator(device=dev).manual_seed(seed)
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            p.normal_(0.0, std, generator=g)
            if name.endswith("norm.weight") or "layernorm" in name:
                p.add_(1.0)


def dense_model_config():
    import transformers

    return transformers.Qwen3Config(hidden_size=2048, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                                    intermediate_size=6144, num_hidden_layers=28, vocab_size=151936, rope_theta=1e6,
                                    rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960,
                                    initializer_range=0.02)


def moe_model_config(layers: int = 2):
    import transformers

    return transformers.Qwen3MoeConfig(hidden_size=2048, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                                       num_hidden_layers=layers, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                                       num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                                       norm_topk_prob=True, tie_word_embeddings=False, max_position_embeddings=40960,
                                       initializer_range=0.02, intermediate_size=6144, decoder_sparse_step=1,
                                       mlp_only_layers=[])


class Steps:
    """Seeded requests -> packed step inputs (one prefill step, then decode steps) on a shared page table."""

    def __init__(self, prompt_lens, vocab, page, seed, device):
        g = torch.Generator().manual_seed(seed)
        self.S, self.page, self.device = len(prompt_lens), page, device
        self.prompt_lens = list(prompt_lens)
        self.prompts = [torch.randint(0, vocab, (n,), generator=g) for n in prompt_lens]
        self.max_len = max(prompt_lens) + 16
        pages = (self.max_len + page - 1) // page
        self.table = torch.randperm(self.S * pages, generator=g).view(self.S, pages).to(torch.int32)
        self.nblocks = self.S * pages

    def step(self, tokens_per_seq, start_pos):
        """tokens_per_seq[s]: 1-D token tensor fed for sequence s, starting at position start_pos[s]."""
        ids, pos, slots, cu, ctx = [], [], [], [0], []
        for s, toks in enumerate(tokens_per_seq):
            n = len(toks)
            p = torch.arange(start_pos[s], start_pos[s] + n)
            ids.append(toks.cpu())
            pos.append(p)
            slots.append(self.table[s, (p // self.page)].long() * self.page + p % self.page)
            cu.append(cu[-1] + n)
            ctx.append(start_pos[s] + n)
        d = self.device
        return dict(input_ids=torch.cat(ids).to(d), positions=torch.cat(pos).to(d),
                    slot_mapping=torch.cat(slots).to(torch.int32).to(d),
                    query_start_loc=torch.tensor(cu, dtype=torch.int32, device=d),
                    context_lens=torch.tensor(ctx, dtype=torch.int32, device=d), block_tables=self.table.to(d),
                    max_seqlen_q=max(len(t) for t in tokens_per_seq))

    def prefill(self):
        return self.step(self.prompts, [0] * self.S)

    def decode(self, tokens, i):
        """Decode step i (0-based) feeding `tokens` [S] at positions prompt_len + i."""
        return self.step([tokens[s:s + 1] for s in range(self.S)], [self.prompt_lens[s] + i for s in range(self.S)])
