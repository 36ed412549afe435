"""Generates tests/golden/step_inputs.pt from the reference's own host step path.

    python tests/golden/make_step_inputs_golden.py /path/to/vexact

`Inferencer._prepare_gen_ctx` (vexact/inferencer/inferencer.py:193-291) and
`Inferencer._prepare_input_buffers_from_gen_ctx` (:293-349) are called unbound on a stand-in
object that carries only what the two methods touch (page size, device, CPU stand-ins for the
static input buffers); requests are plain objects with the attributes the methods read.  Every
case stores the per-request inputs next to the padded buffers the reference produced.
"""
from __future__ import annotations

import os
import random
import sys
from types import SimpleNamespace

os.environ.setdefault("VEXACT_DISABLE_MODEL_PATCH", "1")
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("VEXACT_SRC", "")
if not os.path.isdir(REF):
    raise SystemExit("usage: pass the path of a vexact checkout (or set VEXACT_SRC)")
sys.path.insert(0, REF)

import torch  # noqa: E402

from vexact.inferencer.inferencer import Inferencer  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


class CpuBuffers:
    """CPU stand-in for vexact.core.runtime_data.InputBuffers (:68): same fields, same fills."""

    def __init__(self, max_num_seqs, max_num_batched_tokens, max_blocks_per_req, hidden_size=8):
        def buf(*size, dtype, fill=None):
            t = torch.empty(size, dtype=dtype) if fill is None else torch.full(size, fill, dtype=dtype)
            return SimpleNamespace(gpu=t)

        self.max_num_seqs, self.max_num_batched_tokens = max_num_seqs, max_num_batched_tokens
        self.max_blocks_per_req = max_blocks_per_req
        self.slot_mapping = buf(max_num_batched_tokens, dtype=torch.int32, fill=0)
        self.context_lens = buf(max_num_seqs, dtype=torch.int32, fill=0)
        self.query_start_loc = buf(max_num_seqs + 1, dtype=torch.int32, fill=0)
        self.block_tables = buf(max_num_seqs, max_blocks_per_req, dtype=torch.int32, fill=-1)
        self.input_ids = buf(1, max_num_batched_tokens, dtype=torch.long, fill=0)
        self.intermediate_tensors = buf(1, max_num_batched_tokens, hidden_size, dtype=torch.bfloat16, fill=0)
        self.position_ids = buf(1, max_num_batched_tokens, dtype=torch.long, fill=0)

    def get_kv_context_tensors(self, num_seqs, num_tokens):
        return (self.block_tables.gpu[:num_seqs, :], self.context_lens.gpu[:num_seqs],
                self.slot_mapping.gpu[:num_tokens], self.query_start_loc.gpu[: num_seqs + 1])


def make_requests(rng, num_seqs, page_size, max_blocks, mode, vocab=50000):
    """Requests in the states a scheduler step can hold: prefill chunks, decode, a mix."""
    reqs, next_block = [], 0
    all_blocks = list(range(num_seqs * max_blocks))
    rng.shuffle(all_blocks)
    for i in range(num_seqs):
        prompt_len = rng.randint(1, page_size * (max_blocks - 1) - 1)
        input_ids = [rng.randrange(vocab) for _ in range(prompt_len)]
        kind = mode if mode != "mixed" else rng.choice(["prefill", "decode", "chunk"])
        if kind == "prefill":            # whole prompt in this step
            tokens_this_step, num_computed, generated = prompt_len, prompt_len, []
        elif kind == "chunk":            # a middle chunk of the prompt
            start = rng.randint(0, prompt_len - 1)
            tokens_this_step = rng.randint(1, prompt_len - start)
            num_computed, generated = start + tokens_this_step, []
        else:                            # decode: one token at position num_computed - 1
            n_gen = rng.randint(1, page_size)
            generated = [rng.randrange(vocab) for _ in range(n_gen)]
            tokens_this_step, num_computed = 1, prompt_len + n_gen
        n_blocks = (num_computed + page_size - 1) // page_size
        block_ids = all_blocks[next_block: next_block + n_blocks]
        next_block += n_blocks
        reqs.append(SimpleNamespace(input_ids_list=input_ids, tokens_this_step=tokens_this_step,
                                    num_computed_tokens=num_computed, block_ids=block_ids,
                                    generated_tokens=generated, generation_config=None))
    return reqs


def run_case(seed, num_seqs, page_size, max_blocks, mode, pad_seqs, pad_tokens):
    rng = random.Random(seed)
    reqs = make_requests(rng, num_seqs, page_size, max_blocks, mode)
    total = sum(r.tokens_this_step for r in reqs)
    graph_num_seqs, capture_tokens = num_seqs + pad_seqs, total + pad_tokens
    buffers = CpuBuffers(graph_num_seqs + 3, capture_tokens + 5, max_blocks)
    me = SimpleNamespace(input_buffers=buffers, page_size=page_size, device=torch.device("cpu"),
                         cache_store=SimpleNamespace(key_cache={}, value_cache={}))
    gen_ctx = Inferencer._prepare_gen_ctx(me, reqs)
    desc = SimpleNamespace(num_tokens=capture_tokens, num_seqs=graph_num_seqs)
    Inferencer._prepare_input_buffers_from_gen_ctx(me, gen_ctx, desc)
    bt, cl, sm, qsl = buffers.get_kv_context_tensors(graph_num_seqs, capture_tokens)
    return dict(
        # what a step is made of, per request
        page_size=page_size, max_blocks=max_blocks, graph_num_seqs=graph_num_seqs, capture_tokens=capture_tokens,
        num_computed_tokens=torch.tensor([r.num_computed_tokens for r in reqs], dtype=torch.int32),
        tokens_this_step=torch.tensor([r.tokens_this_step for r in reqs], dtype=torch.int32),
        block_ids=[list(r.block_ids) for r in reqs],
        input_ids_list=[list(r.input_ids_list) for r in reqs],
        last_generated=[(r.generated_tokens[-1] if r.generated_tokens else -1) for r in reqs],
        # what the reference built
        max_seqlen_q=int(gen_ctx.max_seqlen_q),
        block_tables=bt.clone(), context_lens=cl.clone(), slot_mapping=sm.clone(), query_start_loc=qsl.clone(),
        input_ids=buffers.input_ids.gpu[0, :capture_tokens].clone(),
        position_ids=buffers.position_ids.gpu[0, :capture_tokens].clone(),
    )


def main():
    cases = [
        run_case(1, 1, 16, 8, "decode", 0, 0),
        run_case(2, 7, 16, 12, "decode", 1, 1),
        run_case(3, 5, 16, 12, "prefill", 0, 0),
        run_case(4, 9, 8, 20, "chunk", 3, 17),
        run_case(5, 33, 16, 10, "mixed", 15, 64),
        run_case(6, 64, 4, 40, "mixed", 0, 200),
        run_case(7, 200, 16, 9, "decode", 56, 56),
    ]
    torch.save(cases, os.path.join(OUT, "step_inputs.pt"))
    for c in cases:
        print("seqs", len(c["block_ids"]), "tokens", int(c["tokens_this_step"].sum()), "max_q", c["max_seqlen_q"])


if __name__ == "__main__":
    main()
