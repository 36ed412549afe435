"""CPU restatement of the reference's host step path (TEST INFRASTRUCTURE ONLY: nothing in the
product imports this file).

Follows vexact/inferencer/inferencer.py: `_prepare_gen_ctx` (:193-291: slot mapping :208-222,
context lens :224-227, block tables :229-234, query_start_loc :236-240, input / position ids
:259-274) and `_prepare_input_buffers_from_gen_ctx` (:293-349: fills :306-312, copies :314-333,
padded request rows :318-324).  Pinned against tests/golden/step_inputs.pt, which the reference's
own two methods produced.
"""
from __future__ import annotations

import numpy as np


def prepare_step(num_computed_tokens, tokens_this_step, block_ids, input_ids_list, last_generated,
                 page_size: int, max_blocks: int, graph_num_seqs: int, capture_tokens: int):
    """Per-request state -> the padded buffers a captured step reads.

    block_ids[i]: the request's block list; input_ids_list[i]: its prompt; last_generated[i]: its
    last generated token (used when the step starts at or beyond the prompt's end, i.e. decode).
    Returns a dict of numpy arrays sized (capture_tokens,), (graph_num_seqs,), ... like the views
    `InputBuffers.get_kv_context_tensors(graph_num_seqs, capture_tokens)` gives.
    """
    num_seqs = len(num_computed_tokens)
    total = int(sum(int(t) for t in tokens_this_step))
    if total > capture_tokens:
        raise ValueError(f"total_tokens exceeds capture_tokens: {total} > {capture_tokens}")
    if graph_num_seqs < num_seqs:
        raise ValueError(f"graph_num_seqs cannot be smaller than num_seqs: {graph_num_seqs} < {num_seqs}")

    slot_mapping = np.full((capture_tokens,), -1, dtype=np.int32)
    input_ids = np.zeros((capture_tokens,), dtype=np.int64)
    position_ids = np.zeros((capture_tokens,), dtype=np.int64)
    context_lens = np.zeros((graph_num_seqs,), dtype=np.int32)
    query_start_loc = np.zeros((graph_num_seqs + 1,), dtype=np.int32)
    block_tables = np.full((graph_num_seqs, max_blocks), -1, dtype=np.int32)

    t = 0
    for i in range(num_seqs):
        n, computed = int(tokens_this_step[i]), int(num_computed_tokens[i])
        start = computed - n
        assert start >= 0
        for pos in range(start, start + n):
            slot_mapping[t] = block_ids[i][pos // page_size] * page_size + pos % page_size
            position_ids[t] = pos
            if start < len(input_ids_list[i]):      # prefill chunk: prompt tokens of this chunk
                input_ids[t] = input_ids_list[i][pos]
            else:                                   # decode: the last generated token
                input_ids[t] = last_generated[i]
            t += 1
        context_lens[i] = computed
        query_start_loc[i + 1] = query_start_loc[i] + n
        for j, b in enumerate(block_ids[i]):
            block_tables[i, j] = b
    # padded request rows are zero-length, point at the real token count and hold block 0
    block_tables[num_seqs:graph_num_seqs, :] = 0
    query_start_loc[num_seqs + 1: graph_num_seqs + 1] = total
    max_seqlen_q = max((int(x) for x in tokens_this_step), default=0)
    return dict(slot_mapping=slot_mapping, input_ids=input_ids, position_ids=position_ids,
                context_lens=context_lens, query_start_loc=query_start_loc, block_tables=block_tables,
                total_tokens=total, max_seqlen_q=max_seqlen_q)
