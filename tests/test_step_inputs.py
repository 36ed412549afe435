"""Step-input construction: oracle vs the reference's own outputs (CPU), CUDA kernel vs both (GPU)."""
import os
import random

import numpy as np
import pytest
import torch

from oracle import step_inputs as oracle_step

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "step_inputs.pt")
FIELDS = ["slot_mapping", "input_ids", "position_ids", "context_lens", "query_start_loc", "block_tables"]


def _cases():
    return torch.load(GOLDEN, weights_only=False)


def _oracle(c):
    return oracle_step.prepare_step(c["num_computed_tokens"].tolist(), c["tokens_this_step"].tolist(), c["block_ids"],
                                    c["input_ids_list"], c["last_generated"], c["page_size"], c["max_blocks"],
                                    c["graph_num_seqs"], c["capture_tokens"])


def test_oracle_matches_reference_outputs():
    for c in _cases():
        got = _oracle(c)
        for f in FIELDS:
            assert np.array_equal(got[f], c[f].numpy()), f
        assert got["max_seqlen_q"] == c["max_seqlen_q"]


def test_oracle_rejects_what_the_reference_rejects():
    c = _cases()[2]
    with pytest.raises(ValueError):
        oracle_step.prepare_step(c["num_computed_tokens"].tolist(), c["tokens_this_step"].tolist(), c["block_ids"],
                                 c["input_ids_list"], c["last_generated"], c["page_size"], c["max_blocks"],
                                 c["graph_num_seqs"], int(c["tokens_this_step"].sum()) - 1)
    with pytest.raises(ValueError):
        oracle_step.prepare_step(c["num_computed_tokens"].tolist(), c["tokens_this_step"].tolist(), c["block_ids"],
                                 c["input_ids_list"], c["last_generated"], c["page_size"], c["max_blocks"],
                                 len(c["block_ids"]) - 1, c["capture_tokens"])


def _run_kernel(c, extra_seqs=3, extra_tokens=5):
    from vexact_b200.step_inputs import StepBuffers

    n = len(c["block_ids"])
    buf = StepBuffers("cuda", c["graph_num_seqs"] + extra_seqs, c["capture_tokens"] + extra_tokens, c["max_blocks"],
                      c["page_size"])
    chunks = {}
    for i in range(n):
        buf.set_request_blocks(i, c["block_ids"][i])
        tts, comp = int(c["tokens_this_step"][i]), int(c["num_computed_tokens"][i])
        if comp - tts < len(c["input_ids_list"][i]):
            chunks[i] = c["input_ids_list"][i][comp - tts: comp]
    buf.last_tokens[:n] = torch.tensor(c["last_generated"], dtype=torch.long)
    inp = buf.prepare(c["num_computed_tokens"].tolist(), c["tokens_this_step"].tolist(), chunks,
                      c["graph_num_seqs"], c["capture_tokens"])
    torch.cuda.synchronize()
    return buf, inp


@pytest.mark.gpu
def test_kernel_matches_reference_outputs():
    from vexact_b200 import _lib

    for c in _cases():
        buf, inp = _run_kernel(c)
        got = dict(slot_mapping=inp.slot_mapping, input_ids=inp.input_ids, position_ids=inp.positions,
                   context_lens=inp.context_lens, query_start_loc=inp.query_start_loc, block_tables=inp.block_tables)
        for f in FIELDS:
            assert torch.equal(got[f].cpu(), c[f]), f
        assert inp.max_seqlen_q == c["max_seqlen_q"]
        assert buf.step_info.tolist() == [int(c["tokens_this_step"].sum()), c["max_seqlen_q"]]
        assert _lib.read_status()[0] == 0


@pytest.mark.gpu
def test_kernel_matches_oracle_large_random_steps():
    """Steps at the benchmark's size and beyond, checked against the oracle."""
    rng = random.Random(7)
    for num_seqs, page, max_blocks, pad_s, pad_t in [(512, 16, 129, 0, 0), (1000, 16, 40, 24, 300), (8192, 8, 6, 0, 0)]:
        reqs_comp, reqs_tts, blocks, prompts, last = [], [], [], [], []
        ids = list(range(num_seqs * max_blocks))
        rng.shuffle(ids)
        nxt = 0
        for i in range(num_seqs):
            decode = rng.random() < 0.8
            plen = rng.randint(1, page * (max_blocks - 1) - 1)
            if decode:
                gen = rng.randint(1, page)
                comp, tts = plen + gen, 1
            else:
                start = rng.randint(0, plen - 1)
                tts = rng.randint(1, min(plen - start, 64))
                comp = start + tts
            nb = (comp + page - 1) // page
            reqs_comp.append(comp); reqs_tts.append(tts); blocks.append(ids[nxt: nxt + nb]); nxt += nb
            prompts.append([rng.randrange(150000) for _ in range(plen)]); last.append(rng.randrange(150000))
        total = sum(reqs_tts)
        c = dict(num_computed_tokens=torch.tensor(reqs_comp, dtype=torch.int32),
                 tokens_this_step=torch.tensor(reqs_tts, dtype=torch.int32), block_ids=blocks, input_ids_list=prompts,
                 last_generated=last, page_size=page, max_blocks=max_blocks, graph_num_seqs=num_seqs + pad_s,
                 capture_tokens=total + pad_t)
        want = _oracle(c)
        _, inp = _run_kernel(c, extra_seqs=0, extra_tokens=0)
        got = dict(slot_mapping=inp.slot_mapping, input_ids=inp.input_ids, position_ids=inp.positions,
                   context_lens=inp.context_lens, query_start_loc=inp.query_start_loc, block_tables=inp.block_tables)
        for f in FIELDS:
            assert np.array_equal(got[f].cpu().numpy(), want[f]), (num_seqs, f)


@pytest.mark.gpu
def test_block_table_deltas_and_device_resident_tokens():
    """A decode request crossing a page boundary: one delta upload, token taken from device memory."""
    from vexact_b200.step_inputs import StepBuffers

    page, max_blocks = 4, 8
    buf = StepBuffers("cuda", 4, 16, max_blocks, page)
    buf.set_request_blocks(0, [5, 2])        # 8 cached positions
    buf.set_request_blocks(1, [7])
    buf.last_tokens[:2] = torch.tensor([111, 222])
    # request 0 now computes position 8 -> needs a third block
    sent = buf.append_blocks([0], [2], [9])
    assert sent == 24
    inp = buf.prepare([9, 3], [1, 1], None, graph_num_seqs=3, capture_tokens=4)
    torch.cuda.synchronize()
    assert inp.slot_mapping.tolist() == [9 * page + 0, 7 * page + 2, -1, -1]
    assert inp.input_ids.tolist() == [111, 222, 0, 0]
    assert inp.positions.tolist() == [8, 2, 0, 0]
    assert inp.query_start_loc.tolist() == [0, 1, 2, 2]
    assert inp.context_lens.tolist() == [9, 3, 0]
    assert inp.block_tables.tolist() == [[5, 2, 9, -1, -1, -1, -1, -1], [7, -1, -1, -1, -1, -1, -1, -1], [0] * 8]
    assert buf.h2d_bytes_last_step == 24 + 3 * 4
    assert inp.seq_order.tolist() == [0, 1, 2]          # contexts 9, 3, then the padded row
    with pytest.raises(ValueError):
        buf.prepare([9, 3], [1, 1], None, graph_num_seqs=1, capture_tokens=4)
    with pytest.raises(ValueError):
        buf.prepare([9, 3], [1, 1], None, graph_num_seqs=2, capture_tokens=1)


@pytest.mark.gpu
def test_token_feedback_keeps_tokens_on_device_and_reads_them_with_one_wait():
    from vexact_b200.step_inputs import StepBuffers, TokenFeedback

    sb = StepBuffers("cuda", 8, 32, 4, 16)
    fb = TokenFeedback(sb, depth=2)
    t1 = torch.tensor([5, 6, 7], device="cuda")
    t2 = torch.tensor([8, 9, 10], device="cuda")
    k1 = fb.push(t1, torch.tensor([-0.5, -1.0, -1.5], device="cuda"))
    assert torch.equal(sb.last_tokens[:3], t1)
    k2 = fb.push(t2)                       # the next step is queued before the first one is read
    assert fb.pop(k1) == ([5, 6, 7], [-0.5, -1.0, -1.5])
    assert fb.pop(k2) == ([8, 9, 10], None)
    assert torch.equal(sb.last_tokens[:3], t2)
