"""Stage hand-off over gloo with world_size 2 and 3 on CPU
(reference: tests/test_pp_messager.py:68-157 does the same over NCCL on GPUs)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ctx(T, S, W, H, first):
    from vexact_b200.pp_messager import GenerationContext

    g = torch.Generator().manual_seed(T * 131 + S)
    return GenerationContext(
        batch_input_ids=torch.randint(0, 1000, (1, T), generator=g) if first else None,
        intermediate_tensors=None if first else torch.randn(1, T, H, generator=g).to(torch.bfloat16),
        query_start_loc=torch.arange(S + 1, dtype=torch.int32) * (T // S),
        batch_position_ids=torch.randint(0, 4096, (1, T), generator=g),
        block_tables=torch.randint(-1, 50, (S, W), generator=g, dtype=torch.int32),
        context_lens=torch.randint(1, 4096, (S,), generator=g, dtype=torch.int32),
        slot_mapping=torch.randint(-1, 800, (T,), generator=g, dtype=torch.int32),
        max_seqlen_q=T // S,
        tokens_generated=torch.arange(S, dtype=torch.int32),
    )


def _same(a, b):
    for name in ("batch_input_ids", "intermediate_tensors", "query_start_loc", "batch_position_ids", "block_tables",
                 "context_lens", "slot_mapping", "tokens_generated"):
        x, y = getattr(a, name), getattr(b, name)
        assert (x is None) == (y is None), name
        if x is not None:
            assert torch.equal(x.reshape(-1), y.reshape(-1)), name
    assert a.max_seqlen_q == b.max_seqlen_q


def _worker(rank, world, port, fail_q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        from vexact_b200.pp_messager import InferencerOutput, PPMessager

        H = 64
        m = PPMessager(rank, world, torch.device("cpu"), hidden_size=H, max_tokens=64, max_seqs=8,
                       max_blocks_per_seq=5, vocab_size=32, backend="gloo")
        for step, (T, S, W) in enumerate([(8, 4, 5), (64, 8, 3), (2, 1, 1)]):
            # ring: rank r sends to r + 1; rank 0 sends token ids, the others hidden states
            if rank == 0:
                m.send_gen_ctx(_ctx(T, S, W, H, first=True))
            else:
                got = m.recv_gen_ctx()
                _same(got, _ctx(T, S, W, H, first=(rank == 1)))
                if rank < world - 1:
                    m.send_gen_ctx(_ctx(T, S, W, H, first=False))
            # last -> first
            out = InferencerOutput(token_ids=torch.arange(S) * 3 + step,
                                   logits=torch.full((S, 32), 0.5, dtype=torch.bfloat16) if step == 1 else torch.empty(0),
                                   logprobs=-torch.arange(S, dtype=torch.float32))
            if rank == world - 1:
                m.send_infer_out(out)
            if rank == 0:
                got = m.recv_infer_out()
                assert torch.equal(got.token_ids, out.token_ids) and torch.equal(got.logprobs, out.logprobs)
                assert got.logits.numel() == out.logits.numel()
                if out.logits.numel():
                    assert torch.equal(got.logits, out.logits)
        if rank == 0:
            with pytest.raises(ValueError):
                m.send_gen_ctx(_ctx(128, 8, 5, H, first=True))  # beyond max_tokens
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    except Exception as e:  # surface the failure to the parent
        import traceback

        fail_q.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


@pytest.mark.parametrize("world", [2, 3])
def test_ring_handoff_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    errs = []
    while not q.empty():
        errs.append(q.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            errs.append("a rank did not finish in time")
    assert not errs, "\n".join(errs)
    assert all(p.exitcode == 0 for p in procs)


def test_layer_split_matches_oracle():
    from oracle import ops
    from vexact_b200.inferencer import get_pp_indices

    for L in (27, 28, 48):
        for pp in (1, 2, 4, 8):
            assert [get_pp_indices(L, r, pp) for r in range(pp)] == [ops.get_pp_indices(L, r, pp) for r in range(pp)]


def test_block_manager_matches_reference_fixture():
    from types import SimpleNamespace as NS

    from conftest import load_golden
    from vexact_b200.kv_cache_context import KVCacheManager

    want = load_golden("kv_manager")
    mgr = KVCacheManager(NS(max_cache_blocks=8, page_size=16))
    a1 = mgr.allocate_blocks(40)
    a2 = mgr.allocate_blocks(30)
    mgr.free_blocks(a1[:2])
    a3 = mgr.allocate_blocks(70, num_current_blocks=2)
    a4 = mgr.allocate_blocks(16 * 9)
    assert (a1, a2, a3, a4) == (want["a1"], want["a2"], want["a3"], want["a4"])
    assert mgr.num_free_blocks() == want["free"] and mgr.num_allocated_blocks() == want["allocated"]
