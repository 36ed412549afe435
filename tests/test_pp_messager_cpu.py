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


def _ctx(T, S, W, H, first, with_requests=True):
    from types import SimpleNamespace as NS

    from vexact_b200.pp_messager import GenerationContext

    g = torch.Generator().manual_seed(T * 131 + S)
    cfgs = [NS(do_sample=bool(i % 2), temperature=0.5 + i, top_k=None if i % 3 == 0 else 40 + i, top_p=0.9,
               output_scores=True, output_logits=False, seed=None if i % 2 else 1234 + i) for i in range(S)]
    return GenerationContext(
        batch_input_ids=torch.randint(0, 1000, (1, T), generator=g) if first else None,
        intermediate_tensors=None if first else torch.randn(1, T, H, generator=g).to(torch.bfloat16),
        query_start_loc=torch.arange(S + 1, dtype=torch.int32) * (T // S),
        batch_position_ids=torch.randint(0, 4096, (1, T), generator=g),
        block_tables=torch.randint(-1, 50, (S, W), generator=g, dtype=torch.int32),
        context_lens=torch.randint(1, 4096, (S,), generator=g, dtype=torch.int32),
        slot_mapping=torch.randint(-1, 800, (T,), generator=g, dtype=torch.int32),
        max_seqlen_q=T // S,
        generation_configs=cfgs if with_requests else [],
        tokens_generated=list(range(3, 3 + S)) if with_requests else None,
    )


def _same(a, b):
    for name in ("batch_input_ids", "intermediate_tensors", "query_start_loc", "batch_position_ids", "block_tables",
                 "context_lens", "slot_mapping"):
        x, y = getattr(a, name), getattr(b, name)
        assert (x is None) == (y is None), name
        if x is not None:
            assert torch.equal(x.reshape(-1).cpu(), y.reshape(-1).cpu()), name
    assert a.max_seqlen_q == b.max_seqlen_q
    assert a.tokens_generated == b.tokens_generated          # a list of ints, or None: the optional field survives
    assert len(a.generation_configs) == len(b.generation_configs)
    for x, y in zip(a.generation_configs, b.generation_configs):
        for f in ("do_sample", "temperature", "top_k", "top_p", "output_scores", "output_logits", "seed"):
            assert getattr(x, f) == getattr(y, f), f


def _worker(rank, world, port, fail_q, use_cuda=False, shared_cpu=None):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        from vexact_b200.config import ParallelConfig, PPInfo
        from vexact_b200.pp_messager import InferencerOutput, PPMessager

        H = 64
        device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
        if use_cuda:          # payloads over NCCL P2P; NVLS off: a test rank may exit while peers still hold buffers
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            torch.cuda.set_device(device)
        # the reference's constructor: (pp_info, parallel_config, device)
        m = PPMessager(PPInfo(world, rank), ParallelConfig(world, "127.0.0.1", str(port)), device,
                       shared_cpu_group=shared_cpu)
        # ring topology under the reference's attribute names (tests/test_pp_messager.py:128-143); the world's own
        # ranks here, since this process group holds one replica
        assert m._next_msger_rank == (rank + 1) % world and m._prev_msger_rank == (rank - 1) % world
        for pair in (m._next_msger_cpu_pair, m._next_msger_gpu_pair, m._prev_msger_cpu_pair, m._prev_msger_gpu_pair):
            assert pair is not None
        for step, (T, S, W) in enumerate([(8, 4, 5), (64, 8, 3), (2, 1, 1)]):
            req = step != 2          # the last step carries neither sampling configs nor tokens_generated
            # ring: rank r sends to r + 1; rank 0 sends token ids, the others hidden states
            if rank == 0:
                m.send_gen_ctx(_ctx(T, S, W, H, first=True, with_requests=req))
            else:
                got = m.recv_gen_ctx()
                _same(got, _ctx(T, S, W, H, first=(rank == 1), with_requests=req))
                if rank < world - 1:
                    m.send_gen_ctx(_ctx(T, S, W, H, first=False, with_requests=req))
            # last -> first
            out = InferencerOutput(token_ids=torch.arange(S) * 3 + step,
                                   logits=torch.full((S, 32), 0.5, dtype=torch.bfloat16) if step == 1 else torch.empty(0),
                                   logprobs=-torch.arange(S, dtype=torch.float32))
            if rank == world - 1:
                m.send_infer_out(out)
            if rank == 0:
                got = m.recv_infer_out()
                assert got.token_ids.device.type == device.type
                assert torch.equal(got.token_ids.cpu(), out.token_ids) and torch.equal(got.logprobs.cpu(), out.logprobs)
                assert got.logits.numel() == out.logits.numel()
                if out.logits.numel():
                    assert torch.equal(got.logits.cpu(), out.logits)

        # two contexts in flight: the first one received must survive the second receive (two slots)
        if rank == 0:
            m.send_gen_ctx(_ctx(8, 4, 5, H, first=True))
            m.send_gen_ctx(_ctx(16, 4, 5, H, first=True))
        elif rank == 1:
            first, second = m.recv_gen_ctx(), m.recv_gen_ctx()
            _same(first, _ctx(8, 4, 5, H, first=True))
            _same(second, _ctx(16, 4, 5, H, first=True))

        # block tables as deltas: a full table opens slot 7, then two steps ship only the changed entries
        S, W = 4, 6
        base = _ctx(8, S, W, H, first=True)
        if rank == 0:
            m.send_gen_ctx(base, slot=7)
            full_bytes = m.bytes_sent_last
            rows, cols, vals = torch.tensor([1, 3]), torch.tensor([2, 5]), torch.tensor([41, 42])
            m.send_gen_ctx(base, slot=7, block_delta=(rows, cols, vals))
            assert m.bytes_sent_last < full_bytes
            m.send_gen_ctx(base, slot=7, block_delta=(rows[:0], cols[:0], vals[:0]))
        elif rank == 1:
            want = base.block_tables.clone()
            assert torch.equal(m.recv_gen_ctx().block_tables.cpu(), want)
            want[1, 2], want[3, 5] = 41, 42
            assert torch.equal(m.recv_gen_ctx().block_tables.cpu(), want)
            assert torch.equal(m.recv_gen_ctx().block_tables.cpu(), want)
        m.flush()
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    except Exception as e:  # surface the failure to the parent
        import traceback

        fail_q.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


def _run_ring(world, use_cuda, shared_cpu=None):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, use_cuda, shared_cpu)) for r in range(world)]
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


@pytest.mark.parametrize("world", [2, 3])
def test_ring_handoff_gloo(world):
    _run_ring(world, use_cuda=False)


def test_ring_handoff_with_one_header_group_for_all_ranks():
    """Headers over a single gloo group of every rank instead of one per pair: what the messager falls back
    to under a device-bound default group, where torch's subgroup creation would otherwise never finish with
    three or more ranks (ranks outside a gloo pair take part in a communicator split its members skip)."""
    _run_ring(3, use_cuda=False, shared_cpu=True)


@pytest.mark.gpu
def test_ring_handoff_nccl_two_gpus():
    """The same exchange with device tensors: headers on gloo, payloads on the pair's NCCL group
    (reference: tests/test_pp_messager.py:68-157).  Needs two GPUs; skipped on a one-GPU box."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run_ring(2, use_cuda=True)


@pytest.mark.gpu
def test_ring_handoff_nccl_four_gpus():
    """Four ranks: every pair group has ranks outside it (the case in which per-pair header groups cannot be
    made under the device-bound default group the messager initialises for NCCL)."""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    _run_ring(4, use_cuda=True)


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


def _pipeline_worker(rank, pp, port, fail_q):
    """The benchmark's choreography with stand-in stages: a set-up round in which every stage sends before
    it receives its feedback, then steady-state steps with `pp` batches in flight, feedback last -> first."""
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import torch.distributed as dist

        from vexact_b200.config import PPInfo
        from vexact_b200.pp_messager import GenerationContext, InferencerOutput, PPMessager

        dist.init_process_group("gloo", rank=rank, world_size=pp)      # the world exists before the messager
        S, H, W = 8, 16, 4
        msg = PPMessager(PPInfo(pp, rank), None, torch.device("cpu"), recv_slots=pp, send_slots=2)
        msg.reserve(H, S, S, W, 0)
        no_delta = tuple(torch.empty(0, dtype=torch.int32) for _ in range(3))
        mine = [GenerationContext(None, torch.full((1, S, H), float(b), dtype=torch.bfloat16),
                                  torch.arange(S + 1, dtype=torch.int32), torch.zeros(1, S, dtype=torch.long),
                                  torch.full((S, W), b, dtype=torch.int32), torch.ones(S, dtype=torch.int32),
                                  torch.zeros(S, dtype=torch.int32), 1) for b in range(pp)]
        first = [None] * pp

        def hand_on(b, ctx, opening):
            if rank < pp - 1:
                msg.send_gen_ctx(ctx, slot=b, block_delta=None if opening else no_delta)
            else:
                msg.send_infer_out(InferencerOutput(torch.full((S,), b), torch.empty(0), torch.zeros(S)))

        for b in range(pp):                       # set-up round
            if rank > 0:
                first[b] = msg.recv_gen_ctx()
                mine[b] = first[b]
            hand_on(b, mine[b], True)
        pending = [rank == 0] * pp
        for _ in range(6):                        # steady state
            for b in range(pp):
                if rank == 0:
                    if pending[b]:
                        assert int(msg.recv_infer_out().token_ids[0]) == b
                    pending[b] = True
                else:
                    got = msg.recv_gen_ctx()
                    # batch b of every round lands where its first message landed (graphs capture on these views)
                    assert got.intermediate_tensors.data_ptr() == first[b].intermediate_tensors.data_ptr()
                    assert got.block_tables.data_ptr() == first[b].block_tables.data_ptr()
                    assert float(got.intermediate_tensors[0, 0, 0]) == b and int(got.block_tables[0, 0]) == b
                hand_on(b, mine[b], False)
        for b in range(pp):
            if rank == 0 and pending[b]:
                msg.recv_infer_out()
        msg.flush()
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        import traceback

        fail_q.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


@pytest.mark.parametrize("world", [2, 4])
def test_pipeline_ring_where_every_stage_sends_before_it_receives(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pipeline_worker, args=(r, world, port, q)) for r in range(world)]
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
            errs.append("a rank did not finish in time (a send blocked on its receiver?)")
    assert not errs, "\n".join(errs)
    assert all(p.exitcode == 0 for p in procs)


def _replica_worker(rank, world, pp, port, fail_q):
    """torch.distributed belongs to somebody else (a trainer's world of `world` ranks); the messager finds its
    replica's ring inside it (pp_messager.py:62-87 of the reference)."""
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import torch.distributed as dist

        dist.init_process_group("gloo", rank=rank, world_size=world)
        from vexact_b200.config import PPInfo
        from vexact_b200.pp_messager import InferencerOutput, PPMessager

        replica, pp_rank = rank // pp, rank % pp
        m = PPMessager(PPInfo(pp, pp_rank), None, torch.device("cpu"))
        H, T, S, W = 32, 6, 3, 2
        mine = _ctx(T + replica, S, W, H, first=True)            # every replica sends its own content
        if pp_rank == 0:
            m.send_gen_ctx(mine)
            got = m.recv_infer_out()
            assert torch.equal(got.token_ids, torch.arange(S) + 100 * replica)
        else:
            got = m.recv_gen_ctx()
            _same(got, mine)                                     # not another replica's message
            m.send_infer_out(InferencerOutput(token_ids=torch.arange(S) + 100 * replica, logits=torch.empty(0),
                                              logprobs=torch.zeros(S)))
        m.flush()
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        import traceback

        fail_q.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


def test_two_replicas_inside_one_world():
    world, pp = 4, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_replica_worker, args=(r, world, pp, port, q)) for r in range(world)]
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
