"""Stage-boundary transport for the pipeline-parallel layout.

Mirror of vexact/distributed/pp_messager.py (`PPMessager.__init__` :36, `_create_pp_pair_groups` :89,
`send_gen_ctx` :116, `recv_gen_ctx` :131, `send_infer_out` :147, `recv_infer_out` :156): the same ring
(rank r -> r + 1, last -> first), the same constructor `(pp_info, parallel_config, device)`, the same
two group modes (this library owns the process group, or the world was initialised by the trainer and
holds several replicas), and one CPU group plus one device group per adjacent pair.

The wire format differs:
  * the reference pickles shapes, dtypes and Python objects over the CPU group, then posts one NCCL
    isend per tensor into freshly allocated tensors;
  * here a message is a fixed 32-word int64 header (+ one small per-request record when the step
    carries sampling parameters) on the CPU group and ONE packed byte payload on the device group,
    received into persistent staging buffers.  Nothing is pickled, nothing is allocated per step, and
    no device-to-host read is needed to learn the payload's size (the header arrives on the CPU side).
  * block tables may travel as deltas: the receiver keeps the table of every in-flight batch slot on
    its device and a step ships only the (row, column, block id) triples that changed.

Returned tensors are views into the receive staging buffers.  Each direction has `recv_slots` (default
2) buffers used in turn, so a received context or output stays valid until `recv_slots` further
messages of the same kind have been received; clone what must live longer.  With `recv_slots` equal to
the number of batches in flight and `reserve()` called up front, batch b of every round lands at the
same addresses, so a CUDA graph can be captured directly on the received views.
Sends are asynchronous: a payload is packed into one of `send_slots` staging buffers and the transfer
is waited for only when that buffer comes round again.
"""
from __future__ import annotations

import os
from datetime import timedelta
from types import SimpleNamespace
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .config import PPInfo
from .runtime_data import GenerationContext, InferencerOutput  # noqa: F401  (re-exported)

HEADER_WORDS = 32
MAGIC_CTX = 0x56584358   # "VXCX"
MAGIC_OUT = 0x56584F54   # "VXOT"
# per-request sampling record (float64): the GenerationConfig fields the last stage reads
_REQ_FIELDS = ("do_sample", "temperature", "top_k", "top_p", "output_scores", "output_logits", "seed",
               "tokens_generated")


def _align16(n: int) -> int:
    return (n + 15) // 16 * 16


def _esize(dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


class PPMessager:
    _world_cpu_group = None     # the all-ranks gloo group, made once per process when per-pair ones cannot be

    def __init__(self, pp_info, parallel_config=None, device=None, *, backend: Optional[str] = None,
                 recv_slots: int = 2, send_slots: int = 2, init_timeout: timedelta = timedelta(minutes=30),
                 group_timeout: timedelta = timedelta(days=7), shared_cpu_group: Optional[bool] = None):
        """`pp_info`: PPInfo(pp_size, pp_rank); `parallel_config`: address / port of the rendezvous when
        this call has to initialise torch.distributed; `device`: where payloads live.  `backend` defaults
        to NCCL for CUDA devices and gloo for CPU (tests)."""
        self._device = torch.device(device if device is not None else "cuda")
        self._pp = pp_info
        self.pp_rank, self.pp_size = pp_info.pp_rank, pp_info.pp_size
        self._dev_backend = backend or ("nccl" if self._device.type == "cuda" else "gloo")
        self._group_timeout = group_timeout
        self._shared_cpu = shared_cpu_group     # None: decided from the default group (see _create_pp_pair_groups)
        if not dist.is_initialized():
            if parallel_config is not None:
                os.environ.setdefault("MASTER_ADDR", str(parallel_config.torch_distributed_addr))
                os.environ.setdefault("MASTER_PORT", str(parallel_config.torch_distributed_port))
            kw = {"device_id": self._device} if self._dev_backend == "nccl" else {}
            dist.init_process_group(backend=self._dev_backend, rank=self.pp_rank, world_size=self.pp_size,
                                    timeout=init_timeout, **kw)
            self._create_pp_pair_groups(list(range(self.pp_size)))
        else:
            self._init_pp_groups_within_world()
        self._recv_slots = max(1, int(recv_slots))
        self._send_slots = max(1, int(send_slots))
        self._send_bufs = [torch.empty(0, dtype=torch.uint8, device=self._device) for _ in range(self._send_slots)]
        self._send_work = [None] * self._send_slots     # per staging buffer: the transfers that read it
        self._send_keep = [None] * self._send_slots
        self._send_turn = 0
        self._recv_bufs = {kind: [torch.empty(0, dtype=torch.uint8, device=self._device)
                                  for _ in range(self._recv_slots)] for kind in ("ctx", "out")}
        self._recv_turn = {"ctx": 0, "out": 0}
        self._slot_tables: dict[int, torch.Tensor] = {}   # batch slot -> [S, W] int32 block table kept here
        self.bytes_sent_last = 0

    # ---------------------------------------------------------------- groups
    def _init_pp_groups_within_world(self):
        """torch.distributed was initialised by someone else (the trainer): world ranks are laid out
        replica by replica, and new_group is collective, so every rank creates every replica's pairs."""
        world_rank, world_size = dist.get_rank(), dist.get_world_size()
        if world_size % self.pp_size:
            raise ValueError(f"world size {world_size} is not a multiple of the pipeline size {self.pp_size}")
        mine = world_rank // self.pp_size
        for replica in range(world_size // self.pp_size):
            base = replica * self.pp_size
            self._create_pp_pair_groups([base + i for i in range(self.pp_size)], store=replica == mine)

    def _create_pp_pair_groups(self, world_ranks: Sequence[int], store: bool = True):
        """One CPU (gloo) and one device group per adjacent pair of the ring, created in ring order by
        every rank (new_group is collective).  pp_size 1 has no pair."""
        if self.pp_size == 1:
            return
        # A default group that is bound to a device (init_process_group(..., device_id=...)) creates NCCL
        # subgroups by splitting its communicator, and torch makes the ranks that are NOT in a new subgroup
        # take part in that split whatever the subgroup's backend is, while the members of a gloo subgroup
        # do not: with three or more ranks a per-pair gloo group then never finishes.  In that case the
        # headers travel over one gloo group of all ranks (every rank a member, point-to-point by rank);
        # the payload groups stay per pair.
        bound = getattr(dist.distributed_c10d._get_default_group(), "bound_device_id", None) is not None
        shared_cpu = None
        if self._shared_cpu if self._shared_cpu is not None else (bound and self._dev_backend != "gloo"):
            if PPMessager._world_cpu_group is None:
                PPMessager._world_cpu_group = dist.new_group(backend="gloo", timeout=self._group_timeout)
            shared_cpu = PPMessager._world_cpu_group
        for r in range(self.pp_size):
            nxt = (r + 1) % self.pp_size
            pair = [world_ranks[r], world_ranks[nxt]]
            cpu = shared_cpu if shared_cpu is not None else dist.new_group(backend="gloo", ranks=pair,
                                                                           timeout=self._group_timeout)
            dev = cpu if self._dev_backend == "gloo" else dist.new_group(backend=self._dev_backend, ranks=pair,
                                                                         timeout=self._group_timeout)
            if store and self.pp_rank == r:
                self._next_rank, self._next_cpu, self._next_dev = pair[1], cpu, dev
            if store and self.pp_rank == nxt:
                self._prev_rank, self._prev_cpu, self._prev_dev = pair[0], cpu, dev

    # the reference's attribute names (pp_messager.py:97-114; tests/test_pp_messager.py:128-143 read them)
    _next_msger_rank = property(lambda self: self._next_rank)
    _prev_msger_rank = property(lambda self: self._prev_rank)
    _next_msger_cpu_pair = property(lambda self: self._next_cpu)
    _next_msger_gpu_pair = property(lambda self: self._next_dev)
    _prev_msger_cpu_pair = property(lambda self: self._prev_cpu)
    _prev_msger_gpu_pair = property(lambda self: self._prev_dev)

    # ---------------------------------------------------------------- staging
    def reserve(self, hidden_size: int, max_tokens: int, max_seqs: int, max_blocks_per_seq: int,
                vocab_size: int = 0) -> None:
        """Size the staging buffers once for the configured maxima (otherwise they grow on demand)."""
        ctx = self._ctx_layout(max_tokens, max_seqs, max_blocks_per_seq, hidden_size, True, 0, False)[1]
        out = _align16(max_seqs * 8) + _align16(max_seqs * 4) + _align16(max_seqs * vocab_size * 2)
        for i in range(self._send_slots):
            self._grow_send(max(ctx, out), i)
        for i in range(self._recv_slots):
            self._grow_recv("ctx", i, ctx)
            self._grow_recv("out", i, out)

    def _grow_send(self, n: int, i: int) -> torch.Tensor:
        if self._send_bufs[i].numel() < n:
            self._send_bufs[i] = torch.empty(max(n, 16), dtype=torch.uint8, device=self._device)
        return self._send_bufs[i]

    def _next_send(self, n: int) -> tuple[int, torch.Tensor]:
        """The staging buffer of this message; the transfer that last used it is waited for first."""
        i = self._send_turn
        self._send_turn = (i + 1) % self._send_slots
        self._wait_slot(i)
        return i, self._grow_send(n, i)

    def _wait_slot(self, i: int) -> None:
        for w in self._send_work[i] or ():
            w.wait()
        self._send_work[i] = None

    def flush(self) -> None:
        """Wait for every payload still in flight (call before tearing the process group down)."""
        for i in range(self._send_slots):
            self._wait_slot(i)

    def _grow_recv(self, kind: str, i: int, n: int) -> torch.Tensor:
        bufs = self._recv_bufs[kind]
        if bufs[i].numel() < n:
            bufs[i] = torch.empty(max(n, 16), dtype=torch.uint8, device=self._device)
        return bufs[i]

    def _next_recv(self, kind: str, n: int) -> torch.Tensor:
        i = self._recv_turn[kind]
        self._recv_turn[kind] = (i + 1) % self._recv_slots
        return self._grow_recv(kind, i, n)

    @staticmethod
    def _ctx_layout(T: int, S: int, W: int, H: int, has_hidden: bool, n_delta: int, delta_mode: bool):
        """[(name, dtype, shape, byte offset)] of a gen-ctx payload and its total size."""
        secs, off = [], 0

        def add(name, dtype, shape):
            nonlocal off
            n = 1
            for d in shape:
                n *= d
            secs.append((name, dtype, shape, off))
            off += _align16(n * _esize(dtype))

        if has_hidden:
            add("intermediate_tensors", torch.bfloat16, (1, T, H))
        else:
            add("batch_input_ids", torch.int64, (1, T))
        add("batch_position_ids", torch.int64, (1, T))
        add("slot_mapping", torch.int32, (T,))
        add("query_start_loc", torch.int32, (S + 1,))
        add("context_lens", torch.int32, (S,))
        if delta_mode:
            add("block_delta", torch.int32, (3, n_delta))
        else:
            add("block_tables", torch.int32, (S, W))
        return secs, off

    @staticmethod
    def _view(buf, dtype, shape, off):
        n = 1
        for d in shape:
            n *= d
        return buf[off:off + n * _esize(dtype)].view(dtype).view(shape)

    @staticmethod
    def _wait(reqs):
        for r in reqs:
            r.wait()

    # ---------------------------------------------------------------- per-request sampling record
    @staticmethod
    def _pack_requests(S: int, generation_configs, tokens_generated) -> Optional[torch.Tensor]:
        if not generation_configs and tokens_generated is None:
            return None
        rec = torch.zeros((S, len(_REQ_FIELDS)), dtype=torch.float64)
        rec[:, 6] = float("nan")
        for i, cfg in enumerate(generation_configs or []):
            seed = getattr(cfg, "seed", None)
            top_k = getattr(cfg, "top_k", None)
            top_p = getattr(cfg, "top_p", None)
            rec[i, :7] = torch.tensor([
                float(bool(getattr(cfg, "do_sample", False))), float(getattr(cfg, "temperature", 1.0) or 0.0),
                float(top_k) if top_k is not None else float("nan"),
                float(top_p) if top_p is not None else float("nan"),
                float(bool(getattr(cfg, "output_scores", False))), float(bool(getattr(cfg, "output_logits", False))),
                float(seed) if seed is not None else float("nan")], dtype=torch.float64)
        if tokens_generated is not None:
            tg = tokens_generated.detach().cpu() if isinstance(tokens_generated, torch.Tensor) \
                else torch.as_tensor(list(tokens_generated))
            rec[:, 7] = tg.to(torch.float64)
        return rec

    @staticmethod
    def _unpack_requests(rec: torch.Tensor, has_cfg: bool, has_tg: bool):
        cfgs, tg = [], None
        if has_cfg:
            for row in rec.tolist():
                nan = lambda v: v != v  # noqa: E731
                cfgs.append(SimpleNamespace(
                    do_sample=bool(row[0]), temperature=row[1], top_k=None if nan(row[2]) else int(row[2]),
                    top_p=None if nan(row[3]) else row[3], output_scores=bool(row[4]), output_logits=bool(row[5]),
                    seed=None if nan(row[6]) else int(row[6])))
        if has_tg:
            tg = [int(v) for v in rec[:, 7].tolist()]
        return cfgs, tg

    # ---------------------------------------------------------------- gen ctx: rank r -> r + 1
    def send_gen_ctx(self, ctx: GenerationContext, slot: Optional[int] = None, block_delta=None) -> None:
        """Send a step's context to the next stage.

        slot / block_delta (optional): `slot` names the in-flight batch slot the context belongs to;
        with `block_delta = (rows, cols, block_ids)` (int tensors on this device, possibly empty) the
        block table is NOT shipped: the receiver applies the triples to the table it keeps for that
        slot.  The first message of a slot must carry the full table (block_delta=None)."""
        has_hidden = ctx.intermediate_tensors is not None
        T = ctx.batch_position_ids.shape[-1]
        S = ctx.context_lens.shape[0]
        W = ctx.block_tables.shape[1] if ctx.block_tables is not None and ctx.block_tables.ndim == 2 else 0
        H = ctx.intermediate_tensors.shape[-1] if has_hidden else 0
        delta_mode = block_delta is not None
        if delta_mode and slot is None:
            raise ValueError("block_delta needs the batch slot it applies to")
        n_delta = int(block_delta[0].numel()) if delta_mode else 0
        secs, total = self._ctx_layout(T, S, W, H, has_hidden, n_delta, delta_mode)
        turn, buf = self._next_send(total)
        for name, dtype, shape, off in secs:
            dst = self._view(buf, dtype, shape, off)
            if name == "block_delta":
                if n_delta:
                    dst.copy_(torch.stack([t.reshape(-1).to(torch.int32) for t in block_delta]))
            else:
                dst.copy_(getattr(ctx, name).reshape(shape))
        rec = self._pack_requests(S, ctx.generation_configs, ctx.tokens_generated)
        hdr = torch.zeros(HEADER_WORDS, dtype=torch.int64)
        hdr[:14] = torch.tensor([MAGIC_CTX, T, S, W, -1 if ctx.max_seqlen_q is None else int(ctx.max_seqlen_q),
                                 int(has_hidden), total, H, -1 if slot is None else int(slot), int(delta_mode), n_delta,
                                 int(rec is not None), int(bool(ctx.generation_configs)),
                                 int(ctx.tokens_generated is not None)], dtype=torch.int64)
        # nothing here blocks on the receiver: header, record and payload are all posted asynchronously
        # (a blocking header send deadlocks a ring in which every rank sends before it receives)
        work = [dist.isend(hdr, dst=self._next_rank, group=self._next_cpu)]
        if rec is not None:
            work.append(dist.isend(rec, dst=self._next_rank, group=self._next_cpu))
        work.append(dist.isend(buf[:total], dst=self._next_rank, group=self._next_dev))
        self._send_work[turn] = work
        self._send_keep[turn] = (hdr, rec)     # the CPU tensors must outlive their transfers
        self.bytes_sent_last = total + hdr.numel() * 8 + (rec.numel() * 8 if rec is not None else 0)

    def recv_gen_ctx(self) -> GenerationContext:
        hdr = torch.zeros(HEADER_WORDS, dtype=torch.int64)
        dist.recv(hdr, src=self._prev_rank, group=self._prev_cpu)
        h = hdr.tolist()
        if h[0] != MAGIC_CTX:
            raise RuntimeError(f"unexpected message header {h[0]:#x} from rank {self._prev_rank}")
        T, S, W, max_q, has_hidden, total, H, slot, delta_mode, n_delta, has_rec, has_cfg, has_tg = h[1:14]
        cfgs, tg = [], None
        if has_rec:
            rec = torch.zeros((S, len(_REQ_FIELDS)), dtype=torch.float64)
            dist.recv(rec, src=self._prev_rank, group=self._prev_cpu)
            cfgs, tg = self._unpack_requests(rec, bool(has_cfg), bool(has_tg))
        buf = self._next_recv("ctx", total)
        self._wait([dist.irecv(buf[:total], src=self._prev_rank, group=self._prev_dev)])
        secs, _ = self._ctx_layout(T, S, W, H, bool(has_hidden), n_delta, bool(delta_mode))
        vals = {name: self._view(buf, dtype, shape, off) for name, dtype, shape, off in secs}
        if delta_mode:
            table = self._slot_tables.get(slot)
            if table is None or table.shape != (S, W):
                raise RuntimeError(f"block-table delta for slot {slot} without a matching full table before it")
            if n_delta:
                d = vals["block_delta"].long()
                table.index_put_((d[0], d[1]), d[2].to(torch.int32))
            block_tables = table
        else:
            block_tables = vals["block_tables"]
            if slot >= 0:   # keep this slot's table for later deltas
                kept = self._slot_tables.get(slot)
                if kept is None or kept.shape != block_tables.shape:
                    kept = torch.empty_like(block_tables)
                    self._slot_tables[slot] = kept
                kept.copy_(block_tables)
                block_tables = kept
        return GenerationContext(
            batch_input_ids=vals.get("batch_input_ids"), intermediate_tensors=vals.get("intermediate_tensors"),
            query_start_loc=vals["query_start_loc"], batch_position_ids=vals["batch_position_ids"],
            block_tables=block_tables, context_lens=vals["context_lens"], slot_mapping=vals["slot_mapping"],
            max_seqlen_q=None if max_q < 0 else max_q, generation_configs=cfgs, tokens_generated=tg)

    # ---------------------------------------------------------------- infer out: last -> first
    def send_infer_out(self, out: InferencerOutput) -> None:
        S = out.token_ids.shape[0]
        V = out.logits.shape[-1] if out.logits.numel() else 0
        has_lp = int(out.logprobs.numel() > 0)
        esz = out.logits.element_size() if V else 2
        o_lp = _align16(S * 8)
        o_logits = o_lp + _align16(S * 4)
        total = o_logits + _align16(S * V * esz)
        turn, buf = self._next_send(total)
        self._view(buf, torch.int64, (S,), 0).copy_(out.token_ids)
        if has_lp:
            self._view(buf, torch.float32, (S,), o_lp).copy_(out.logprobs)
        if V:
            self._view(buf, out.logits.dtype, (S, V), o_logits).copy_(out.logits)
        hdr = torch.zeros(HEADER_WORDS, dtype=torch.int64)
        hdr[:6] = torch.tensor([MAGIC_OUT, S, V, has_lp, total, 1 if (V and out.logits.dtype == torch.float32) else 0])
        self._send_work[turn] = [dist.isend(hdr, dst=self._next_rank, group=self._next_cpu),
                                 dist.isend(buf[:total], dst=self._next_rank, group=self._next_dev)]
        self._send_keep[turn] = (hdr, None)
        self.bytes_sent_last = total + hdr.numel() * 8

    def recv_infer_out(self) -> InferencerOutput:
        hdr = torch.zeros(HEADER_WORDS, dtype=torch.int64)
        dist.recv(hdr, src=self._prev_rank, group=self._prev_cpu)
        h = hdr.tolist()
        if h[0] != MAGIC_OUT:
            raise RuntimeError(f"unexpected message header {h[0]:#x} from rank {self._prev_rank}")
        S, V, has_lp, total, f32 = h[1:6]
        buf = self._next_recv("out", total)
        self._wait([dist.irecv(buf[:total], src=self._prev_rank, group=self._prev_dev)])
        o_lp = _align16(S * 8)
        o_logits = o_lp + _align16(S * 4)
        empty = torch.empty(0, device=self._device)
        return InferencerOutput(
            token_ids=self._view(buf, torch.int64, (S,), 0),
            logits=self._view(buf, torch.float32 if f32 else torch.bfloat16, (S, V), o_logits) if V else empty,
            logprobs=self._view(buf, torch.float32, (S,), o_lp) if has_lp else empty)


def make_pp_info(pp_size: int, pp_rank: int) -> PPInfo:
    return PPInfo(pp_size=pp_size, pp_rank=pp_rank)
