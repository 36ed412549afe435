"""Stage-boundary transport for the pipeline-parallel layout.

Mirror of vexact/distributed/pp_messager.py:36-200 (`PPMessager.send_gen_ctx`,
`recv_gen_ctx`, `send_infer_out`, `recv_infer_out`) over the same ring
(rank r -> r + 1, last -> first), with a different wire format:

* the reference pickles shapes/dtypes and Python objects over a gloo pair group and then
  posts one NCCL isend per tensor into freshly allocated tensors;
* here every message is a fixed-layout int32 header (16 words) followed by ONE packed byte
  payload, both sent with torch.distributed P2P on the default group (NCCL over NVLink on
  GPUs; gloo on CPU for tests), into persistent buffers sized once from the configured
  maxima.  No pickling, no per-step allocation, no collective.

Python-object fields of the reference's GenerationContext (the per-request GenerationConfig
list) belong to the sampler, which is outside this library; `tokens_generated` travels as an
int32 tensor.
"""
from __future__ import annotations

from dataclasses import dataclass
from datetime import timedelta
from typing import Optional

import torch
import torch.distributed as dist

HEADER_WORDS = 16
MAGIC_CTX = 0x56584358   # "VXCX"
MAGIC_OUT = 0x56584F54   # "VXOT"


@dataclass
class GenerationContext:
    """Per-step carrier between stages (vexact/core/runtime_data.py:120-131)."""

    batch_input_ids: Optional[torch.Tensor]      # [1, T] int64 (first stage only)
    intermediate_tensors: Optional[torch.Tensor]  # [1, T, H] bf16 (from the previous stage)
    query_start_loc: torch.Tensor                # [S + 1] int32
    batch_position_ids: torch.Tensor             # [1, T] int64
    block_tables: torch.Tensor                   # [S, W] int32
    context_lens: torch.Tensor                   # [S] int32
    slot_mapping: torch.Tensor                   # [T] int32
    max_seqlen_q: int
    tokens_generated: Optional[torch.Tensor] = None  # [S] int32


@dataclass
class InferencerOutput:
    """Last stage -> first stage (vexact/core/runtime_data.py:134-137)."""

    token_ids: torch.Tensor   # [S] int64
    logits: torch.Tensor      # [S, V] or empty
    logprobs: torch.Tensor    # [S] fp32 or empty


def _align16(n: int) -> int:
    return (n + 15) // 16 * 16


class PPMessager:
    def __init__(self, pp_rank: int, pp_size: int, device: torch.device, hidden_size: int, max_tokens: int,
                 max_seqs: int, max_blocks_per_seq: int, vocab_size: int = 0, world_ranks: Optional[list] = None,
                 init_method: Optional[str] = None, backend: Optional[str] = None,
                 timeout: timedelta = timedelta(minutes=30)):
        self._device = torch.device(device)
        self.pp_rank, self.pp_size = pp_rank, pp_size
        if not dist.is_initialized():
            backend = backend or ("nccl" if self._device.type == "cuda" else "gloo")
            dist.init_process_group(backend=backend, rank=pp_rank, world_size=pp_size, init_method=init_method,
                                    timeout=timeout)
        ranks = world_ranks if world_ranks is not None else list(range(pp_size))
        self._next_rank = ranks[(pp_rank + 1) % pp_size]
        self._prev_rank = ranks[(pp_rank - 1) % pp_size]
        self.hidden_size, self.max_tokens = hidden_size, max_tokens
        self.max_seqs, self.max_blocks = max_seqs, max_blocks_per_seq
        self.vocab_size = vocab_size
        cap = (_align16(max_tokens * hidden_size * 2) + _align16(max_tokens * 8) + _align16(max_tokens * 4)
               + _align16((max_seqs + 1) * 4) + 2 * _align16(max_seqs * 4)
               + _align16(max_seqs * max_blocks_per_seq * 4))
        cap_out = _align16(max_seqs * 8) + _align16(max_seqs * 4) + _align16(max_seqs * vocab_size * 2)
        self._cap = max(cap, cap_out)
        # persistent staging buffers: one pair per direction
        self._send_hdr = torch.zeros(HEADER_WORDS, dtype=torch.int32, device=self._device)
        self._recv_hdr = torch.zeros(HEADER_WORDS, dtype=torch.int32, device=self._device)
        self._send_buf = torch.empty(self._cap, dtype=torch.uint8, device=self._device)
        self._recv_buf = torch.empty(self._cap, dtype=torch.uint8, device=self._device)

    # ---------------------------------------------------------------- packing helpers
    @staticmethod
    def _sections(T: int, S: int, W: int, H: int, has_hidden: bool):
        """(name, dtype, shape, byte offset) of every section of a gen-ctx payload, and its size."""
        secs, off = [], 0

        def add(name, dtype, shape):
            nonlocal off
            n = 1
            for d in shape:
                n *= d
            secs.append((name, dtype, shape, off))
            off += _align16(n * torch.empty((), dtype=dtype).element_size())

        if has_hidden:
            add("intermediate_tensors", torch.bfloat16, (1, T, H))
        else:
            add("batch_input_ids", torch.int64, (1, T))
        add("batch_position_ids", torch.int64, (1, T))
        add("slot_mapping", torch.int32, (T,))
        add("query_start_loc", torch.int32, (S + 1,))
        add("context_lens", torch.int32, (S,))
        add("tokens_generated", torch.int32, (S,))
        add("block_tables", torch.int32, (S, W))
        return secs, off

    def _view(self, buf, dtype, shape, off):
        n = 1
        for d in shape:
            n *= d
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return buf[off:off + nbytes].view(dtype).view(shape)

    def _p2p(self, ops):
        for req in dist.batch_isend_irecv(ops):
            req.wait()

    # ---------------------------------------------------------------- gen ctx: rank r -> r + 1
    def send_gen_ctx(self, ctx: GenerationContext) -> None:
        has_hidden = ctx.intermediate_tensors is not None
        T = ctx.batch_position_ids.shape[-1]
        S = ctx.context_lens.shape[0]
        W = ctx.block_tables.shape[1] if ctx.block_tables.ndim == 2 else 0
        if T > self.max_tokens or S > self.max_seqs or W > self.max_blocks:
            raise ValueError(f"gen ctx (T={T}, S={S}, W={W}) exceeds the configured maxima "
                             f"({self.max_tokens}, {self.max_seqs}, {self.max_blocks})")
        secs, total = self._sections(T, S, W, self.hidden_size, has_hidden)
        for name, dtype, shape, off in secs:
            src = getattr(ctx, name)
            if src is None:  # tokens_generated is optional
                self._view(self._send_buf, dtype, shape, off).zero_()
            else:
                self._view(self._send_buf, dtype, shape, off).copy_(src.reshape(shape).to(dtype))
        hdr = torch.tensor([MAGIC_CTX, T, S, W, int(ctx.max_seqlen_q), int(has_hidden), total] + [0] * 9,
                           dtype=torch.int32)
        self._send_hdr.copy_(hdr)
        self._p2p([dist.P2POp(dist.isend, self._send_hdr, self._next_rank)])
        self._p2p([dist.P2POp(dist.isend, self._send_buf[:total], self._next_rank)])

    def recv_gen_ctx(self) -> GenerationContext:
        self._p2p([dist.P2POp(dist.irecv, self._recv_hdr, self._prev_rank)])
        hdr = self._recv_hdr.tolist()
        if hdr[0] != MAGIC_CTX:
            raise RuntimeError(f"unexpected message header {hdr[0]:#x} from rank {self._prev_rank}")
        T, S, W, max_q, has_hidden, total = hdr[1:7]
        self._p2p([dist.P2POp(dist.irecv, self._recv_buf[:total], self._prev_rank)])
        secs, _ = self._sections(T, S, W, self.hidden_size, bool(has_hidden))
        vals = {name: self._view(self._recv_buf, dtype, shape, off) for name, dtype, shape, off in secs}
        return GenerationContext(
            batch_input_ids=vals.get("batch_input_ids"),
            intermediate_tensors=vals.get("intermediate_tensors"),
            query_start_loc=vals["query_start_loc"],
            batch_position_ids=vals["batch_position_ids"],
            block_tables=vals["block_tables"],
            context_lens=vals["context_lens"],
            slot_mapping=vals["slot_mapping"],
            max_seqlen_q=max_q,
            tokens_generated=vals["tokens_generated"],
        )

    # ---------------------------------------------------------------- infer out: last -> first
    def send_infer_out(self, out: InferencerOutput) -> None:
        S = out.token_ids.shape[0]
        V = out.logits.shape[-1] if out.logits.numel() else 0
        has_lp = int(out.logprobs.numel() > 0)
        o_tok, o_lp = 0, _align16(S * 8)
        o_logits = o_lp + _align16(S * 4)
        total = o_logits + _align16(S * V * 2)
        if total > self._cap:
            raise ValueError("infer output exceeds the configured maxima")
        self._view(self._send_buf, torch.int64, (S,), o_tok).copy_(out.token_ids)
        if has_lp:
            self._view(self._send_buf, torch.float32, (S,), o_lp).copy_(out.logprobs)
        if V:
            self._view(self._send_buf, torch.bfloat16, (S, V), o_logits).copy_(out.logits)
        self._send_hdr.copy_(torch.tensor([MAGIC_OUT, S, V, has_lp, total] + [0] * 11, dtype=torch.int32))
        self._p2p([dist.P2POp(dist.isend, self._send_hdr, self._next_rank)])
        self._p2p([dist.P2POp(dist.isend, self._send_buf[:total], self._next_rank)])

    def recv_infer_out(self) -> InferencerOutput:
        self._p2p([dist.P2POp(dist.irecv, self._recv_hdr, self._prev_rank)])
        hdr = self._recv_hdr.tolist()
        if hdr[0] != MAGIC_OUT:
            raise RuntimeError(f"unexpected message header {hdr[0]:#x} from rank {self._prev_rank}")
        S, V, has_lp, total = hdr[1:5]
        self._p2p([dist.P2POp(dist.irecv, self._recv_buf[:total], self._prev_rank)])
        o_lp = _align16(S * 8)
        o_logits = o_lp + _align16(S * 4)
        empty = torch.empty(0, device=self._device)
        return InferencerOutput(
            token_ids=self._view(self._recv_buf, torch.int64, (S,), 0),
            logits=self._view(self._recv_buf, torch.bfloat16, (S, V), o_logits) if V else empty,
            logprobs=self._view(self._recv_buf, torch.float32, (S,), o_lp) if has_lp else empty,
        )

    # ---------------------------------------------------------------- raw activation hand-off
    def send_hidden(self, hidden: torch.Tensor) -> None:
        """Fixed-shape activation hand-off for a steady-state pipeline (shape known to both sides)."""
        self._p2p([dist.P2POp(dist.isend, hidden, self._next_rank)])

    def recv_hidden(self, out: torch.Tensor) -> torch.Tensor:
        self._p2p([dist.P2POp(dist.irecv, out, self._prev_rank)])
        return out
