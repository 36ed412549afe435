"""Device-built step inputs: the reference's host step path without per-token Python.

Stands in for `Inferencer._prepare_gen_ctx` (vexact/inferencer/inferencer.py:193-291) and
`Inferencer._prepare_input_buffers_from_gen_ctx` (:293-349) over the static buffers of
`InputBuffers` (vexact/core/runtime_data.py:68-113).  The host hands over three int32 counters per
request (context length after the step, tokens this step, where the request's prompt chunk starts
in the packed prompt-token array, or -1 for decode); one kernel (`b200_prepare_step`) writes
slot_mapping, position ids, input ids (prompt chunk, or the previous step's token straight from
device memory), context_lens, query_start_loc and the padded block tables of the captured shape.
Block tables live on the device and are updated by deltas (a request gains a block once per
page), so a decode step uploads a few KB instead of the whole [S, max_blocks] table.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _lib
from .inferencer import StepInputs


class StepBuffers:
    """Static step-input buffers (mirror of `InputBuffers`) plus per-request state on the device."""

    def __init__(self, device, max_num_seqs: int, max_num_batched_tokens: int, max_blocks_per_req: int,
                 page_size: int, buffers=None):
        """`buffers` (an `InputBuffers`, optional): write the step into its device tensors instead of
        allocating a second set, so that graphs captured over those buffers read what this kernel writes."""
        if max_num_seqs > 8192:
            raise ValueError("at most 8192 requests per step")
        self.device = torch.device(device)
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_blocks_per_req = max_blocks_per_req
        self.page_size = page_size
        dev, S, T, B = self.device, max_num_seqs, max_num_batched_tokens, max_blocks_per_req
        # what a captured step reads (same shapes and fills as InputBuffers)
        if buffers is not None:
            if (buffers.max_num_seqs, buffers.max_num_batched_tokens, buffers.max_blocks_per_req) != (S, T, B):
                raise ValueError("the InputBuffers were sized for other maxima")
            self.slot_mapping, self.context_lens = buffers.slot_mapping.gpu, buffers.context_lens.gpu
            self.query_start_loc, self.block_tables = buffers.query_start_loc.gpu, buffers.block_tables.gpu
            self.input_ids, self.position_ids = buffers.input_ids.gpu, buffers.position_ids.gpu
        else:
            self.slot_mapping = torch.full((T,), -1, dtype=torch.int32, device=dev)
            self.context_lens = torch.zeros(S, dtype=torch.int32, device=dev)
            self.query_start_loc = torch.zeros(S + 1, dtype=torch.int32, device=dev)
            self.block_tables = torch.full((S, B), -1, dtype=torch.int32, device=dev)
            self.input_ids = torch.zeros(1, T, dtype=torch.long, device=dev)
            self.position_ids = torch.zeros(1, T, dtype=torch.long, device=dev)
        self.step_info = torch.zeros(2, dtype=torch.int32, device=dev)
        self.seq_order = torch.arange(S, dtype=torch.int32, device=dev)   # requests by descending context
        self._order_host = torch.empty(S, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        # per-request state kept on the device between steps
        self.request_blocks = torch.full((S, B), -1, dtype=torch.int32, device=dev)
        self.last_tokens = torch.zeros(S, dtype=torch.long, device=dev)
        # pinned staging: [num_computed | tokens_this_step | prefill_offset] and packed prompt tokens
        pin = self.device.type == "cuda"
        self._counters_host = torch.empty(3, S, dtype=torch.int32, pin_memory=pin)
        self._counters_dev = torch.empty(3, S, dtype=torch.int32, device=dev)
        self._prefill_host = torch.empty(T, dtype=torch.long, pin_memory=pin)
        self._prefill_dev = torch.empty(T, dtype=torch.long, device=dev)
        self._delta_host = torch.empty(3, S * 2, dtype=torch.int64, pin_memory=pin)
        self.h2d_bytes_last_step = 0

    # ------------------------------------------------------------------ block-table deltas
    def set_request_blocks(self, row: int, block_ids: Sequence[int]) -> None:
        """(Re)write one request's whole block list, e.g. when the request enters the batch."""
        if len(block_ids) > self.max_blocks_per_req:
            raise ValueError("request has more blocks than max_blocks_per_req")
        line = torch.full((self.max_blocks_per_req,), -1, dtype=torch.int32)
        line[: len(block_ids)] = torch.as_tensor(list(block_ids), dtype=torch.int32)
        self.request_blocks[row].copy_(line, non_blocking=True)

    def append_blocks(self, rows: Sequence[int], cols: Sequence[int], block_ids: Sequence[int]) -> int:
        """request_blocks[rows[k], cols[k]] = block_ids[k]; returns the bytes uploaded."""
        n = len(rows)
        if n == 0:
            return 0
        if n > self._delta_host.shape[1]:
            raise ValueError("too many block-table updates in one step")
        d = self._delta_host[:, :n]
        d[0] = torch.as_tensor(list(rows), dtype=torch.int64)
        d[1] = torch.as_tensor(list(cols), dtype=torch.int64)
        d[2] = torch.as_tensor(list(block_ids), dtype=torch.int64)
        dd = d.to(self.device, non_blocking=True)
        self.request_blocks.index_put_((dd[0], dd[1]), dd[2].to(torch.int32))
        return int(d.numel() * d.element_size())

    # ------------------------------------------------------------------ one step
    def prepare(self, num_computed_tokens: Sequence[int], tokens_this_step: Sequence[int],
                prefill_chunks: Optional[dict] = None, graph_num_seqs: Optional[int] = None,
                capture_tokens: Optional[int] = None) -> StepInputs:
        """Build the step's buffers.  prefill_chunks: {request row: prompt tokens fed this step};
        rows not in it are decode requests and read `last_tokens[row]` on the device."""
        num_seqs = len(num_computed_tokens)
        total = int(sum(tokens_this_step))
        graph_num_seqs = num_seqs if graph_num_seqs is None else graph_num_seqs
        capture_tokens = total if capture_tokens is None else capture_tokens
        if total > capture_tokens:
            raise ValueError(f"total_tokens exceeds capture_tokens: {total} > {capture_tokens}")
        if graph_num_seqs < num_seqs:
            raise ValueError(f"graph_num_seqs cannot be smaller than num_seqs: {graph_num_seqs} < {num_seqs}")
        if graph_num_seqs > self.max_num_seqs or capture_tokens > self.max_num_batched_tokens:
            raise ValueError("step exceeds the static buffers")
        c = self._counters_host
        c[0, :num_seqs] = torch.as_tensor(list(num_computed_tokens), dtype=torch.int32)
        c[1, :num_seqs] = torch.as_tensor(list(tokens_this_step), dtype=torch.int32)
        c[2, :num_seqs] = -1
        n_prefill = 0
        if prefill_chunks:
            for row, toks in sorted(prefill_chunks.items()):
                if len(toks) != int(tokens_this_step[row]):
                    raise ValueError(f"request {row}: prompt chunk length != tokens_this_step")
                c[2, row] = n_prefill
                self._prefill_host[n_prefill: n_prefill + len(toks)] = torch.as_tensor(list(toks), dtype=torch.long)
                n_prefill += len(toks)
        self._counters_dev[:, :num_seqs].copy_(c[:, :num_seqs], non_blocking=True)
        if n_prefill:
            self._prefill_dev[:n_prefill].copy_(self._prefill_host[:n_prefill], non_blocking=True)
        # longest context first: the attention kernel deals its tiles in this order (padded rows last)
        order = torch.argsort(torch.as_tensor(list(num_computed_tokens), dtype=torch.int32), descending=True,
                              stable=True)
        self._order_host[:num_seqs] = order.to(torch.int32)
        if graph_num_seqs > num_seqs:
            self._order_host[num_seqs:graph_num_seqs] = torch.arange(num_seqs, graph_num_seqs, dtype=torch.int32)
        self.seq_order[:graph_num_seqs].copy_(self._order_host[:graph_num_seqs], non_blocking=True)
        self.h2d_bytes_last_step = 3 * num_seqs * 4 + graph_num_seqs * 4 + n_prefill * 8
        self.launch(num_seqs, graph_num_seqs, capture_tokens, n_prefill > 0)
        max_q = max((int(t) for t in tokens_this_step), default=0)
        return StepInputs(
            input_ids=self.input_ids[0, :capture_tokens], hidden_in=None,
            positions=self.position_ids[0, :capture_tokens], slot_mapping=self.slot_mapping[:capture_tokens],
            query_start_loc=self.query_start_loc[: graph_num_seqs + 1], context_lens=self.context_lens[:graph_num_seqs],
            block_tables=self.block_tables[:graph_num_seqs], max_seqlen_q=max_q,
            seq_order=self.seq_order[:graph_num_seqs])

    def launch(self, num_seqs: int, graph_num_seqs: int, capture_tokens: int, has_prefill: bool) -> None:
        """The kernel alone, on counters already in `_counters_dev` (what a replayed step calls)."""
        if self.device.type != "cuda":
            raise _lib.B200Error("step inputs are built by a CUDA kernel: no CPU path")
        lib = _lib.load()
        cd = self._counters_dev
        rc = lib.b200_prepare_step(
            cd[0].data_ptr(), cd[1].data_ptr(), self.request_blocks.data_ptr(),
            self._prefill_dev.data_ptr() if has_prefill else None, cd[2].data_ptr() if has_prefill else None,
            self.last_tokens.data_ptr(), num_seqs, graph_num_seqs, capture_tokens, self.max_blocks_per_req,
            self.page_size, self.input_ids.data_ptr(), self.position_ids.data_ptr(), self.slot_mapping.data_ptr(),
            self.context_lens.data_ptr(), self.query_start_loc.data_ptr(), self.block_tables.data_ptr(),
            self.step_info.data_ptr(), _lib.current_stream())
        _lib.check(rc, "b200_prepare_step")



class TokenFeedback:
    """The device half of `Scheduler.update` (vexact/core/scheduler.py:211-235).

    The reference moves a step's tokens to the host with `.cpu()` and then reads them one `.item()` at a
    time while the GPU idles.  Here a step's tokens (and log-probabilities) are (1) written into the step
    buffers' `last_tokens`, so that the next decode step reads its input ids from device memory, and
    (2) copied asynchronously into one of `depth` pinned host buffers; the scheduler collects a step's
    results with ONE event wait, typically a step late, while the next step is already running.
    """

    def __init__(self, step_buffers: StepBuffers, depth: int = 2):
        self.sb = step_buffers
        S = step_buffers.max_num_seqs
        pin = step_buffers.device.type == "cuda"
        self._tok = [torch.empty(S, dtype=torch.long, pin_memory=pin) for _ in range(depth)]
        self._lp = [torch.empty(S, dtype=torch.float32, pin_memory=pin) for _ in range(depth)]
        self._ev = [torch.cuda.Event() if pin else None for _ in range(depth)]
        self._n = [0] * depth
        self._has_lp = [False] * depth
        self._turn = 0

    def push(self, tokens: torch.Tensor, logprobs: Optional[torch.Tensor] = None) -> int:
        """Queue a step's results (row i = request i of the step); returns the ticket to `pop` them with."""
        n = tokens.shape[0]
        if n > self.sb.max_num_seqs:
            raise ValueError("more tokens than requests the step buffers hold")
        i = self._turn
        self._turn = (i + 1) % len(self._tok)
        self.sb.last_tokens[:n].copy_(tokens)                     # next decode step's input ids, on the device
        self._tok[i][:n].copy_(tokens, non_blocking=True)
        self._has_lp[i] = logprobs is not None and logprobs.numel() > 0
        if self._has_lp[i]:
            self._lp[i][:n].copy_(logprobs, non_blocking=True)
        self._n[i] = n
        if self._ev[i] is not None:
            self._ev[i].record()
        return i

    def pop(self, ticket: int):
        """(token ids, log-probabilities or None) of a queued step as Python lists: one wait for the batch."""
        if self._ev[ticket] is not None:
            self._ev[ticket].synchronize()
        n = self._n[ticket]
        lps = self._lp[ticket][:n].tolist() if self._has_lp[ticket] else None
        return self._tok[ticket][:n].tolist(), lps
