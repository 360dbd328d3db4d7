"""The step's batch as the kernels see it: flat token arrays plus per-request rows,
packed into one int32 buffer that goes to the device in one copy.

A batch is a list of request segments.  A segment of one token at the end of a
request is a decode token, a longer one is a portion of a prompt; the kernels do
not distinguish them: every token carries its position and the index of its
request, every request its block-table row.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them
    (0-based, within ``tokens``) whose logits are wanted."""
    rid: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepBatch:
    T: int
    R: int
    token_ids: torch.Tensor       # [T] int32
    positions: torch.Tensor       # [T] int32
    req_of_token: torch.Tensor    # [T] int32, index into the per-request rows
    cu_q: torch.Tensor            # [R+1] int32, token offsets of the segments
    q_start: torch.Tensor         # [R] int32, position of each segment's first token
    kv_len: torch.Tensor          # [R] int32, request length after this step
    state_slot: torch.Tensor      # [R] int32
    logit_rows: torch.Tensor      # [n_want] int32, token indices
    block_tables: Dict[int, torch.Tensor]  # group -> [R, max_blocks] int32
    # host mirrors
    h_q_start: List[int] = field(default_factory=list)
    h_q_len: List[int] = field(default_factory=list)
    h_kv_len: List[int] = field(default_factory=list)
    h_slots: List[int] = field(default_factory=list)
    rids: List[object] = field(default_factory=list)
    static_bound: Optional[int] = None  # set for graph replay: kernels size grids for this many keys
    # Data that kernels derive once per step and share between layers.  `extras`: made on the
    # device from this step's values (recomputed inside a captured graph at every replay);
    # `static_extras`: made on the host from the batch's shape alone (kept across replays).
    extras: Dict[object, object] = field(default_factory=dict)
    static_extras: Dict[object, object] = field(default_factory=dict)

    @property
    def max_q_len(self) -> int:
        return max(self.h_q_len) if self.h_q_len else 0

    @property
    def max_kv_len(self) -> int:
        return max(self.h_kv_len) if self.h_kv_len else 0


class BatchBuilder:
    """Uploads a step that the host runtime packed into pinned host memory (one copy) and
    hands out the views of it.

    A small ring of pinned buffers, each guarded by an event, lets the host prepare
    the next step while the previous copy may still be in flight."""

    def __init__(self, device: torch.device, ring: int = 4):
        self.device = device
        self._ring = ring
        self._bufs: List[Optional[torch.Tensor]] = [None] * ring
        self._events: List[Optional[torch.cuda.Event]] = [None] * ring
        self._next = 0

    def _pinned(self, n: int) -> torch.Tensor:
        i = self._next
        self._next = (i + 1) % self._ring
        if self._events[i] is not None:
            self._events[i].synchronize()
        buf = self._bufs[i]
        if buf is None or buf.numel() < n:
            cap = max(1024, 1 << (n - 1).bit_length())
            buf = torch.empty(cap, dtype=torch.int32, pin_memory=self.device.type == "cuda")
            self._bufs[i] = buf
        self._slot = i
        return buf

    def pinned(self, n: int) -> torch.Tensor:
        """A pinned int32 buffer of at least ``n`` words from the ring (the one :meth:`finish` sends)."""
        return self._pinned(n)

    @property
    def last_ring_slot(self) -> int:
        """The ring slot of the buffer that :meth:`pinned` handed out last."""
        return self._slot

    def mark_sent(self, ring_slot: int) -> None:
        """A copy from the buffer in ``ring_slot`` was queued on the current stream by someone else: the
        slot is busy until that copy is done."""
        if self.device.type == "cuda":
            ev = self._events[ring_slot] or torch.cuda.Event()
            ev.record()
            self._events[ring_slot] = ev

    def send(self, host: torch.Tensor, total: int, into: Optional[torch.Tensor] = None,
             ring_slot: Optional[int] = None) -> torch.Tensor:
        """Copies the first ``total`` words of the pinned buffer to the device (into ``into``, a buffer of
        exactly that size at a fixed address, or a new tensor) and marks the ring slot busy until then
        (``ring_slot``: the buffer's slot if it is not the one handed out last)."""
        if into is not None:
            if into.numel() != total:
                raise ValueError(f"static batch buffer holds {into.numel()} words, this batch needs {total}")
            dev = into
        else:
            dev = torch.empty(total, dtype=torch.int32, device=self.device)
        dev.copy_(host[:total], non_blocking=True)
        if self.device.type == "cuda":
            i = self._slot if ring_slot is None else ring_slot
            ev = self._events[i] or torch.cuda.Event()
            ev.record()
            self._events[i] = ev
        return dev

    def finish(self, host: torch.Tensor, T: int, R: int, n_want: int, widths: Dict[int, int], rids: List[object],
               into: Optional[torch.Tensor] = None) -> StepBatch:
        """Sends a packed step (the layout of :meth:`build`: token ids, positions, request of token,
        cu_q, q_start, kv_len, slot, logit rows, one block table per group) to the device in one
        copy and returns the views of it."""
        total = 3 * T + (R + 1) + 3 * R + n_want + sum(R * w for w in widths.values())
        dev = self.send(host, total, into)
        h = host[:total].numpy()
        off = 0

        def take(n):
            nonlocal off
            a = (off, off + n)
            off += n
            return a

        a_tok, a_pos, a_req = take(T), take(T), take(T)
        a_cu, a_qs, a_kv, a_sl = take(R + 1), take(R), take(R), take(R)
        a_lr = take(n_want)
        a_bt = {g: take(R * w) for g, w in widths.items()}
        cu = h[a_cu[0]:a_cu[1]]

        def d(a):
            return dev[a[0]:a[1]]

        return StepBatch(
            T=T, R=R, token_ids=d(a_tok), positions=d(a_pos), req_of_token=d(a_req), cu_q=d(a_cu),
            q_start=d(a_qs), kv_len=d(a_kv), state_slot=d(a_sl), logit_rows=d(a_lr),
            block_tables={g: d(a_bt[g]).view(R, widths[g]) for g in widths},
            h_q_start=h[a_qs[0]:a_qs[1]].tolist(), h_q_len=(cu[1:] - cu[:-1]).tolist(),
            h_kv_len=h[a_kv[0]:a_kv[1]].tolist(), h_slots=h[a_sl[0]:a_sl[1]].tolist(), rids=list(rids))
