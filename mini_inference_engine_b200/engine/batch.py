"""Turns a step's rows -- (request, its next tokens, wanted places) -- into the device-side
``StepContext``: all integers of the step are packed into one pinned host buffer and copied with
one asynchronous transfer (the reference builds 3-6 device tensors per step plus three per
continued prompt portion, inference_engine/engine.py:159-178, among them an O(n x context) mask
that does not exist here: the attention kernel masks from positions).

Rows keep the order they are given in.  Each row is one request: ``tokens`` are its next tokens,
which start at position ``pos0`` (= positions already in its cache), ``tables[g]`` is its block
table in cache group g, ``want`` lists places among ``tokens`` whose logits are asked for.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import StepContext


@dataclass
class BatchRow:
    tokens: list
    pos0: int
    tables: list                      # per cache group: list[int] of physical pages
    state_slot: int = 0
    want: list = field(default_factory=list)


_TORCH_DTYPES = {"<i4": torch.int32, "<f4": torch.float32, "<i8": torch.int64, "<u4": torch.int32}


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class BatchBuilder:
    def __init__(self, num_groups: int, page_size: int, device, max_position: int | None = None):
        self.num_groups = num_groups
        self.page_size = page_size
        self.device = torch.device(device)
        self.max_position = max_position
        self._host: list = []              # ring of pinned buffers with the event of their last copy
        self._turn = 0

    # ------------------------------------------------------------------ packing
    def pack(self, rows: list[BatchRow], pad_rows: int | None = None, table_width: int | None = None,
             extras: dict | None = None):
        """Returns (numpy int32 buffer, layout dict).  ``pad_rows`` pads with scratch rows (one
        token at position 0 in page 0, state slot 0) up to that many rows, and ``table_width`` fixes
        the block-table width -- both for steps replayed from a captured graph, whose shapes are
        static.  ``extras`` are small per-step arrays of 4- or 8-byte elements (sampling inputs)
        that ride in the same transfer; they come back as ``ctx.extras[name]`` on the device."""
        R_real = len(rows)
        R = max(R_real, pad_rows or 0)
        lens = [len(r.tokens) for r in rows]
        if R_real and min(lens) == 0:
            raise ValueError("a batch row needs at least one token")
        q_len = np.ones(R, dtype=np.int32)
        pos0 = np.zeros(R, dtype=np.int32)
        q_len[:R_real] = lens
        pos0[:R_real] = [r.pos0 for r in rows]
        q_start = np.zeros(R + 1, dtype=np.int32)
        np.cumsum(q_len, out=q_start[1:])
        T = int(q_start[-1])
        ctx_len = pos0 + q_len
        if self.max_position is not None and R_real and int(ctx_len[:R_real].max()) > self.max_position:
            raise ValueError(f"a request would reach position {int(ctx_len.max())}, beyond the model's "
                             f"max_position_embeddings {self.max_position}")
        width = table_width or max(1, max((len(t) for r in rows for t in r.tables), default=1))
        W = sum(len(r.want) for r in rows) + (R - R_real)      # every scratch row "wants" its one token

        off = {}
        n = 0
        for name, size in (("token_ids", T), ("positions", T), ("token_row", T), ("row_q_start", R),
                           ("row_q_len", R), ("row_ctx_len", R), ("state_slots", R), ("want", W)):
            off[name] = (n, size)
            n = _align(n + size)
        for g in range(self.num_groups):
            off[f"slots{g}"] = (n, T)
            n = _align(n + T)
        for g in range(self.num_groups):
            off[f"tables{g}"] = (n, R * width)
            n = _align(n + R * width)
        extra_off = {}
        for name, arr in (extras or {}).items():
            arr = np.ascontiguousarray(arr)
            if arr.dtype.itemsize not in (4, 8):
                raise ValueError(f"extra {name!r}: elements must be 4 or 8 bytes")
            words = arr.size * arr.dtype.itemsize // 4
            extra_off[name] = (n, words, arr.dtype.str, arr)
            n = _align(n + words)
        buf = np.zeros(n, dtype=np.int32)
        for name, (o, words, _, arr) in extra_off.items():
            buf[o:o + words] = arr.reshape(-1).view(np.int32)

        def seg(name):
            o, s = off[name]
            return buf[o:o + s]

        seg("row_q_start")[:] = q_start[:R]
        seg("row_q_len")[:] = q_len
        seg("row_ctx_len")[:] = ctx_len
        seg("state_slots")[:R_real] = [r.state_slot for r in rows]
        tok, pos, trow = seg("token_ids"), seg("positions"), seg("token_row")
        # Per row only what has to be: its tokens, its block tables, its wanted places.  Positions and
        # cache slots of all tokens come from the rows' numbers in one go (a decode step has one token
        # a row, and many rows).
        if R_real and max(lens) == 1:
            trow[:] = np.arange(R, dtype=np.int32)
            pos[:] = pos0
            tok[:R_real] = [r.tokens[0] for r in rows]
        else:
            trow[:] = np.repeat(np.arange(R, dtype=np.int32), q_len)
            pos[:] = pos0[trow] + (np.arange(T, dtype=np.int32) - q_start[:R][trow])
            for r, a, m in zip(rows, q_start.tolist(), lens):
                tok[a:a + m] = r.tokens
        ps = self.page_size
        last_page = (ctx_len[:R_real] - 1) // ps
        for g in range(self.num_groups):
            tg = seg(f"tables{g}").reshape(R, width)
            held = np.zeros(R_real, dtype=np.int32)
            for i, r in enumerate(rows):
                t = r.tables[g]
                m = len(t)
                if m > width:
                    raise ValueError(f"block table of {m} pages exceeds the width {width}")
                tg[i, :m] = t
                held[i] = m
            if R_real and bool((last_page >= held).any()):
                raise ValueError("a batch row has no page for its last new token")
            seg(f"slots{g}")[:] = tg[trow, pos // ps] * ps + pos % ps
        wanted = []
        for r, a, m in zip(rows, q_start.tolist(), lens):
            for j in r.want:
                if not 0 <= j < m:
                    raise ValueError(f"wanted place {j} is outside the row's {m} tokens")
                wanted.append(a + j)
        wanted.extend(q_start[R_real:R].tolist())            # scratch rows
        seg("want")[:] = wanted
        layout = dict(off=off, T=T, R=R, W=W, width=width, size=n, real_rows=R_real,
                      extras={k: v[:3] for k, v in extra_off.items()},
                      max_q_len=int(q_len.max()) if R else 0, max_ctx_len=int(ctx_len.max()) if R else 0,
                      q_len=q_len.tolist(), ctx_len=ctx_len.tolist(), q_start=q_start[:R].tolist(),
                      state_slots=[r.state_slot for r in rows] + [0] * (R - R_real))
        return buf, layout

    # ------------------------------------------------------------------ to the device
    def _pinned(self, n: int):
        """A pinned buffer of at least n ints whose previous transfer has finished."""
        if len(self._host) < 3:
            self._host.append([torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=True), None])
        self._turn = (self._turn + 1) % len(self._host)
        slot = self._host[self._turn]
        if slot[1] is not None:
            slot[1].synchronize()
        if slot[0].numel() < n:
            slot[0] = torch.empty(max(n, 2 * slot[0].numel()), dtype=torch.int32, pin_memory=True)
        return slot

    def to_device(self, buf: np.ndarray, layout: dict, into: torch.Tensor | None = None) -> StepContext:
        n = layout["size"]
        if self.device.type == "cuda":
            slot = self._pinned(n)
            slot[0][:n].numpy()[:] = buf
            dev = into if into is not None else torch.empty(n, dtype=torch.int32, device=self.device)
            dev[:n].copy_(slot[0][:n], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            slot[1] = ev
        else:                                    # host-only use (tests of the packing)
            dev = torch.from_numpy(buf.copy())
        return self.view(dev, layout)

    def view(self, dev: torch.Tensor, layout: dict) -> StepContext:
        off, T, R, width = layout["off"], layout["T"], layout["R"], layout["width"]

        def seg(name):
            o, s = off[name]
            return dev[o:o + s]

        return StepContext(
            num_tokens=T, num_rows=R, token_ids=seg("token_ids"), positions=seg("positions"),
            token_row=seg("token_row"), row_q_start=seg("row_q_start"), row_q_len=seg("row_q_len"),
            row_ctx_len=seg("row_ctx_len"), state_slots=seg("state_slots"),
            block_tables=[seg(f"tables{g}").view(R, width) for g in range(self.num_groups)],
            slots=[seg(f"slots{g}") for g in range(self.num_groups)], want=seg("want"),
            max_q_len=layout["max_q_len"], max_ctx_len=layout["max_ctx_len"],
            extras={k: dev[o:o + w].view(_TORCH_DTYPES[d]) for k, (o, w, d) in layout.get("extras", {}).items()},
            host=dict(q_len=layout["q_len"], ctx_len=layout["ctx_len"], q_start=layout["q_start"],
                      state_slots=layout["state_slots"], real_rows=layout["real_rows"],
                      few_single_rows=layout.get("few_single_rows", False)))

    def build(self, rows: list[BatchRow]) -> StepContext:
        buf, layout = self.pack(rows)
        return self.to_device(buf, layout)
