"""The step function: one batch of (request, its next tokens) through the model.

A batch holds at most one entry per request: a contiguous run of that request's
next tokens, starting at its committed length; portions of prompts ride beside
single decoded tokens, cut anywhere (the reference's slices,
``sched/plan.py:124-162``; packed without padding, ``:316-319``).  The step runs
only these tokens, from the cache that earlier steps left, and returns float32
logits at the wanted places only, in the order of the entries and of ``want``.

Inside the packed batch the entries that bring a single token come first, whatever
order the caller gave them in (the reference packs decodes first too,
``sched/continuous.py:325-328``): a mixed step can then run its decode rows and its
prompt rows through different attention kernels, each on one contiguous range of
rows.  ``want_rows`` keeps the caller's order.

All step metadata is packed into one pinned int32 buffer and copied to the
device with one transfer; kernels read block tables and row maps from there
(the reference uploads one tensor per field, ``runner/buffers.py:369-462``, and
builds a CSR slot list per step, which these kernels do not need).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..parts.base import KVNeed


@dataclass
class StepEntry:
    slot: int                    # the request's slot in the cache manager
    start: int                   # position of the first token (= tokens cached so far)
    tokens: Sequence[int]        # its next tokens
    want: Sequence[int] = ()     # places among ``tokens`` whose logits are asked for


@dataclass
class StepContext:
    """What parts may read during a step.  Device tensors are int32."""
    num_rows: int
    num_requests: int
    num_wanted: int
    tokens: torch.Tensor         # [T]
    positions: torch.Tensor      # [T] absolute positions
    row_req: torch.Tensor        # [T] index of the row's request within this step
    want_rows: torch.Tensor      # [S] rows whose logits are wanted
    req_q_start: torch.Tensor    # [R + 1] first row of each request
    req_pos0: torch.Tensor       # [R] position of each request's first row
    req_slot: torch.Tensor       # [R] cache slot of each request
    req_kv_len: torch.Tensor     # [R] tokens cached after this step
    take_rows: torch.Tensor      # [R] for a step whose tokens come from another step's sampled rows: which row each takes
    tables: list                 # per cache group: [R, columns] block-table rows, or None
    cache: CacheManager
    dtype: torch.dtype
    host: dict = field(default_factory=dict)   # the same arrays as NumPy, for host-side decisions
    max_q_len: int = 1
    max_kv_len: int = 1
    # The first ``num_single`` requests of the step (= its first rows) bring one token each.
    num_single: int = 0
    # Cache rows that earlier steps wrote are complete when this step's kernels start: the upload
    # of the step's inputs (or a graph launch) lies between.  Kernels may read them ahead of the
    # kernels launched just before them.
    earlier_rows_settled: bool = False


class StepRunner:
    def __init__(self, model, cache: CacheManager, max_tokens: int = 2048, max_requests: int | None = None):
        self.model = model
        self.cache = cache
        self.device = model.device
        self.max_requests = max_requests or cache.max_requests
        self.kv_groups = [g for g, spec in enumerate(cache.groups) if isinstance(spec.need, KVNeed)]
        self._allocate(max_tokens)
        self._program = None              # the model's step as a native program; made at the first step
        self._lowered = False
        self.steps = 0
        self.rows_run = 0

    def _allocate(self, max_tokens: int) -> None:
        self.max_tokens = max_tokens
        total = self._layout(max_tokens, self.max_requests, max_tokens)[1]
        self.host_buf = torch.zeros(total, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        self.host_np = self.host_buf.numpy()
        self.dev_buf = torch.zeros(total, dtype=torch.int32, device=self.device)
        self._copied = None      # event after the last upload: the pinned buffer is free again
        self.h2d_bytes = 0       # bytes of the last step's upload
        self.generation = getattr(self, "generation", 0) + 1    # graphs captured on the old buffer are stale

    def _layout(self, T: int, R: int, S: int):
        """Offsets of the step's fields, packed back to back (16-byte aligned),
        so that one copy of ``total`` ints brings exactly what the step needs."""
        sizes = {"tokens": T, "positions": T, "row_req": T, "want_rows": S,
                 "req_q_start": R + 1, "req_pos0": R, "req_slot": R, "req_kv_len": R, "take_rows": R}
        for g in self.kv_groups:
            sizes[f"table{g}"] = R * self.cache.columns
        offsets, total = {}, 0
        for name, n in sizes.items():
            offsets[name] = (total, n)
            total += (n + 3) // 4 * 4
        return offsets, total

    def _field(self, buf, name: str, n: int):
        lo, cap = self.offsets[name]
        return buf[lo:lo + n]

    def prepare(self, entries: Sequence[StepEntry], pad_to: int | None = None,
                take_rows: Sequence[int] | None = None) -> StepContext:
        """Validates, packs and uploads a step.  ``pad_to``: for a pure-decode
        step, add padding lanes up to that many requests (position 0, the
        padding page, the spare state slot, token 0): they read nothing that
        lives and write nothing, and keep the step's shape fixed for a graph."""
        if not entries and not pad_to:
            raise ValueError("a step needs at least one entry")
        if self._copied is not None:
            self._copied.synchronize()
        n = len(entries)
        R = max(n, pad_to or 0)
        if R > max(self.max_requests, pad_to or 0):
            raise ValueError(f"{R} requests in one step, the engine was built for {self.max_requests}")
        # single-token entries first (stable): packed place -> index in ``entries``
        lengths = [len(e.tokens) for e in entries]
        if all(k == 1 for k in lengths):
            order = list(range(n))
        else:
            order = sorted(range(n), key=lambda i: lengths[i] != 1)
            entries = [entries[i] for i in order]
        counts = np.ones(R, dtype=np.int64)
        counts[:n] = [lengths[i] for i in order]
        if (counts < 1).any():
            raise ValueError("every entry must bring at least one token")
        if pad_to and (counts != 1).any():
            raise ValueError("only steps of single tokens can be padded")
        T = int(counts.sum())
        if T > self.max_tokens or R > self.max_requests:
            self.max_requests = max(R, self.max_requests)
            self._allocate(max(T, 2 * self.max_tokens))
        slots = np.full(R, self.cache.max_requests, dtype=np.int64)        # padding lanes: the spare slot
        slots[:n] = [e.slot for e in entries]
        starts = np.zeros(R, dtype=np.int64)
        starts[:n] = [e.start for e in entries]
        ends = starts + counts
        live = slots[:n]
        if n:
            if live.min() < 0 or live.max() >= self.cache.max_requests or len(np.unique(live)) != n:
                raise ValueError("a request appears twice in one step, or a slot that does not exist")
            if not self.cache.in_step[live].all():          # only open slots of a reserved step are marked
                bad = int(live[~self.cache.in_step[live]][0])
                raise RuntimeError(f"slot {bad} was not reserved for this step")
            wrong = starts[:n] != self.cache.length[live]
            if wrong.any():
                i = int(np.flatnonzero(wrong)[0])
                raise ValueError(f"slot {int(live[i])}: entry starts at {int(starts[i])}, the cache holds {int(self.cache.length[live[i]])}")
        limit = self.model.max_positions
        if int(ends.max()) > limit:
            raise ValueError(f"a request would reach {int(ends.max())} tokens, the model has {limit} positions")

        want_counts = [len(e.want) for e in entries]
        S = sum(want_counts) + (R - n)
        self.offsets, total = self._layout(T, R, S)
        h = self.host_np
        q_start = np.zeros(R + 1, dtype=np.int64)
        np.cumsum(counts, out=q_start[1:])
        tok = self._field(h, "tokens", T)
        pos = self._field(h, "positions", T)
        row_req = self._field(h, "row_req", T)
        # rows of the live entries, packed: tokens in order, positions = start + place within the entry
        live_rows = int(q_start[n])
        if live_rows:
            tok[:live_rows] = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=live_rows)
            of_row = np.repeat(np.arange(n, dtype=np.int64), counts[:n])
            row_req[:live_rows] = of_row
            pos[:live_rows] = starts[of_row] + (np.arange(live_rows, dtype=np.int64) - q_start[of_row])
        wanted_of = [None] * n          # by place in the caller's list: the logits keep the caller's order
        for r, e in enumerate(entries):
            if want_counts[r]:
                a, width = int(q_start[r]), int(counts[r])
                for w in e.want:
                    if not 0 <= w < width:
                        raise ValueError(f"want {w} is outside the entry's {width} tokens")
                wanted_of[order[r]] = [a + int(w) for w in e.want]
        wanted = [row for rows in wanted_of if rows for row in rows]
        for r in range(n, R):                      # padding lanes
            a = int(q_start[r])
            tok[a], pos[a], row_req[a] = 0, 0, r
            wanted.append(a)
        if tok.min() < 0 or tok.max() >= self.model.vocab_size:
            raise ValueError(f"token id outside [0, {self.model.vocab_size})")
        self._field(h, "want_rows", S)[:] = wanted
        self._field(h, "req_q_start", R + 1)[:] = q_start
        self._field(h, "req_pos0", R)[:] = starts
        self._field(h, "req_slot", R)[:] = slots
        self._field(h, "req_kv_len", R)[:] = ends
        if take_rows is not None:
            k = len(take_rows)
            if k > n or any(order[i] != i or lengths[i] != 1 for i in range(k)):
                raise ValueError("rows of another step's tokens can be named only for the first entries, of one token each")
            self._field(h, "take_rows", R)[:k] = take_rows
        C = self.cache.columns
        for g in self.kv_groups:
            rows = self._field(h, f"table{g}", R * C).reshape(R, C)
            rows[:n] = self.cache.table_rows(g, slots[:n])
            rows[n:] = 0                           # the padding page
        self.dev_buf[:total].copy_(self.host_buf[:total], non_blocking=True)
        self.h2d_bytes = total * 4
        if self.dev_buf.is_cuda:
            self._copied = torch.cuda.Event()
            self._copied.record()

        d = self.dev_buf
        tables = [None] * len(self.cache.groups)
        for g in self.kv_groups:
            tables[g] = self._field(d, f"table{g}", R * C).view(R, C)
        self.steps += 1
        self.rows_run += T
        return StepContext(
            num_rows=T, num_requests=R, num_wanted=S,
            tokens=self._field(d, "tokens", T), positions=self._field(d, "positions", T),
            row_req=self._field(d, "row_req", T), want_rows=self._field(d, "want_rows", S),
            req_q_start=self._field(d, "req_q_start", R + 1), req_pos0=self._field(d, "req_pos0", R),
            req_slot=self._field(d, "req_slot", R), req_kv_len=self._field(d, "req_kv_len", R),
            take_rows=self._field(d, "take_rows", R),
            tables=tables, cache=self.cache, dtype=self.model.dtype,
            host={"q_start": q_start, "pos0": starts, "slots": slots, "kv_len": ends, "counts": counts,
                  "order": np.asarray(order + list(range(n, R)), dtype=np.int64)},   # packed place -> caller's index
            max_q_len=int(counts.max()), max_kv_len=int(ends.max()), earlier_rows_settled=True,
            num_single=int((counts == 1).sum()))

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """The model on a prepared step: through the native step program when every part of the
        model can be lowered to one (``engine/program.py``), else through ``Model.forward``."""
        if not self._lowered:
            self._lowered = True
            if getattr(self.model, "loaded", False) and hasattr(self.model, "spec"):
                from .program import lower_model
                self._program = lower_model(self.model, self.cache)
        if self._program is not None:
            return self._program.run(ctx)
        return self.model.forward(ctx)

    def run(self, entries: Sequence[StepEntry], tokens_from: torch.Tensor | None = None,
            take_rows: Sequence[int] | None = None) -> torch.Tensor:
        """Logits [S, V] float32 on the device.  The caller has reserved the
        step in the cache manager and commits it afterwards.  ``tokens_from``
        (int32 on the device): tokens whose host copies are not known yet, entry i of
        the first ``len(take_rows)`` (each of one token) taking row ``take_rows[i]`` of
        it (None: every entry brings one token and takes row i)."""
        ctx = self.prepare(entries, take_rows=take_rows)
        if tokens_from is not None:
            self.place_tokens(ctx, len(entries), tokens_from, take_rows)
        return self.forward(ctx)

    @staticmethod
    def place_tokens(ctx: StepContext, n: int, tokens_from: torch.Tensor, take_rows) -> None:
        """Copies tokens of the step on the device from the sampled tokens of the step before:
        the first n entries' (row i of them each), or the first len(take_rows) entries' (row
        take_rows[i] each).  Single-token entries are packed first and in the caller's order, so
        these are the step's first rows."""
        if take_rows is None:
            if ctx.num_rows != ctx.num_requests:
                raise ValueError("without named rows, tokens can come from the device only for a step of single tokens")
            ctx.tokens[:n].copy_(tokens_from[:n])
        elif len(take_rows):
            k = len(take_rows)
            torch.index_select(tokens_from, 0, ctx.take_rows[:k], out=ctx.tokens[:k])
