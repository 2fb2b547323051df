"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes first, finishes and frees; decides what happens when pages run
out.  It is host code and needs no GPU: it talks to the cache manager's
bookkeeping only.

Rules, after the reference's continuous scheduler (``sched/continuous.py``):

* decoding first: every running request whose prompt is done gets one token, in
  round-robin order from a cursor, while the budget lasts (``:392-429``);
* then prompt portions: a request that is in the middle of its prompt goes on
  first, then waiting requests in arrival order; a portion is
  ``min(remaining, prefill_chunk, budget left)``; at most one request is in the
  middle of its prompt at a time: a new one is started only when its whole
  remaining prompt fits into this step or no other prompt is unfinished
  (``:431-534``, ``configs/scheduler.py:125``);
* a request's logits are wanted only when the portion ends at its last known
  token (``:527-529``);
* when pages run out (``:540-729``): halve the largest prompt portion; drop
  prompt portions of one token; then preempt the newest running request
  (its pages return, it goes back to the head of the waiting line and later
  recomputes its prompt and the tokens it generated); a request that could
  never fit was refused at admission, so a lone request always gets its pages.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np

from ..cache.manager import CacheManager, NoFreeSlot, OutOfPages, Reservation
from ..parts.base import KVNeed
from .request import GenerationResult, Request


class RequestRefused(ValueError):
    """The request can never run in this engine (too long, duplicate id, ...)."""


@dataclass(eq=False)             # a request is itself: lists of states are searched by identity
class RequestState:
    request: Request
    ordinal: int                      # admission order: FCFS key and seed source
    seed: int
    tokens: list[int]                 # prompt + generated so far
    computed: int = 0                 # tokens whose keys and values are cached
    slot: int | None = None
    generated: int = 0
    preemptions: int = 0
    finish_reason: str | None = None

    @property
    def prompt_len(self) -> int:
        return len(self.request.prompt_token_ids)

    @property
    def remaining(self) -> int:
        return len(self.tokens) - self.computed


@dataclass
class ScheduledEntry:
    state: RequestState
    start: int
    count: int
    sample: bool                      # the portion ends at the last known token
    pending: bool = False             # its one token is being sampled by the step in flight (see ``lookahead``)

    @property
    def is_decode(self) -> bool:
        """One token of a request whose other tokens are all cached."""
        state = self.state
        return self.pending or (len(state.tokens) - state.computed == 1 and state.computed > 0)


@dataclass
class ScheduledStep:
    entries: list[ScheduledEntry]
    reservation: Reservation
    decode_only: bool
    # A step planned ahead of the tokens of the step before it: its first len(token_rows) entries are the
    # ``pending`` ones, and token_rows[i] is the row of that step's sampled tokens that is entry i's token
    # (None: no entry is pending).
    token_rows: list[int] | None = None


@dataclass
class SchedulerStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    recomputed_tokens: int = 0
    shrunk_steps: int = 0
    blocked_steps: int = 0


class Scheduler:
    def __init__(self, cache: CacheManager, *, batch_tokens: int, prefill_chunk: int,
                 max_model_len: int, eos_token_id: int | None = None, base_seed: int = 0):
        from ..sampling.params import derive_seed

        self._derive_seed = derive_seed
        self.cache = cache
        self.batch_tokens = batch_tokens
        self.prefill_chunk = prefill_chunk
        self.max_model_len = max_model_len
        self.eos_token_id = eos_token_id
        self.base_seed = base_seed
        self.waiting: deque[RequestState] = deque()
        self.running: list[RequestState] = []       # in admission order
        self.states: dict[str, RequestState] = {}
        self.cursor = 0
        self.ordinal = 0
        self.stats = SchedulerStats()
        self.with_min_tokens = 0          # live requests that ask for a minimum of tokens (their stop ids are banned at first)

    # ------------------------------------------------------------ admission --
    def add(self, request: Request) -> RequestState:
        if request.request_id in self.states:
            raise RequestRefused(f"request id {request.request_id!r} is already in use")
        if request.max_total_len > self.max_model_len:
            raise RequestRefused(
                f"prompt of {len(request.prompt_token_ids)} tokens + max_tokens {request.stop.max_tokens} "
                f"exceeds the model length {self.max_model_len}")
        P = self.cache.page_size
        for g, group in enumerate(self.cache.groups):
            if not isinstance(group.need, KVNeed):
                continue
            # what the request holds in this group at its longest: all its tokens, or, behind a
            # window, the window plus the largest portion that one step may add
            tokens = request.max_total_len
            if group.need.window is not None:
                tokens = min(tokens, group.need.window + min(self.prefill_chunk, self.batch_tokens) + P)
            have = self.cache.pages_of[g] - 1
            if -(-tokens // P) > have:
                raise RequestRefused(
                    f"the request needs {-(-tokens // P)} pages of cache group {group.name!r}, which has {have}")
        seed = request.sampling.seed
        if seed is None:
            seed = self._derive_seed(self.base_seed + self.ordinal)
        state = RequestState(request, self.ordinal, seed, list(request.prompt_token_ids))
        self.ordinal += 1
        self.states[request.request_id] = state
        self.waiting.append(state)
        if request.stop.min_tokens > 0:
            self.with_min_tokens += 1
        return state

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------- planning --
    def schedule(self) -> ScheduledStep | None:
        """The next step, or None when nothing can run (no work, or a single request that the
        cache cannot hold).  A pass that ends with nothing to run although several requests
        hold pages gives the newest holder's pages back and plans again: two half-recomputed
        prompts that fill the cache between them must not wait for each other for ever."""
        while True:
            before = self.stats.preemptions
            plan = self._plan()
            if plan is not None:
                return plan
            if self.stats.preemptions == before:          # the pass itself freed nothing
                victim = self._pick_victim([])
                if victim is None:
                    self.stats.blocked_steps += 1
                    return None
                self._preempt(victim)

    def _plan(self, after: ScheduledStep | None = None) -> ScheduledStep | None:
        """One pass of the rules above.  ``after``: the step in flight (already advanced, its
        tokens not yet known), when the step is planned ahead of them: see ``lookahead``."""
        budget = self.batch_tokens
        entries: list[ScheduledEntry] = []
        ahead = after is not None
        row_of: dict[int, int] = {}            # id(state) -> row of the step in flight that samples its next token
        leaving: set[int] = set()              # requests that the token on its way finishes by length
        if ahead:
            row = 0
            for e in after.entries:
                if not e.sample:
                    continue
                s = e.state
                if s.finish_reason is None:
                    if len(s.tokens) != s.computed:
                        return None            # not advanced, or resolved already: nothing to plan ahead of
                    stop = s.request.stop
                    if s.generated + 1 >= stop.max_tokens or len(s.tokens) + 1 >= self.max_model_len:
                        leaving.add(id(s))
                    else:
                        row_of[id(s)] = row
                row += 1

        # 1. decoding first, round robin from the cursor
        if ahead:
            # every decoder's token is on its way; one whose token is known was left out of the step in
            # flight for want of budget, and the pass that knows the tokens takes the turns
            if any(len(s.tokens) - s.computed == 1 and s.computed > 0 for s in self.running):
                return None
            decoders = [s for s in self.running if id(s) in row_of]
            if len(decoders) > budget:
                return None
            for s in decoders:
                entries.append(ScheduledEntry(s, s.computed, 1, True, pending=True))
                budget -= 1
        else:
            decoders = [s for s in self.running if len(s.tokens) - s.computed == 1 and s.computed > 0]
            if decoders:
                if len(decoders) > budget:          # not all fit: take turns
                    start = self.cursor % len(decoders)
                    decoders = (decoders[start:] + decoders[:start])[:budget]
                    self.cursor += budget
                for s in decoders:
                    entries.append(ScheduledEntry(s, s.computed, 1, True))
                    budget -= 1

        # 2. prompt portions: the unfinished prompt first, then waiting requests
        partial = [s for s in self.running if (len(s.tokens) - s.computed > 1 or s.computed == 0)
                   and id(s) not in row_of and id(s) not in leaving]
        admitted: list[RequestState] = []
        for s in partial:
            if budget < 1:
                break
            n = min(s.remaining, self.prefill_chunk, budget)
            entries.append(ScheduledEntry(s, s.computed, n, n == s.remaining))
            budget -= n
        unfinished = any(e.count < e.state.remaining for e in entries if e.state in partial) or \
            any(s not in [e.state for e in entries] for s in partial)
        while self.waiting and budget >= 1:
            s = self.waiting[0]
            n = min(s.remaining, self.prefill_chunk, budget)
            if n < s.remaining and unfinished:
                break                       # one unfinished prompt at a time
            try:
                s.slot = self.cache.open(s.request.request_id)
            except NoFreeSlot:
                break
            self.waiting.popleft()
            self.running.append(s)
            admitted.append(s)
            entries.append(ScheduledEntry(s, 0, n, n == s.remaining))
            budget -= n
            if n < s.remaining:
                unfinished = True

        # 3. pages.  What each entry needs is worked out once, per group, from the pages its request holds; a rung
        # of the ladder below (halve the largest portion, drop the last portion, preempt the newest request) then
        # changes one number, and the reservation is made once, for the entries that fit.  (Reserving anew at every
        # rung cost a step of 200 requests a dozen passes over all of them.)
        shrunk = False
        reservation = None
        page = self.cache.page_size
        held = self.cache.pages_held([e.state.slot for e in entries]) if entries else []
        paged = [g for g, h in enumerate(held) if h is not None]
        decode = [e.is_decode for e in entries]

        def needs(i: int) -> list[int]:
            end_pages = -(-(entries[i].start + entries[i].count) // page)
            return [max(0, end_pages - int(held[g][i])) for g in paged]

        need = [needs(i) for i in range(len(entries))]
        total = [sum(n[k] for n in need) for k in range(len(paged))]

        def drop(i: int) -> None:
            for k in range(len(paged)):
                total[k] -= need[i][k]
            del entries[i], need[i], decode[i]
            for g in paged:
                held[g] = np.delete(held[g], i)

        while entries:
            if all(total[k] <= self.cache.free_pages(g) for k, g in enumerate(paged)):
                try:
                    reservation = self.cache.reserve([(e.state.slot, e.start, e.count) for e in entries])
                    break
                except OutOfPages:            # not expected after the arithmetic above; the ladder goes on
                    pass
            if ahead:
                # short of pages: the pass that knows who has finished decides what gives; what this pass
                # admitted goes back to the head of the line, in its order
                for s in reversed(admitted):
                    self.cache.close(s.slot)
                    s.slot = None
                    self.running.remove(s)
                    self.waiting.appendleft(s)
                return None
            shrunk = True
            prefills = [i for i in range(len(entries)) if not decode[i]]
            big = [i for i in prefills if entries[i].count > 1]
            if big:
                i = max(big, key=lambda i: entries[i].count)
                entries[i].count //= 2
                entries[i].sample = False
                fresh = needs(i)
                for k in range(len(paged)):
                    total[k] += fresh[k] - need[i][k]
                need[i] = fresh
            elif prefills:
                drop(prefills[-1])
            else:
                victim = self._pick_victim(entries)
                if victim is None:
                    entries.clear()
                    break
                for i in reversed([i for i, e in enumerate(entries) if e.state is victim]):
                    drop(i)
                self._preempt(victim)
        if shrunk:
            self.stats.shrunk_steps += 1
        if not entries:
            return None
        self.stats.steps += 1
        decoding = sum(1 for e in entries if e.is_decode)
        self.stats.decode_tokens += decoding
        self.stats.prefill_tokens += sum(e.count for e in entries) - decoding
        return ScheduledStep(entries, reservation, decoding == len(entries),
                             [row_of[id(e.state)] for e in entries if e.pending] or None)

    def _pick_victim(self, entries) -> RequestState | None:
        """The newest running request that holds pages; never the only one."""
        holders = [s for s in self.running if s.computed > 0 or any(e.state is s for e in entries)]
        if len(holders) <= 1:
            return None
        return max(holders, key=lambda s: s.ordinal)

    def _preempt(self, state: RequestState) -> None:
        self.cache.close(state.slot)
        self.stats.preemptions += 1
        self.stats.recomputed_tokens += state.computed
        state.slot, state.computed = None, 0
        state.preemptions += 1
        self.running.remove(state)
        self.waiting.appendleft(state)

    # -------------------------------------------------------------- results --
    def update(self, step: ScheduledStep, sampled: dict[str, int]) -> list[RequestState]:
        """The step ran: commit it, append the sampled tokens, finish and free.
        ``sampled``: request id -> token for every entry with ``sample``."""
        self.advance(step)
        return self.resolve(step, sampled)

    def advance(self, step: ScheduledStep) -> None:
        """The step has been handed to the GPU and will complete: its tokens count
        as cached from now on (the cache manager's lengths move, pages that a window
        has passed return).  The sampled tokens come later, through ``resolve``."""
        self.cache.commit(step.reservation)
        for e in step.entries:
            e.state.computed = e.start + e.count

    def resolve(self, step: ScheduledStep, sampled: dict[str, int]) -> list[RequestState]:
        """The step's sampled tokens are on the host: append them, finish and free.
        An entry whose request has finished meanwhile (it was planned ahead, see
        ``lookahead``) is skipped: its token belongs to nobody."""
        finished = []
        for e in step.entries:
            s = e.state
            if not e.sample or s.finish_reason is not None:
                continue
            token = int(sampled[s.request.request_id])
            s.tokens.append(token)
            s.generated += 1
            reason = self._finish_reason(s, token)
            if reason is not None:
                self._finish(s, reason)
                finished.append(s)
        return finished

    def lookahead(self, step: ScheduledStep) -> ScheduledStep | None:
        """The step after ``step``, planned before ``step``'s tokens are known, or None
        when that cannot be done without guessing more than "nobody stops on a stop
        id".  ``step`` has been advanced.  The rules are ``_plan``'s, with three
        differences.  A request whose next token ``step`` samples decodes with that
        token, which the engine takes from the device (``pending`` entries, first in
        the step; ``token_rows``).  A request that reaches a length limit with the
        token on its way is known to finish: it is left out, and its pages and slot
        stay taken until its token is there.  And nothing is taken away to make room:
        when pages are short, or more requests decode than the budget holds, the
        answer is None and the step is planned when the tokens are known.  A request
        that stops on the token on its way (EOS, a stop id) has then one more token
        computed than it needed; ``resolve`` drops it.  The reference keeps one step in
        flight (``configs/scheduler.py:131``); this is the same loop with the host's
        share of the next step done while the GPU works on this one."""
        if not self.running and not self.waiting:
            return None
        return self._plan(after=step)

    def banned_tokens(self, s: RequestState, pending: int = 0) -> tuple[int, ...]:
        """Token ids that ``s`` must not sample next: its stop ids, and EOS unless it
        ignores it, while it has generated fewer than ``min_tokens``
        (``request/stream.py:130-136``).  ``pending``: tokens of ``s`` that are sampled
        but not yet on the host."""
        stop = s.request.stop
        if s.generated + pending >= stop.min_tokens:
            return ()
        ids = tuple(stop.stop_token_ids)
        if not stop.ignore_eos and self.eos_token_id is not None:
            ids += (self.eos_token_id,)
        return ids

    def _finish_reason(self, s: RequestState, token: int) -> str | None:
        """``request/stream.py:138-163``: a stop id or EOS ends the request once more than
        ``min_tokens`` tokens exist, this one included (earlier ones are banned before
        sampling and cannot appear); the length limit always."""
        stop = s.request.stop
        if s.generated > stop.min_tokens:
            if token in stop.stop_token_ids:
                return "stop"
            if not stop.ignore_eos and self.eos_token_id is not None and token == self.eos_token_id:
                return "eos"
        if s.generated >= stop.max_tokens or len(s.tokens) >= self.max_model_len:
            return "length"
        return None

    def _finish(self, s: RequestState, reason: str) -> None:
        s.finish_reason = reason
        if s.slot is not None:
            self.cache.close(s.slot)
            s.slot = None
        if s in self.running:
            self.running.remove(s)
        if s in self.waiting:
            self.waiting.remove(s)
        del self.states[s.request.request_id]
        if s.request.stop.min_tokens > 0:
            self.with_min_tokens -= 1

    def abort(self, request_id: str) -> RequestState | None:
        s = self.states.get(request_id)
        if s is None:
            return None
        if s.slot is not None and self.cache.in_step[s.slot]:
            raise RuntimeError("a request cannot be aborted while its step runs")
        self._finish(s, "abort")
        return s

    def result_of(self, s: RequestState) -> GenerationResult:
        return GenerationResult(s.request.request_id, list(s.request.prompt_token_ids),
                                s.tokens[s.prompt_len:], s.finish_reason, s.preemptions)
