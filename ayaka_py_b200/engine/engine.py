"""The generation loop: schedule, step, sample, read back, commit.

One step is in flight at a time, as in the reference's default
(``configs/scheduler.py:131``; ``runtime/engine.py:180-279``).  With
``EngineConfig.lookahead`` the host's share of the next step overlaps the GPU's
work on this one: the next step is planned by the scheduler's own rules while
this step's tokens are on their way (``Scheduler.lookahead``: requests whose
token is being sampled decode with it, prompts go on in portions, waiting
requests are admitted; nothing is preempted or shrunk ahead of the tokens),
uploaded and launched, the tokens that are not on the host yet copied from the
sampler's output on the device.  The tokens a request sees are the same either
way; a request that stops on EOS or a stop id has one more position
computed than it needed, which is dropped.
"""

from __future__ import annotations

import time

import torch

from ..cache.manager import CacheManager, pages_for_budget
from ..config.engine import EngineConfig
from ..sampling.sampler import Sampler
from .request import GenerationResult, Request
from .scheduler import ScheduledStep, Scheduler
from .step import StepEntry, StepRunner


class Engine:
    def __init__(self, model, config: EngineConfig, eos_token_id: int | None = None):
        self.model = model
        self.config = config
        self.max_model_len = min(config.max_model_len or model.max_positions, model.max_positions)
        pages = config.kv_pages
        if config.kv_cache_bytes is not None:
            pages = pages_for_budget(model.groups, config.kv_cache_bytes, page_size=config.page_size,
                                     max_requests=config.max_requests, max_len=self.max_model_len,
                                     step_tokens=config.batch_tokens, dtype=model.dtype)
        self.cache = CacheManager(model.groups, kv_pages=pages, page_size=config.page_size,
                                  max_requests=config.max_requests, max_len=self.max_model_len,
                                  dtype=model.dtype, device=model.device)
        self.runner = StepRunner(model, self.cache, max_tokens=config.batch_tokens,
                                 max_requests=config.max_requests)
        self.scheduler = Scheduler(self.cache, batch_tokens=config.batch_tokens,
                                   prefill_chunk=config.prefill_chunk, max_model_len=self.max_model_len,
                                   eos_token_id=eos_token_id, base_seed=config.seed)
        self.sampler = Sampler(model.device, max_rows=config.max_requests)
        self.finished: dict[str, GenerationResult] = {}
        self.decode_graphs = None
        if config.decode_graph:
            from .graphs import DecodeGraphs
            self.decode_graphs = DecodeGraphs(self.runner, model, config.max_requests)
        self.lookahead = bool(getattr(config, "lookahead", True)) and torch.cuda.is_available()
        self._inflight: _Launched | None = None
        self._copy_stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self._pinned: list[torch.Tensor] = []      # host landing places of sampled tokens, reused
        self.host_seconds = 0.0                    # time inside step() that was not spent waiting for the GPU
        self.steps_run = 0

    def submit(self, request: Request) -> None:
        self.scheduler.add(request)

    def abort(self, request_id: str) -> None:
        self._drain()
        s = self.scheduler.abort(request_id)
        if s is not None:
            self.finished[request_id] = self.scheduler.result_of(s)

    def has_work(self) -> bool:
        return self._inflight is not None or self.scheduler.has_work()

    def step(self) -> list[GenerationResult]:
        """Runs one step to its end (its tokens on the host) and returns the
        requests that finished in it.  The step after it may already be running."""
        began = time.perf_counter()
        self._waited = 0.0
        if self._inflight is None:
            plan = self.scheduler.schedule()
            if plan is None:
                if self.scheduler.has_work():
                    raise RuntimeError("the scheduler can run nothing although requests wait: the cache is "
                                       "too small for what was admitted")
                return []
            self._inflight = self._launch(plan)
        current = self._inflight
        ahead = None
        if self.lookahead:
            plan = self.scheduler.lookahead(current.plan)
            if plan is not None:
                ahead = self._launch(plan, tokens_from=current.sampled)
        self._inflight = ahead
        results = self._finish_step(current)
        self.host_seconds += time.perf_counter() - began - self._waited
        self.steps_run += 1
        return results

    def _launch(self, plan: ScheduledStep, tokens_from: torch.Tensor | None = None) -> "_Launched":
        """Hands a planned step to the GPU: upload, forward, sampling, and the copy
        of the sampled tokens to the host on a stream of its own.  ``tokens_from``:
        the sampled tokens of the step before, still on the device; the plan's
        ``pending`` entries take theirs from there (``token_rows``)."""
        take = plan.token_rows                  # the first len(take) entries decode with tokens that are still on their way
        if take and tokens_from is None:
            raise RuntimeError("a step planned ahead needs the sampled tokens of the step before it")
        try:
            entries = [StepEntry(e.state.slot, e.start,
                                 [0] if e.pending else e.state.tokens[e.start:e.start + e.count],
                                 [e.count - 1] if e.sample else []) for e in plan.entries]
            sampling = [e for e in plan.entries if e.sample]
            rows = [e.state for e in sampling]
            if self.decode_graphs is not None and plan.decode_only:
                logits = self.decode_graphs.run(entries, tokens_from=tokens_from if take else None, take_rows=take)
            else:
                logits = self.runner.run(entries, tokens_from=tokens_from if take else None, take_rows=take)
            sampled = host = done = None
            if rows:
                pending = [1 if e.pending else 0 for e in sampling]      # a token of the row is still on its way
                banned = ([(i, t) for i, s in enumerate(rows) for t in self.scheduler.banned_tokens(s, pending[i])]
                          if self.scheduler.with_min_tokens else ())
                sampled = self.sampler.sample(logits, [s.request.sampling for s in rows], [s.seed for s in rows],
                                              [s.generated + p for s, p in zip(rows, pending)], banned=banned)
                host = self._pinned.pop() if self._pinned else None
                if host is None or host.numel() < len(rows):
                    host = torch.empty(max(len(rows), self.config.max_requests), dtype=torch.int32, pin_memory=True)
                ready = torch.cuda.Event()
                ready.record()
                with torch.cuda.stream(self._copy_stream):
                    self._copy_stream.wait_event(ready)
                    host[:len(rows)].copy_(sampled, non_blocking=True)
                    done = torch.cuda.Event()
                    done.record()
        except BaseException:
            self.cache.rollback(plan.reservation)
            raise
        self.scheduler.advance(plan)
        return _Launched(plan, rows, sampled, host, done)

    def _finish_step(self, launched: "_Launched") -> list[GenerationResult]:
        sampled = {}
        if launched.rows:
            t0 = time.perf_counter()
            launched.done.synchronize()
            self._waited = getattr(self, "_waited", 0.0) + time.perf_counter() - t0
            tokens = launched.host[:len(launched.rows)].tolist()
            self._pinned.append(launched.host)
            for s, token in zip(launched.rows, tokens):
                sampled[s.request.request_id] = token
        elif self._inflight is None:
            t0 = time.perf_counter()
            torch.cuda.synchronize()
            self._waited = getattr(self, "_waited", 0.0) + time.perf_counter() - t0
        done = self.scheduler.resolve(launched.plan, sampled)
        results = [self.scheduler.result_of(s) for s in done]
        for r in results:
            self.finished[r.request_id] = r
        return results

    def _drain(self) -> None:
        """Brings the loop to a point where no step is in flight."""
        while self._inflight is not None:
            current, self._inflight = self._inflight, None
            self._finish_step(current)

    def run_until_idle(self) -> dict[str, GenerationResult]:
        while self.has_work():
            self.step()
        out, self.finished = self.finished, {}
        return out


class _Launched:
    """A step on the GPU: its plan, the requests whose tokens it samples, the
    sampler's output on the device, its landing place on the host and the event
    that says it has landed."""

    __slots__ = ("plan", "rows", "sampled", "host", "done")

    def __init__(self, plan, rows, sampled, host, done):
        self.plan, self.rows, self.sampled, self.host, self.done = plan, rows, sampled, host, done
