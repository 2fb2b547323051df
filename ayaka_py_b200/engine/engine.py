"""The generation loop: schedule, step, sample, read back, commit.

One step is in flight at a time, as in the reference's default
(``configs/scheduler.py:131``): the next step is planned after this step's
tokens are on the host (``runtime/engine.py:180-279``)."""

from __future__ import annotations

import torch

from ..cache.manager import CacheManager
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
        self.cache = CacheManager(model.groups, kv_pages=config.kv_pages, page_size=config.page_size,
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

    def submit(self, request: Request) -> None:
        self.scheduler.add(request)

    def abort(self, request_id: str) -> None:
        s = self.scheduler.abort(request_id)
        if s is not None:
            self.finished[request_id] = self.scheduler.result_of(s)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> list[GenerationResult]:
        """Plans and runs one step.  Returns the requests that finished in it."""
        plan = self.scheduler.schedule()
        if plan is None:
            if self.scheduler.has_work():
                raise RuntimeError("the scheduler can run nothing although requests wait: the cache is "
                                   "too small for what was admitted")
            return []
        try:
            tokens = self._run(plan)
        except BaseException:
            self.cache.rollback(plan.reservation)
            raise
        sampled = {}
        rows = [e for e in plan.entries if e.sample]
        for e, token in zip(rows, tokens):
            sampled[e.state.request.request_id] = token
        done = self.scheduler.update(plan, sampled)
        results = [self.scheduler.result_of(s) for s in done]
        for r in results:
            self.finished[r.request_id] = r
        return results

    def _run(self, plan: ScheduledStep) -> list[int]:
        entries = [StepEntry(e.state.slot, e.start, e.state.tokens[e.start:e.start + e.count],
                             [e.count - 1] if e.sample else []) for e in plan.entries]
        rows = [e.state for e in plan.entries if e.sample]
        if self.decode_graphs is not None and plan.decode_only:
            logits = self.decode_graphs.run(entries)
        else:
            logits = self.runner.run(entries)
        if not rows:
            torch.cuda.synchronize()
            return []
        tokens = self.sampler.sample(logits, [s.request.sampling for s in rows], [s.seed for s in rows],
                                     [s.generated for s in rows])
        return tokens.cpu().tolist()

    def run_until_idle(self) -> dict[str, GenerationResult]:
        while self.has_work():
            self.step()
        out, self.finished = self.finished, {}
        return out
