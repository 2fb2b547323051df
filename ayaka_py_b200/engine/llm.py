"""The Python entry point: ``LLM(model).generate(prompts, ...)``.

The reference's facade is ``AyakaLLM.submit(Request) -> Future[OutputStream]``
over an owner thread (``runtime/llm.py:27-277``); this one submits all prompts,
runs the engine loop to completion in the caller's thread and returns the
results in the order of the prompts.  It works on token ids."""

from __future__ import annotations

from typing import Sequence

from ..config.engine import EngineConfig
from ..config.model import ModelConfig
from ..sampling.params import SamplingParams
from .engine import Engine
from .loading import load_model, random_model
from .request import GenerationResult, Request, StopCriteria


class LLM:
    def __init__(self, model, engine_config: EngineConfig | None = None, *, seed: int = 0, **options):
        """``model``: a folder with config.json and model.safetensors, or a
        ``ModelConfig`` for random weights drawn from ``seed``.  ``options``
        are ``EngineConfig`` fields (dtype, kv_pages, page_size, max_requests,
        batch_tokens, prefill_chunk, max_model_len, decode_graph, lookahead)."""
        self.engine_config = engine_config or EngineConfig(**options)
        if isinstance(model, ModelConfig):
            self.model_config = model
            self.model = random_model(model, seed, self.engine_config.dtype)
        else:
            self.model_config, self.model = load_model(model, self.engine_config.dtype)
        self.engine = Engine(self.model, self.engine_config,
                             eos_token_id=getattr(self.model_config, "eos_token_id", None))
        self._next_id = 0

    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling: SamplingParams | Sequence[SamplingParams] | None = None,
                 stop: StopCriteria | Sequence[StopCriteria] | None = None) -> list[GenerationResult]:
        n = len(prompts)
        samplings = list(sampling) if isinstance(sampling, (list, tuple)) else [sampling or SamplingParams()] * n
        stops = list(stop) if isinstance(stop, (list, tuple)) else [stop or StopCriteria()] * n
        if len(samplings) != n or len(stops) != n:
            raise ValueError("one SamplingParams / StopCriteria per prompt, or one for all")
        ids = []
        for prompt, sp, st in zip(prompts, samplings, stops):
            rid = f"req-{self._next_id}"
            self._next_id += 1
            self.engine.submit(Request(rid, list(prompt), sp, st))
            ids.append(rid)
        done = self.engine.run_until_idle()
        return [done[rid] for rid in ids]
