"""Trace replay: feeds given token ids through a model step by step and writes
logits.  It samples nothing.  It drives the model, step function, cache manager
and kernels that generation uses, and has no forward pass, cache or loader of
its own.  (The reference has no such program; its nearest instrument is the
forward observer of ``runner/paged_runner.py:215-239``.)

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input: one JSON object a line,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose
logits are wanted; all entries of a step run as one batch.  ``end``: requests
that are finished after this step; their pages and slot are given back.  For a
step that wants something, ``<out>/<step>.f32`` holds the logits at the wanted
places, in the order of the entries and of ``want``, as little-endian float32
[wanted, vocab].  After every step a line ``done <step>`` is printed and
flushed.  ``--max-tokens``: the most tokens that live requests hold at any
time, each request's count rounded up to a multiple of 64; the cache pool is
made for exactly that many.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

MAX_LIVE = 4
ROUND_TO = 64


class ReplaySession:
    """The engine parts that a replay drives: model, cache manager, step runner."""

    def __init__(self, model_dir, dtype: str, max_tokens: int, page_size: int = 16,
                 max_requests: int = MAX_LIVE, device: str = "cuda"):
        from . import ops
        from .cache.manager import CacheManager
        from .engine.loading import load_model
        from .engine.step import StepRunner

        ops.library()
        self.config, self.model = load_model(model_dir, dtype, device)
        pages = -(-max_tokens // page_size) + 1                # + the padding page
        self.cache = CacheManager(self.model.groups, kv_pages=pages, page_size=page_size,
                                  max_requests=max_requests, max_len=self.model.max_positions,
                                  dtype=self.model.dtype, device=device)
        self.runner = StepRunner(self.model, self.cache,
                                 max_tokens=min(max_tokens, 4 * self.model.max_positions))
        self.slots: dict[str, int] = {}

    def step(self, record: dict):
        """Runs one trace record.  Returns logits [wanted, vocab] (device,
        float32) or None when the step brought no entries."""
        from .engine.step import StepEntry

        entries = []
        for item in record.get("entries", []):
            rid = str(item["id"])
            if rid not in self.slots:
                self.slots[rid] = self.cache.open(rid)
            slot = self.slots[rid]
            entries.append(StepEntry(slot, int(self.cache.length[slot]), item["tokens"], item.get("want", [])))
        logits = None
        if entries:
            reservation = self.cache.reserve([(e.slot, e.start, len(e.tokens)) for e in entries])
            try:
                logits = self.runner.run(entries)
            except BaseException:
                self.cache.rollback(reservation)
                raise
            self.cache.commit(reservation)
        for rid in record.get("end", []):
            rid = str(rid)
            if rid in self.slots:
                self.cache.close(self.slots.pop(rid))
        return logits


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True)
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--max-requests", type=int, default=MAX_LIVE)
    args = parser.parse_args(argv)
    if ROUND_TO % args.page_size:
        parser.error(f"--page-size must divide {ROUND_TO}")

    print("[trace_run] loading the model (kernels are compiled at the first call)", file=sys.stderr, flush=True)
    import torch

    session = ReplaySession(args.model, args.dtype, args.max_tokens, args.page_size, args.max_requests)
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    print("[trace_run] ready", file=sys.stderr, flush=True)

    for number, line in enumerate(sys.stdin, 1):
        line = line.strip()
        if not line:
            continue
        # A step that cannot run (not JSON, an unknown token, more tokens than the pool holds, a fifth
        # live request, ...) ends the program with one line that says which and why, and status 1.
        record = None
        try:
            record = json.loads(line)
            logits = session.step(record)
        except Exception as problem:
            step = record.get("step", "?") if isinstance(record, dict) else "?"
            print(f"trace_run: input line {number} (step {step}): {type(problem).__name__}: {problem}", file=sys.stderr, flush=True)
            return 1
        if logits is not None and logits.shape[0]:
            logits.to(torch.float32).cpu().numpy().astype("<f4").tofile(out_dir / f"{record['step']}.f32")
        else:
            torch.cuda.synchronize()
        print(f"done {record['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
