"""Command line: ``python -m ayaka_py_b200 <command>``.

``generate MODEL_PATH``  generate from prompts given as token ids;
``random-weights OUT``   write a model folder from a configuration and a seed;
``replay``               the trace replay program (same as ``bin/trace_run``).

Engine options carry the reference's names and defaults
(``commands/cli.py:19-47``: ``--dtype``, ``--kv-pages``, ``--page-size``,
``--max-requests``, ``--max-model-len``, ``--batch-tokens``, ``--prefill-chunk``,
``--decode-graph``); sampling options those of its ``SamplingParams`` and
``StopCriteria``.  The reference's only command is an HTTP server; servers and
tokenizers are not part of this engine, so prompts and results are token ids.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PRESETS = {
    "gpt2": dict(n_layer=12, n_embd=768, n_head=12),
    "gpt2-medium": dict(n_layer=24, n_embd=1024, n_head=16),
    "gpt2-large": dict(n_layer=36, n_embd=1280, n_head=20),
    "gpt2-xl": dict(n_layer=48, n_embd=1600, n_head=25),
}


def _add_engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--dtype", choices=("float32", "bfloat16"), default="bfloat16")
    p.add_argument("--kv-pages", type=int, default=1024)
    p.add_argument("--kv-cache-bytes", type=int, default=None,
                   help="instead of --kv-pages: a byte budget for the whole cache, split over the cache groups")
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--max-requests", type=int, default=32)
    p.add_argument("--max-model-len", type=int, default=None)
    p.add_argument("--batch-tokens", type=int, default=256)
    p.add_argument("--prefill-chunk", type=int, default=128)
    p.add_argument("--decode-graph", action=argparse.BooleanOptionalAction, default=True,
                   help="replay pure-decode steps from CUDA graphs (on by default; --no-decode-graph launches every kernel)")


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="ayaka_py_b200")
    commands = parser.add_subparsers(dest="command", required=True)

    gen = commands.add_parser("generate", help="generate token ids from prompts of token ids")
    gen.add_argument("model_path", type=Path)
    _add_engine_options(gen)
    gen.add_argument("--prompt-ids", action="append", default=[],
                     help="comma-separated token ids; may be given several times")
    gen.add_argument("--prompt-file", type=Path, help="JSON list of lists of token ids")
    gen.add_argument("--random-prompts", type=int, default=0, help="number of prompts of random ids")
    gen.add_argument("--prompt-len", type=int, default=16)
    gen.add_argument("--max-tokens", type=int, default=128)
    gen.add_argument("--min-tokens", type=int, default=0)
    gen.add_argument("--temperature", type=float, default=1.0)
    gen.add_argument("--top-k", type=int, default=-1)
    gen.add_argument("--top-p", type=float, default=1.0)
    gen.add_argument("--min-p", type=float, default=0.0)
    gen.add_argument("--seed", type=int, default=None)
    gen.add_argument("--stop-token-ids", default="", help="comma-separated token ids")
    gen.add_argument("--ignore-eos", action="store_true")

    rnd = commands.add_parser("random-weights", help="write config.json and model.safetensors from a seed")
    rnd.add_argument("out", type=Path)
    rnd.add_argument("--config", type=Path, help="a config.json to take the sizes from")
    rnd.add_argument("--preset", choices=sorted(PRESETS), default=None)
    rnd.add_argument("--seed", type=int, default=1234)
    rnd.add_argument("--dtype", choices=("float32", "bfloat16"), default="bfloat16")

    ben = commands.add_parser("bench", help="decode and prefill throughput of a model folder, one JSON line")
    ben.add_argument("model_path", type=Path)
    _add_engine_options(ben)
    ben.add_argument("--batch", type=int, default=8, help="requests that decode together")
    ben.add_argument("--prompt-len", type=int, default=128)
    ben.add_argument("--steps", type=int, default=64, help="decode steps that are timed")
    ben.add_argument("--warmup", type=int, default=8)
    ben.add_argument("--seed", type=int, default=0)

    commands.add_parser("replay", help="trace replay; see bin/trace_run", add_help=False)
    return parser


def _generate(args) -> int:
    import numpy as np

    from ..config.engine import EngineConfig
    from ..engine.llm import LLM
    from ..engine.request import StopCriteria
    from ..sampling.params import SamplingParams

    if not (args.model_path / "config.json").is_file():
        print(f"model_path does not contain config.json: {args.model_path}", file=sys.stderr)
        return 2
    config = EngineConfig(dtype=args.dtype, kv_pages=args.kv_pages, kv_cache_bytes=args.kv_cache_bytes, page_size=args.page_size,
                          max_requests=args.max_requests, max_model_len=args.max_model_len,
                          batch_tokens=args.batch_tokens, prefill_chunk=args.prefill_chunk,
                          decode_graph=args.decode_graph)
    llm = LLM(args.model_path, config)
    prompts = [[int(x) for x in text.split(",") if x.strip()] for text in args.prompt_ids]
    if args.prompt_file:
        prompts += json.loads(args.prompt_file.read_text())
    if args.random_prompts:
        rs = np.random.RandomState(args.seed or 0)
        prompts += [rs.randint(0, llm.model.vocab_size, args.prompt_len).tolist()
                    for _ in range(args.random_prompts)]
    if not prompts:
        print("no prompts: give --prompt-ids, --prompt-file or --random-prompts", file=sys.stderr)
        return 2
    stop_ids = tuple(int(x) for x in args.stop_token_ids.split(",") if x.strip())
    sampling = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                              min_p=args.min_p, seed=args.seed)
    stop = StopCriteria(max_tokens=args.max_tokens, min_tokens=args.min_tokens, stop_token_ids=stop_ids,
                        ignore_eos=args.ignore_eos)
    for result in llm.generate(prompts, sampling, stop):
        print(json.dumps({"request_id": result.request_id, "prompt_tokens": len(result.prompt_token_ids),
                          "token_ids": result.token_ids, "finish_reason": result.finish_reason}))
    return 0


def _bench(args) -> int:
    """Prompts of random ids through the engine's own loop: the time of the prompt steps, then
    ``--steps`` decode steps between two CUDA events (after ``--warmup`` untimed ones)."""
    import time

    import numpy as np
    import torch

    from ..config.engine import EngineConfig
    from ..engine.llm import LLM
    from ..engine.request import Request, StopCriteria
    from ..sampling.params import SamplingParams

    if not (args.model_path / "config.json").is_file():
        print(f"model_path does not contain config.json: {args.model_path}", file=sys.stderr)
        return 2
    pages = max(args.kv_pages, args.batch * -(-(args.prompt_len + args.steps + args.warmup + 2) // args.page_size) + 1)
    config = EngineConfig(dtype=args.dtype, kv_pages=pages, kv_cache_bytes=args.kv_cache_bytes, page_size=args.page_size,
                          max_requests=max(args.max_requests, args.batch), max_model_len=args.max_model_len,
                          batch_tokens=max(args.batch_tokens, args.batch), prefill_chunk=args.prefill_chunk,
                          decode_graph=args.decode_graph)
    llm = LLM(args.model_path, config)
    engine = llm.engine
    new_tokens = args.steps + args.warmup + 2
    if args.prompt_len + new_tokens > engine.max_model_len:
        raise ValueError(f"prompts of {args.prompt_len} ids and {new_tokens} new tokens exceed the model length {engine.max_model_len}")
    rs = np.random.RandomState(args.seed)
    for i in range(args.batch):
        engine.submit(Request(f"bench-{i}", rs.randint(0, llm.model.vocab_size, args.prompt_len).tolist(),
                              SamplingParams(temperature=0.0), StopCriteria(max_tokens=new_tokens, ignore_eos=True)))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    prompt_steps = 0
    while any(s.computed < s.prompt_len for s in engine.scheduler.states.values()):
        engine.step()
        prompt_steps += 1
    torch.cuda.synchronize()
    prompt_s = time.perf_counter() - t0
    for _ in range(args.warmup):
        engine.step()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.steps):
        engine.step()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    engine.run_until_idle()
    engine.cache.assert_clean()
    print(json.dumps({"model": str(args.model_path), "dtype": config.dtype, "batch": args.batch, "prompt_len": args.prompt_len,
                      "prompt_tokens_per_s": round(args.batch * args.prompt_len / prompt_s, 1), "prompt_steps": prompt_steps,
                      "decode_tokens_per_s": round(args.batch * args.steps / (ms / 1e3), 1),
                      "decode_ms_per_step": round(ms / args.steps, 4), "steps": args.steps, "decode_graph": config.decode_graph}))
    return 0


def _random_weights(args) -> int:
    from .. import models  # noqa: F401
    from ..registry import architecture_for
    from ..weights.random_init import write_random_model

    if args.config:
        document = json.loads(args.config.read_text())
    else:
        document = {"architectures": ["GPT2LMHeadModel"], **PRESETS[args.preset or "gpt2"]}
    arch = architecture_for(document)
    folder = write_random_model(args.out, arch.config_class.from_dict(document), args.seed, args.dtype)
    print(folder)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        from ..replay import main as replay_main
        return replay_main(argv[1:])
    args = build_parser().parse_args(argv)
    # What the user can put right (a folder, a configuration, weights, a request, a size that a kernel
    # refuses) comes back as one line and status 1; anything else keeps its traceback.
    from ..cache.manager import NoFreeSlot, OutOfPages
    from ..ops import KernelError
    try:
        if args.command == "generate":
            return _generate(args)
        if args.command == "random-weights":
            return _random_weights(args)
        if args.command == "bench":
            return _bench(args)
    except (ValueError, KernelError, OutOfPages, NoFreeSlot, FileNotFoundError) as problem:
        print(f"ayaka_py_b200 {args.command}: {type(problem).__name__}: {problem}", file=sys.stderr)
        return 1
    return 2


if __name__ == "__main__":
    sys.exit(main())
