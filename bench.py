"""Decode and prefill throughput of GPT-2 shapes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A step is one decode step of ``--batch`` requests (default 8) of the GPT-2 XL
shape whose prompts of 512 ids are cached; ``value`` is decoded tokens per
second, timed on the device with CUDA events between two synchronisations, over
regions of exactly K steps each, repeated until at least 64 steps are timed
(``config.timed_steps``).  ``e2e`` is the same through the engine's public loop
(scheduler, cache manager, step, sampling) by the wall clock, with the step's
tokens copied in from pinned host memory and the sampled tokens read back every
step.  One JSON line is printed; besides the contract's keys it carries

* ``prefill``: 2 prompts x 1,024 ids in one step, with the fraction of the
  measured bf16 matrix peak;
* ``roofline``: bytes the decode step must read / its time / measured HBM copy
  bandwidth;
* ``points``: decode at 1 and 64 requests; the eager (no CUDA graph) figure and the
  host time per step at ``--batch``; the GPT-2 small shape under continuous
  batching of 256 requests (prompts U[16,1024], outputs U[16,256], all at t = 0,
  2,048-token step budget) through ``LLM.generate``; and the GPT-2 large shape in
  mixed steps of 64 decoding requests at context ~900 beside one 512-token prompt
  portion.

Weights are random (seeded), token ids synthetic.  The inputs of every step
(3 GB of weights at the XL shape) exceed the 126 MB L2, so no flush is needed
between iterations.  ``--impl reference`` runs the unmodified reference from
``baseline/_ref`` (see ``baseline/reference_arm.py``) on the same shape, batch,
prompts and step counts and prints the same line with ``"impl": "reference"``.

``--only prefill|small|large|products`` runs one workload alone (for profiling):
``products`` prints, a JSON line each, the four matrix products of an XL layer
through the engine's dispatcher over row counts beside ``torch.matmul`` on the same
operands.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

XL = dict(n_layer=48, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257, n_positions=1024,
          layer_norm_epsilon=1e-5, activation_function="gelu_new")
SMALL = dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024,
             layer_norm_epsilon=1e-5, activation_function="gelu_new")
LARGE = dict(n_layer=36, n_embd=1280, n_head=20, n_inner=5120, vocab_size=50257, n_positions=1024,
             layer_norm_epsilon=1e-5, activation_function="gelu_new")
PROMPT_LEN = 512
MIN_TIMED_STEPS = 64
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            data = json.load(fh)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi gave no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(self.rows[0][1]), "reasons": reasons, "samples": len(mhz)}


def build_engine(shape: dict, layers: int, *, max_requests: int, kv_pages: int, decode_graph: bool,
                 batch_tokens: int = 2048, prefill_chunk: int = 2048, seed: int = 1):
    from ayaka_py_b200 import EngineConfig, GPT2Config
    from ayaka_py_b200.engine.engine import Engine
    from ayaka_py_b200.engine.loading import random_model

    config = GPT2Config(**{**shape, "n_layer": layers})
    model = random_model(config, seed, "bfloat16", "cuda", generate_on_device=True)
    engine_config = EngineConfig(dtype="bfloat16", kv_pages=kv_pages, page_size=16, max_requests=max_requests,
                                 batch_tokens=batch_tokens, prefill_chunk=prefill_chunk, decode_graph=decode_graph)
    return config, model, Engine(model, engine_config, eos_token_id=None)


def prompts_for(config, batch: int, length: int, seed: int):
    import numpy as np
    rs = np.random.RandomState(seed)
    return [rs.randint(0, config.vocab_size, length).tolist() for _ in range(batch)]


def decode_bytes(model, engine, contexts):
    """Bytes a decode step has to read: every weight once (the position table
    only contributes the rows used) and the cached keys and values of the live
    requests."""
    weights = model.weight_bytes() - model.position.weight.numel() * model.position.weight.element_size()
    return weights + sum(contexts) * engine.cache.bytes_per_token()


def run_decode(engine, config, batch: int, steps: int, warmup: int, seed: int = 7, repeats: int = 1):
    """Prefills ``batch`` prompts of 512 ids through the public loop, then times
    ``repeats`` regions of exactly ``steps`` decode steps two ways.  Returns a dict of measurements."""
    import torch

    from ayaka_py_b200 import Request, SamplingParams, StopCriteria, ops

    # The requests run 2 * (warmup + repeats * steps) decode steps: first the end-to-end loop, then the device-timed one.
    total_new = 2 * (warmup + repeats * steps) + 40
    if PROMPT_LEN + total_new > config.n_positions:
        raise ValueError(f"{repeats} x {steps} timed steps do not fit {config.n_positions} positions")
    for i, prompt in enumerate(prompts_for(config, batch, PROMPT_LEN, seed)):
        engine.submit(Request(f"b{batch}-{i}", prompt, SamplingParams(temperature=0.0),
                              StopCriteria(max_tokens=total_new, ignore_eos=True)))
    while any(s.computed < s.prompt_len for s in engine.scheduler.states.values()):
        engine.step()                                   # prompt portions (untimed)
    assert len(engine.scheduler.running) == batch

    def count_launches():
        return ops.launches + (engine.decode_graphs.launches if engine.decode_graphs else 0)

    # --- end to end: the engine's own step, host tokens in and out every step, by the wall clock
    for _ in range(warmup):
        engine.step()
    e2e_s, launches = 0.0, 0
    host0, steps0 = engine.host_seconds, engine.steps_run
    for _ in range(repeats):
        torch.cuda.synchronize()
        launches0 = count_launches()
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        e2e_s += time.perf_counter() - t0
        launches += count_launches() - launches0
    host_ms = (engine.host_seconds - host0) / max(1, engine.steps_run - steps0) * 1e3
    h2d = engine.decode_graphs.h2d_bytes if (engine.decode_graphs and engine.decode_graphs.h2d_bytes) else engine.runner.h2d_bytes
    d2h = batch * 4

    # --- device-timed: the same steps between two CUDA events
    for _ in range(warmup):
        engine.step()
    contexts = [int(s.computed) for s in engine.scheduler.running]
    dev_ms = 0.0
    for _ in range(repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            engine.step()
        stop.record()
        torch.cuda.synchronize()
        dev_ms += start.elapsed_time(stop)
    timed = repeats * steps
    mean_ctx = [c + (timed - 1) / 2.0 + 1 for c in contexts]
    bytes_step = decode_bytes(engine.model, engine, mean_ctx)
    for rid in list(engine.scheduler.states):
        engine.abort(rid)
    engine.finished.clear()
    engine.cache.assert_clean()
    return {"tok_s": batch * timed / (dev_ms / 1e3), "ms_per_step": dev_ms / timed, "timed_steps": timed,
            "e2e_tok_s": batch * timed / e2e_s, "launches": launches // repeats, "h2d": h2d, "d2h": d2h,
            "bytes_per_step": bytes_step, "mean_context": sum(mean_ctx) / batch, "host_ms_per_step": host_ms}


def run_prefill(engine, config, repeats: int = 3):
    """2 prompts x 1,024 ids in one step of 2,048 tokens, logits at the two last places."""
    import torch

    from ayaka_py_b200.engine.step import StepEntry

    cache, runner = engine.cache, engine.runner
    prompts = prompts_for(config, 2, config.n_positions, 11)
    times = []
    for rep in range(repeats + 2):
        slots = [cache.open(f"p{rep}-{i}") for i in range(2)]
        entries = [StepEntry(s, 0, p, [len(p) - 1]) for s, p in zip(slots, prompts)]
        reservation = cache.reserve([(e.slot, 0, len(e.tokens)) for e in entries])
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        logits = runner.run(entries)
        stop.record()
        torch.cuda.synchronize()
        cache.commit(reservation)
        for s in slots:
            cache.close(s)
        if rep >= 2:
            times.append(start.elapsed_time(stop))
        assert logits.shape == (2, config.vocab_size)
    ms = sorted(times)[len(times) // 2]
    d, inner, L, n, V = config.n_embd, config.inner_size, config.n_layer, config.n_positions, config.vocab_size
    T = 2 * n
    flops = 2.0 * T * L * (3 * d * d + d * d + 2 * d * inner)      # the four products of a layer
    flops += L * 2 * (2.0 * d * n * (n + 1))                        # causal attention, two sequences
    flops += 2.0 * 2 * V * d                                        # the head on two rows
    return {"tokens": T, "ms": ms, "flops": flops}


def run_products(rows=(16, 64, 128, 256, 512, 576, 1024, 2048, 4096)):
    """The four products of an XL layer through ``ops.linear`` (the engine's dispatcher) over row
    counts, each timed as a CUDA graph of 24 products with eight weights in turn (160 MB for the
    widest: larger than L2), beside ``torch.matmul`` on the same operands as a yardstick (a library
    product is nowhere on the engine's path).  Plain bfloat16 out, no bias."""
    import torch

    from ayaka_py_b200 import ops

    dev = "cuda"
    side = torch.cuda.Stream()

    def chain(fn, n=24, reps=6):
        with torch.cuda.stream(side):
            fn()                                   # eager on the stream that is captured next: first-use set-up
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(n):
                fn()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1000 / reps / n

    d, inner = XL["n_embd"], XL["n_inner"]
    out = []
    for name, N, K in (("qkv", 3 * d, d), ("proj", d, d), ("fc", inner, d), ("proj2", d, inner)):
        weights = [(torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(8)]
        for M in rows:
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            turn = [0]

            def ours():
                turn[0] += 1
                ops.linear(x, weights[turn[0] % 8], out=y, out_dtype=torch.bfloat16)

            def library():
                turn[0] += 1
                torch.matmul(x, weights[turn[0] % 8].t(), out=y)

            t_ours, t_lib = chain(ours), chain(library)
            tile, parts = ops.prefill_plan(M, N, K, ops.sm_count()) if M > 64 else (0, 0)
            out.append({"product": name, "rows": M, "us": round(t_ours, 1), "library_us": round(t_lib, 1),
                        "tflops": round(2.0 * M * N * K / t_ours / 1e6), "tile": tile, "k_parts": parts})
    return out


def run_small_continuous(layers: int | None = None, requests: int = 256, seed: int = 5):
    """GPT-2 small shape, 256 requests at t = 0 through ``LLM.generate``: prompts U[16,1024],
    outputs U[16,256] (cut where prompt + output would pass the model's 1,024 positions),
    chunked prefill under a 2,048-token step budget, greedy.  The cache holds 6,144 pages of
    16 tokens: less than the 256 requests need at their longest (about 7,500), so pages run
    out, requests are preempted and recompute, and pages come back."""
    import numpy as np
    import torch

    from ayaka_py_b200 import LLM, GPT2Config, SamplingParams, StopCriteria

    config = GPT2Config(**{**SMALL, "n_layer": layers or SMALL["n_layer"]})
    pages = 6144
    llm = LLM(config, seed=3, dtype="bfloat16", kv_pages=pages, page_size=16, max_requests=requests,
              batch_tokens=2048, prefill_chunk=2048, decode_graph=True)
    rs = np.random.RandomState(seed)
    prompts, stops = [], []
    for _ in range(requests):
        n = int(rs.randint(16, 1025))
        out = int(rs.randint(16, 257))
        n = min(n, config.n_positions - 16)
        out = min(out, config.n_positions - n)
        prompts.append(rs.randint(0, config.vocab_size, n).tolist())
        stops.append(StopCriteria(max_tokens=out, ignore_eos=True))
    # once untimed (the decode graphs of every batch bucket are captured on the way), then timed
    warm = llm.generate(prompts, SamplingParams(temperature=0.0), stops)
    assert len(warm) == requests
    engine = llm.engine
    steps0 = engine.steps_run
    stats0 = engine.scheduler.stats
    base = (stats0.steps, stats0.preemptions, stats0.prefill_tokens, stats0.decode_tokens)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    results = llm.generate(prompts, SamplingParams(temperature=0.0), stops)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    engine.cache.assert_clean()
    generated = sum(len(r.token_ids) for r in results)
    assert all(len(r.token_ids) == s.max_tokens for r, s in zip(results, stops))
    prompt_tokens = sum(len(p) for p in prompts)
    stats = engine.scheduler.stats
    pool = engine.cache.stats()["groups"]
    high = max(g["high_water"] for g in pool.values())
    return {"total_tok_s": (prompt_tokens + generated) / seconds, "output_tok_s": generated / seconds,
            "seconds": seconds, "steps": stats.steps - base[0], "preemptions": stats.preemptions - base[1],
            "computed_prompt_tokens": stats.prefill_tokens - base[2], "prompt_tokens": prompt_tokens,
            "generated": generated, "page_high_water": high, "pages": pages - 1,
            "engine_steps": engine.steps_run - steps0}


def run_large_mixed(layers: int | None = None, steps: int = 48, warmup: int = 6, decoders: int = 64,
                    context: int = 900, portion: int = 512, seed: int = 9):
    """GPT-2 large shape: every step holds ``decoders`` single decoded tokens at context ~``context``
    and one ``portion``-token portion of a fresh prompt, through the engine's own loop (scheduler,
    sampling at temperature 1 with seeds, tokens to the host every step)."""
    import numpy as np
    import torch

    from ayaka_py_b200 import Request, SamplingParams, StopCriteria

    shape = {**LARGE, "n_layer": layers or LARGE["n_layer"]}
    pages = (decoders + 2) * (LARGE["n_positions"] // 16) + 1
    config, model, engine = build_engine(shape, shape["n_layer"], max_requests=decoders + 2, kv_pages=pages,
                                         decode_graph=False, batch_tokens=decoders + portion, prefill_chunk=portion)
    rs = np.random.RandomState(seed)
    room = config.n_positions - context
    assert warmup + steps + 2 <= room, "the decoders reach the model's last position before the timed steps end"
    for i in range(decoders):
        engine.submit(Request(f"d{i}", rs.randint(0, config.vocab_size, context).tolist(),
                              SamplingParams(temperature=1.0, seed=1000 + i), StopCriteria(max_tokens=room, ignore_eos=True)))
    # prompts of the decoders, untimed, in whatever steps the scheduler cuts
    engine.scheduler.batch_tokens, engine.scheduler.prefill_chunk = 2048, 2048
    while any(s.computed < s.prompt_len for s in engine.scheduler.states.values()):
        engine.step()
    engine.scheduler.batch_tokens, engine.scheduler.prefill_chunk = decoders + portion, portion
    feeders = 0

    def feed():
        # Prompts of two portions; one token each, so a feeder leaves when its prompt is done.
        nonlocal feeders
        while len(engine.scheduler.waiting) < 2:
            engine.submit(Request(f"f{feeders}", rs.randint(0, config.vocab_size, 2 * portion - 1).tolist(),
                                  SamplingParams(temperature=1.0, seed=feeders), StopCriteria(max_tokens=1, ignore_eos=True)))
            feeders += 1

    shapes = []

    def one_step():
        feed()
        before = engine.runner.rows_run
        engine.step()
        shapes.append(engine.runner.rows_run - before)

    for _ in range(warmup):
        one_step()
    shapes.clear()
    contexts = [int(s.computed) for s in engine.scheduler.running if s.remaining <= 1][:decoders]
    host0 = engine.host_seconds
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        one_step()
    stop.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = start.elapsed_time(stop) / steps
    rows = sum(shapes) / len(shapes)
    mean_ctx = sum(contexts) / max(1, len(contexts)) + steps / 2.0
    weights = model.weight_bytes() - model.position.weight.numel() * model.position.weight.element_size()
    kv_bytes = decoders * mean_ctx * engine.cache.bytes_per_token()
    d, inner, L = config.n_embd, config.inner_size, config.n_layer
    flops = 2.0 * rows * L * (4 * d * d + 2 * d * inner)
    for rid in list(engine.scheduler.states):
        engine.abort(rid)
    engine.finished.clear()
    engine.cache.assert_clean()
    return {"ms_per_step": ms, "rows_per_step": rows, "tok_s": rows / (ms / 1e3), "e2e_ms_per_step": wall / steps * 1e3,
            "host_ms_per_step": (engine.host_seconds - host0) / steps * 1e3,
            "gbs": (weights + kv_bytes) / (ms / 1e3) / 1e9, "tflops": flops / (ms / 1e3) / 1e12,
            "mean_context": mean_ctx, "n_layer": L}


def reference_line(args) -> dict:
    """The reference arm: same shape, batch, prompt length and step counts, the reference's own engine."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm
    except Exception as exc:           # noqa: BLE001
        return {"impl": "reference", "unavailable": f"baseline/reference_arm.py cannot be imported: {exc!r}"[:300]}
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "ayaka")):
        return {"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref "
                "(python baseline/install_reference.py <checkout of the reference>)"}
    shape = {**XL, "n_layer": args.layers}
    repeats = -(-MIN_TIMED_STEPS // args.steps)
    sampler = ClockSampler()
    sampler.start()
    try:
        r = reference_arm.run(shape, batch=args.batch, prompt_len=PROMPT_LEN, steps=args.steps * repeats,
                              warmup=args.warmup, points=() if args.no_points else (1, 64), decode_graph=False,
                              prefill_tokens=0 if args.no_points else 2048)
    except BaseException as exc:       # noqa: BLE001
        text = " ".join(f"{type(exc).__name__}: {exc}".split())
        return {"impl": "reference", "unavailable": f"the reference raised on this box: {text}"[:400]}
    finally:
        sampler.stop()
    line = {"metric": "decode tokens per second, GPT-2 XL shape", "value": round(r["tok_s"], 1), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(r["ms_per_step"], 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "reference",
            "config": {"model": "gpt2-xl shape, the reference's own random checkpoint", "global_batch": args.batch,
                       "seq_len": XL["n_positions"], "parallelism": "single GPU", "n_layer": args.layers,
                       "n_layer_of_shape": XL["n_layer"], "prompt_len": PROMPT_LEN, "page_size": 16,
                       "timed_steps": args.steps * repeats, "backend": "triton", "decode_graph": False,
                       "driver": "ServingRuntime's engine, engine.step() in a loop"},
            "e2e": {"value": round(r["e2e_tok_s"], 1), "unit": "tokens/s"},
            "clocks": sampler.summary(), "points": r.get("points", {})}
    if "prefill" in r:
        line["prefill"] = r["prefill"]
    return line


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=XL["n_layer"], help="fewer layers than the XL shape's 48 (sizes stay)")
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--no-graph", action="store_true", help="run decode steps eagerly")
    parser.add_argument("--no-points", action="store_true", help="only the decode steps at --batch")
    parser.add_argument("--only", default=None, choices=("prefill", "small", "large", "products"),
                        help="run one workload alone and print its numbers (for profiling): the 2,048-token prefill "
                             "step, the small shape's continuous batching, the large shape's mixed steps, or the four "
                             "products of an XL layer over row counts beside the library's matmul")
    args = parser.parse_args()

    if args.gpus != 1:
        print("bench.py measures a single-GPU engine: --gpus must be 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.steps < 1:
        args.steps = 1
    if args.impl == "reference":
        print(json.dumps(reference_line(args)))
        return 0

    import torch

    from ayaka_py_b200 import ops

    pk = peaks()
    graph = not args.no_graph
    if args.only == "products":
        for row in run_products():
            print(json.dumps(row))
        return 0
    if args.only == "small":
        print(json.dumps({"small_continuous": run_small_continuous(None if args.layers == XL["n_layer"] else args.layers)}))
        return 0
    if args.only == "large":
        print(json.dumps({"large_mixed": run_large_mixed(None if args.layers == XL["n_layer"] else args.layers,
                                                         steps=args.steps, warmup=args.warmup)}))
        return 0
    sizes = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    config, model, engine = build_engine(XL, args.layers, max_requests=max(max(sizes), 2),
                                         kv_pages=max(sizes) * (XL["n_positions"] // 16) + 1, decode_graph=graph)
    if args.only == "prefill":
        p = run_prefill(engine, config, repeats=max(1, args.steps))
        print(json.dumps({"prefill": {"value": round(p["tokens"] / (p["ms"] / 1e3), 1), "tokens": p["tokens"],
                                      "ms": round(p["ms"], 3), "n_layer": args.layers,
                                      "frac": round(p["flops"] / (p["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0
    repeats = -(-MIN_TIMED_STEPS // args.steps)
    sampler = ClockSampler()
    sampler.start()
    main_run = run_decode(engine, config, args.batch, args.steps, args.warmup, repeats=repeats)
    sampler.stop()
    clocks = sampler.summary()

    points, prefill = {}, None
    if not args.no_points:
        for b in (1, 64):
            r = main_run if b == args.batch else run_decode(engine, config, b, 32, args.warmup, seed=20 + b, repeats=2)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
        p = run_prefill(engine, config)
        prefill = {"value": round(p["tokens"] / (p["ms"] / 1e3), 1), "tokens": p["tokens"], "ms": round(p["ms"], 3),
                   "frac": round(p["flops"] / (p["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        points[f"host_ms_per_step_b{args.batch}"] = round(main_run["host_ms_per_step"], 4)
        if graph:
            # the same decode steps without CUDA graphs: every kernel launched from Python
            engine.decode_graphs = None
            eager = run_decode(engine, config, args.batch, 32, args.warmup, seed=31, repeats=2)
            points[f"decode_b{args.batch}_eager"] = round(eager["tok_s"], 1)
            points[f"host_ms_per_step_b{args.batch}_eager"] = round(eager["host_ms_per_step"], 4)
        del engine, model
        torch.cuda.empty_cache()
        small = run_small_continuous()
        points.update({"small_cb_total_tok_s": round(small["total_tok_s"], 1), "small_cb_output_tok_s": round(small["output_tok_s"], 1),
                       "small_cb_steps": small["steps"], "small_cb_preemptions": small["preemptions"],
                       "small_cb_page_high_water": small["page_high_water"], "small_cb_seconds": round(small["seconds"], 3)})
        torch.cuda.empty_cache()
        large = run_large_mixed()
        points.update({"large_mixed_ms_per_step": round(large["ms_per_step"], 4), "large_mixed_tok_s": round(large["tok_s"], 1),
                       "large_mixed_rows_per_step": round(large["rows_per_step"], 1),
                       "large_mixed_host_ms_per_step": round(large["host_ms_per_step"], 4),
                       "large_mixed_tflops": round(large["tflops"], 1), "large_mixed_gbs": round(large["gbs"], 1)})

    achieved = main_run["bytes_per_step"] / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tokens per second, GPT-2 XL shape", "value": round(main_run["tok_s"], 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "gpt2-xl shape, random weights", "global_batch": args.batch, "seq_len": config.n_positions,
                   "parallelism": "single GPU", "n_layer": args.layers, "n_layer_of_shape": XL["n_layer"],
                   "n_embd": config.n_embd, "n_head": config.n_head, "n_inner": config.inner_size,
                   "vocab_size": config.vocab_size, "prompt_len": PROMPT_LEN,
                   "mean_context": round(main_run["mean_context"], 1), "page_size": 16,
                   "decode_graph": graph, "timed_steps": main_run["timed_steps"],
                   "l2": "inputs larger than L2 (weights 3 GB)", "peaks": pk["source"]},
        "e2e": {"value": round(main_run["e2e_tok_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(main_run["h2d"]), "d2h_bytes_per_step": int(main_run["d2h"])},
        "gpu_launches": int(main_run["launches"]),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if prefill is not None:
        line["prefill"] = prefill
        line["points"] = points
    if ops.tc_error():
        line["error"] = f"a tensor-core kernel's wait ran out (code {ops.tc_error()})"
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
