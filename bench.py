"""Decode and prefill throughput of the GPT-2 XL shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A step is one decode step of ``--batch`` requests (default 8) whose prompts of
512 ids are cached; ``value`` is decoded tokens per second over exactly K steps,
timed on the device with CUDA events between two synchronisations.  ``e2e`` is
the same through the engine's public loop (scheduler, cache manager, step,
sampling) with the step's tokens copied in from pinned host memory and the
sampled tokens read back every step.  One JSON line is printed; besides the
contract's keys it carries ``prefill`` (2 prompts x 1,024 ids in one step),
``roofline`` (bytes the decode step must read / its time / measured HBM copy
bandwidth) and ``points`` (decode at batch 1 and 64).  Weights are random
(seeded), token ids synthetic.  Inputs of every step (3 GB of weights) exceed
the 126 MB L2, so no flush is needed between iterations.
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
PROMPT_LEN = 512
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
                                          "--format=csv,noheader,nounits", "-lms", "100"],
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


def build_engine(layers: int, batch: int, decode_graph: bool, seed: int = 1):
    import torch

    from ayaka_py_b200 import EngineConfig, GPT2Config
    from ayaka_py_b200.engine.engine import Engine
    from ayaka_py_b200.engine.loading import random_model

    config = GPT2Config(**{**XL, "n_layer": layers})
    model = random_model(config, seed, "bfloat16", "cuda", generate_on_device=True)
    pages = batch * (config.n_positions // 16) + 1
    engine_config = EngineConfig(dtype="bfloat16", kv_pages=pages, page_size=16, max_requests=max(batch, 2),
                                 batch_tokens=2048, prefill_chunk=2048, decode_graph=decode_graph)
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


def run_decode(engine, config, batch: int, steps: int, warmup: int, seed: int = 7):
    """Prefills ``batch`` prompts of 512 ids through the public loop, then times
    decode steps two ways.  Returns a dict of measurements."""
    import torch

    from ayaka_py_b200 import Request, SamplingParams, StopCriteria, ops

    # The requests run 2 * (warmup + steps) decode steps: first the end-to-end loop, then the device-timed one.
    total_new = 2 * (warmup + steps) + 40
    for i, prompt in enumerate(prompts_for(config, batch, PROMPT_LEN, seed)):
        engine.submit(Request(f"b{batch}-{i}", prompt, SamplingParams(temperature=0.0),
                              StopCriteria(max_tokens=total_new, ignore_eos=True)))
    while any(s.computed < s.prompt_len for s in engine.scheduler.states.values()):
        engine.step()                                   # prompt portions (untimed)
    assert len(engine.scheduler.running) == batch

    # --- end to end: the engine's own step, host tokens in and out every step
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    launches0 = ops.launches + (engine.decode_graphs.launches if engine.decode_graphs else 0)
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    launches = ops.launches + (engine.decode_graphs.launches if engine.decode_graphs else 0) - launches0
    h2d = engine.decode_graphs.h2d_bytes if (engine.decode_graphs and engine.decode_graphs.h2d_bytes) else engine.runner.h2d_bytes
    d2h = batch * 4

    # --- device-timed: the same steps between two CUDA events
    for _ in range(warmup):
        engine.step()
    contexts = [int(s.computed) for s in engine.scheduler.running]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        engine.step()
    stop.record()
    torch.cuda.synchronize()
    dev_ms = start.elapsed_time(stop)
    mean_ctx = [c + (steps - 1) / 2.0 + 1 for c in contexts]
    bytes_step = decode_bytes(engine.model, engine, mean_ctx)
    for rid in list(engine.scheduler.states):
        engine.abort(rid)
    engine.finished.clear()
    engine.cache.assert_clean()
    return {"tok_s": batch * steps / (dev_ms / 1e3), "ms_per_step": dev_ms / steps,
            "e2e_tok_s": batch * steps / e2e_s, "launches": launches, "h2d": h2d, "d2h": d2h,
            "bytes_per_step": bytes_step, "mean_context": sum(mean_ctx) / batch}


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


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=XL["n_layer"], help="fewer layers than the XL shape's 48 (sizes stay)")
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--no-graph", action="store_true", help="run decode steps eagerly")
    parser.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64 and the prefill")
    parser.add_argument("--prefill-only", action="store_true",
                        help="run only the 2,048-token prefill step and print its numbers (for profiling)")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip refuses the offline install: ayaka requires Python >=3.13,<3.14, this image has 3.12"}))
        return 0
    if args.gpus != 1:
        print("bench.py measures a single-GPU engine: --gpus must be 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from ayaka_py_b200 import ops

    pk = peaks()
    graph = not args.no_graph
    sizes = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    config, model, engine = build_engine(args.layers, max(sizes), graph)
    if args.prefill_only:
        p = run_prefill(engine, config, repeats=max(1, args.steps))
        print(json.dumps({"prefill": {"value": round(p["tokens"] / (p["ms"] / 1e3), 1), "tokens": p["tokens"],
                                      "ms": round(p["ms"], 3), "n_layer": args.layers,
                                      "frac": round(p["flops"] / (p["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0
    sampler = ClockSampler()
    sampler.start()
    main_run = run_decode(engine, config, args.batch, args.steps, args.warmup)
    sampler.stop()
    clocks = sampler.summary()

    points, prefill = {}, None
    if not args.no_points:
        for b in (1, 64):
            r = main_run if b == args.batch else run_decode(engine, config, b, min(args.steps, 32), args.warmup, seed=20 + b)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
        p = run_prefill(engine, config)
        prefill = {"value": round(p["tokens"] / (p["ms"] / 1e3), 1), "tokens": p["tokens"], "ms": round(p["ms"], 3),
                   "frac": round(p["flops"] / (p["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

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
                   "decode_graph": graph, "l2": "inputs larger than L2 (weights 3 GB)", "peaks": pk["source"]},
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
