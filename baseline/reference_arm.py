"""The reference arm of the benchmark: gityuko-hb/ayaka-py itself, unmodified,
through its own public path.

The package is installed under ``baseline/_ref`` by
``baseline/install_reference.py`` and imported from there; nothing of ``ayaka_py_b200`` is
on this path.  What runs is what ``ayaka serve`` builds
(``commands/cli.py:112-171``): ``GPT2Config.from_dict`` ->
``GPT2ForCausalLM(..., backend=...)`` -> ``load_gpt2_weights`` from a
checkpoint written by the reference's own ``write_gpt2_checkpoint`` ->
``ServingRuntime(model, tokenizer_path, pages=..., backend="triton")``.  The
runtime's service owns a thread that steps its engine and sleeps up to a
millisecond between steps (``serving/service.py:610-640``; ``runtime/llm.py``
does the same); stepping that engine from here as well would race with it.  So
the runtime builds a second engine of the same kind with its own builder
(``ServingRuntime._build_tail``, ``runtime/serving.py:787-856``: KV slab, paged
runner, scheduler, worker), which nobody else steps, and that engine is driven
with ``Request`` objects of token ids, ``engine.step()`` after ``engine.step()``
without any sleep: the fastest way the reference's engine can be run.  The
tokenizer folder that ``ServingRuntime`` insists on is a word-level table with
one entry per id; no text is ever encoded.

Timing follows the other arm: prompts are prefilled untimed, W warm-up decode
steps, then K steps between two CUDA events (device time) and K steps by the
wall clock around the engine's own loop, whose every step copies its inputs to
the device and its sampled tokens back (end to end).
"""

from __future__ import annotations

import json
import os
import sys
import tempfile
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


def _write_tokenizer(folder: Path, vocab_size: int) -> None:
    """A tokenizer folder that ``AutoTokenizer.from_pretrained`` loads offline:
    one word per token id."""
    vocab = {f"t{i}": i for i in range(vocab_size)}
    document = {
        "version": "1.0", "truncation": None, "padding": None, "added_tokens": [],
        "normalizer": None, "pre_tokenizer": {"type": "WhitespaceSplit"}, "post_processor": None,
        "decoder": None, "model": {"type": "WordLevel", "vocab": vocab, "unk_token": "t0"},
    }
    (folder / "tokenizer.json").write_text(json.dumps(document))
    (folder / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "t0", "model_max_length": 1 << 20}))


def build_runtime(shape: dict, *, device: str, dtype: str, backend: str, batch: int, max_model_len: int,
                  batch_tokens: int, prefill_chunk: int, decode_graph: bool, workdir: Path, seed: int = 1234):
    """(runtime, config) for a GPT-2 of ``shape`` with the reference's own random checkpoint."""
    if not (REF / "ayaka").is_dir():
        raise RuntimeError(f"the reference is not installed under {REF}")
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    sys.dont_write_bytecode = True          # the installed copy stays as pip left it
    import torch
    from ayaka.models.gpt2 import GPT2Config, GPT2ForCausalLM, load_gpt2_weights, write_gpt2_checkpoint
    from ayaka.runtime.serving import ServingConfig, ServingRuntime

    values = dict(shape, model_type="gpt2", architectures=["GPT2LMHeadModel"], torch_dtype=dtype,
                  tie_word_embeddings=True)
    config = GPT2Config.from_dict(values)
    folder = workdir / "checkpoint"
    folder.mkdir(parents=True, exist_ok=True)
    write_gpt2_checkpoint(folder, config, seed=seed)
    _write_tokenizer(folder, config.vocab_size)
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[dtype]
    layer_backend = "triton" if device.startswith("cuda") else "torch"
    model = GPT2ForCausalLM(config, device=device, dtype=torch_dtype, backend=layer_backend)
    load_gpt2_weights(model, folder)
    model.eval()
    page_size = 16
    pages = batch * (-(-max_model_len // page_size)) + 1
    runtime = ServingRuntime(
        model, folder,
        config=ServingConfig(model="gpt2-bench", structured_outputs=False, decode_graph=decode_graph),
        pages=pages, page_size=page_size, max_requests=max(batch, 2), batch_tokens=batch_tokens,
        prefill_chunk=prefill_chunk, max_model_len=max_model_len, backend=backend, tokenizer_workers=0)
    tail = runtime._build_tail(pages)          # an engine of its own: the service's thread steps only the first one
    return runtime, tail, config


def _close(runtime, tail) -> None:
    try:
        tail.engine.close()
        tail.resources.close()
    finally:
        runtime.close()


def _drive_decode(engine, config, batch: int, prompt_len: int, steps: int, warmup: int, seed: int):
    import numpy as np
    import torch
    from ayaka.request.schema import Request, StopCriteria
    from ayaka.sampling.params import SamplingParams

    rs = np.random.RandomState(seed)
    total_new = 2 * (warmup + steps) + 40
    lifecycles = []
    for i in range(batch):
        prompt = tuple(int(t) for t in rs.randint(0, config.vocab_size, prompt_len))
        lifecycles.append(engine.submit(Request(
            f"ref-b{batch}-{i}", prompt, SamplingParams(temperature=0.0),
            StopCriteria(max_tokens=total_new, ignore_eos=True))))
    cuda = torch.cuda.is_available()

    # prompts (untimed): step until every request has produced its first token
    guard = 0
    while generated_counts(lifecycles) < batch:
        engine.step()
        guard += 1
        if guard > 100000:
            raise RuntimeError("the reference engine made no progress on the prompts")

    def run_steps(n: int) -> None:
        """n decode steps: the engine's loop is stepped until n more tokens per request exist."""
        target = generated_counts(lifecycles) + n * batch
        spins = 0
        while generated_counts(lifecycles) < target:
            engine.step()
            spins += 1
            if spins > 1000 * n + 1000:
                raise RuntimeError("the reference engine stopped producing tokens")

    run_steps(warmup)
    if cuda:
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    run_steps(steps)
    if cuda:
        torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0

    run_steps(warmup)
    if cuda:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        run_steps(steps)
        stop.record()
        torch.cuda.synchronize()
        dev_ms = start.elapsed_time(stop)
    else:
        t0 = time.perf_counter()
        run_steps(steps)
        dev_ms = (time.perf_counter() - t0) * 1e3
    for i in range(batch):
        engine.abort(f"ref-b{batch}-{i}")
    for _ in range(8):
        engine.step()
    return {"tok_s": batch * steps / (dev_ms / 1e3), "ms_per_step": dev_ms / steps,
            "e2e_tok_s": batch * steps / e2e_s}


def generated_counts(lifecycles) -> int:
    """Tokens generated so far by these requests (``RequestLifecycle.output_token_ids``,
    ``request/lifecycle.py``)."""
    return sum(len(lc.output_token_ids) for lc in lifecycles)


def _drive_prefill(engine, config, tokens: int, prompt_len: int, repeats: int, seed: int):
    import numpy as np
    import torch
    from ayaka.request.schema import Request, StopCriteria
    from ayaka.sampling.params import SamplingParams

    rs = np.random.RandomState(seed)
    n = tokens // prompt_len
    times = []
    for rep in range(repeats + 2):
        lifecycles = []
        for i in range(n):
            prompt = tuple(int(t) for t in rs.randint(0, config.vocab_size, prompt_len))
            # prompt_len + 1 must fit the model length: the last position is left to the one new token
            lifecycles.append(engine.submit(Request(f"ref-p{rep}-{i}", prompt[:prompt_len - 1], SamplingParams(temperature=0.0),
                                                    StopCriteria(max_tokens=1, ignore_eos=True))))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        spins = 0
        while generated_counts(lifecycles) < n:
            engine.step()
            spins += 1
            if spins > 10000:
                raise RuntimeError("the reference engine made no progress on the prompts")
        torch.cuda.synchronize()
        if rep >= 2:
            times.append((time.perf_counter() - t0) * 1e3)
        for _ in range(4):
            engine.step()
    ms = sorted(times)[len(times) // 2]
    return {"tokens": n * (prompt_len - 1), "ms": ms}


def run(shape: dict, *, batch: int, prompt_len: int, steps: int, warmup: int, points=(1, 64),
        decode_graph: bool = True, device: str = "cuda", dtype: str = "bfloat16", backend: str = "triton",
        prefill_tokens: int = 2048) -> dict:
    """Measures the reference on ``shape`` and returns the figures of the bench line."""
    import torch

    sizes = sorted({batch, *points})
    out: dict = {"points": {}}
    with tempfile.TemporaryDirectory(prefix="ayaka_ref_") as tmp:
        runtime, tail, config = build_runtime(
            shape, device=device, dtype=dtype, backend=backend, batch=max(sizes),
            max_model_len=shape["n_positions"], batch_tokens=2048, prefill_chunk=2048,
            decode_graph=decode_graph, workdir=Path(tmp))
        try:
            engine = tail.engine
            main = _drive_decode(engine, config, batch, prompt_len, steps, warmup, seed=7)
            out.update(main)
            for b in points:
                if b == batch:
                    out["points"][f"decode_b{b}"] = round(main["tok_s"], 1)
                    continue
                r = _drive_decode(engine, config, b, prompt_len, min(steps, 32), warmup, seed=20 + b)
                out["points"][f"decode_b{b}"] = round(r["tok_s"], 1)
            if prefill_tokens and device.startswith("cuda"):
                p = _drive_prefill(engine, config, prefill_tokens, shape["n_positions"], repeats=3, seed=11)
                out["prefill"] = {"value": round(p["tokens"] / (p["ms"] / 1e3), 1), "tokens": p["tokens"],
                                  "ms": round(p["ms"], 3)}
        finally:
            _close(runtime, tail)
    return out


if __name__ == "__main__":      # a tiny run, on the CPU when there is no GPU: does the arm work at all?
    import torch
    tiny = dict(n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128,
                layer_norm_epsilon=1e-5, activation_function="gelu_new")
    on_gpu = torch.cuda.is_available()
    print(json.dumps(run(tiny, batch=2, prompt_len=16, steps=4, warmup=2, points=(), decode_graph=False,
                         device="cuda" if on_gpu else "cpu", dtype="bfloat16" if on_gpu else "float32",
                         backend="triton" if on_gpu else "reference", prefill_tokens=0)))
