"""Generation through the Python entry point and the command line, compared
with the plain implementation."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_gpt2
import tiny_models

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_greedy_matches_plain_tiny_a(model_folders):
    from ayaka_py_b200 import LLM, SamplingParams, StopCriteria
    folder, cfg, weights = model_folders["A"]
    prompts = tiny_models.prompts(cfg, [5, 17, 40], seed=21)
    llm = LLM(folder, dtype="float32", page_size=16, kv_pages=64, batch_tokens=64, prefill_chunk=32)
    out = llm.generate(prompts, SamplingParams(temperature=0.0), StopCriteria(max_tokens=16, ignore_eos=True))
    for p, r in zip(prompts, out):
        assert r.finish_reason == "length"
        assert r.token_ids == plain_gpt2.greedy_generate(cfg, weights, p, 16)
    llm.engine.cache.assert_clean()


def test_greedy_bfloat16_stays_within_rounding_of_the_best_token(model_folders):
    from ayaka_py_b200 import LLM, SamplingParams, StopCriteria
    folder, cfg, weights = model_folders["A"]
    prompts = tiny_models.prompts(cfg, [5, 17, 40], seed=21)
    llm = LLM(folder, dtype="bfloat16", page_size=16, kv_pages=64, batch_tokens=64, prefill_chunk=32)
    out = llm.generate(prompts, SamplingParams(temperature=0.0), StopCriteria(max_tokens=16, ignore_eos=True))
    for p, r in zip(prompts, out):
        logits = plain_gpt2.forward(cfg, weights, p + r.token_ids)
        slack = 2 * 0.02 * float(np.abs(logits).max())
        for i, token in enumerate(r.token_ids):
            row = logits[len(p) - 1 + i]
            assert row[token] >= row.max() - slack


def test_tiny_b_workload_chunked_mixed_temperature(model_folders):
    """5 prompts of 1/9/33/64/120 ids, prefill chunk 24 mixed with decodes, page
    size 8, temperature 0.8 with a fixed seed, 24 new tokens each: every token
    must be the one the sampling twin draws from the plain model's logits."""
    from ayaka_py_b200 import LLM, SamplingParams, StopCriteria
    folder, cfg, weights = model_folders["B"]
    prompts = tiny_models.prompts(cfg, [1, 9, 33, 64, 120], seed=22)
    llm = LLM(folder, dtype="float32", page_size=8, kv_pages=80, batch_tokens=64, prefill_chunk=24)
    params = [SamplingParams(temperature=0.8, seed=1000 + i) for i in range(5)]
    out = llm.generate(prompts, params, StopCriteria(max_tokens=24, ignore_eos=True))
    for i, (p, r) in enumerate(zip(prompts, out)):
        assert len(r.token_ids) == 24
        logits = plain_gpt2.forward(cfg, weights, p + r.token_ids)
        for j, token in enumerate(r.token_ids):
            probs = plain_gpt2.filtered_probabilities(logits[len(p) - 1 + j], 0.8)
            cum = np.cumsum(probs)
            u = plain_gpt2.philox_uniform(1000 + i, j)
            lo = cum[token - 1] if token > 0 else 0.0
            assert lo - 1e-4 <= u <= cum[token] + 1e-4, (i, j, token)
    stats = llm.engine.scheduler.stats
    assert stats.prefill_tokens >= sum(len(p) for p in prompts) and stats.decode_tokens > 0
    # the same requests again, each alone: a request's tokens do not depend on its neighbours
    alone = LLM(folder, dtype="float32", page_size=8, kv_pages=80, batch_tokens=256, prefill_chunk=256)
    for i in (1, 4):
        again = alone.generate([prompts[i]], params[i], StopCriteria(max_tokens=24, ignore_eos=True))[0]
        assert again.token_ids == out[i].token_ids


def test_few_pages_preempt_and_recompute_same_tokens(model_folders):
    from ayaka_py_b200 import LLM, SamplingParams, StopCriteria
    folder, cfg, weights = model_folders["A"]
    prompts = tiny_models.prompts(cfg, [30, 28, 33, 25], seed=23)
    stop = StopCriteria(max_tokens=30, ignore_eos=True)
    roomy = LLM(folder, dtype="float32", page_size=16, kv_pages=64, batch_tokens=64, prefill_chunk=32)
    want = [r.token_ids for r in roomy.generate(prompts, SamplingParams(temperature=0.0), stop)]
    tight = LLM(folder, dtype="float32", page_size=16, kv_pages=11, batch_tokens=64, prefill_chunk=32)   # 160 tokens
    got = tight.generate(prompts, SamplingParams(temperature=0.0), stop)
    assert [r.token_ids for r in got] == want
    assert tight.engine.scheduler.stats.preemptions > 0 and any(r.preemptions for r in got)
    tight.engine.cache.assert_clean()


def test_few_pages_preempt_and_recompute_in_bfloat16_with_decode_graphs(model_folders):
    """The same pressure in bfloat16 with pure-decode steps replayed from CUDA graphs: requests are
    preempted, recompute their prompt and what they had generated through the prompt kernels, and go
    on decoding from graphs.  Every token is, by the plain model's logits, within bfloat16 rounding of
    the best one, and all of them arrive."""
    from ayaka_py_b200 import LLM, SamplingParams, StopCriteria
    folder, cfg, weights = model_folders["D"]
    prompts = tiny_models.prompts(cfg, [150, 140, 165, 120], seed=29)
    stop = StopCriteria(max_tokens=40, ignore_eos=True)
    tight = LLM(folder, dtype="bfloat16", page_size=16, kv_pages=34, batch_tokens=256, prefill_chunk=128,
                max_requests=4, decode_graph=True)                       # 528 tokens for up to 820
    got = tight.generate(prompts, SamplingParams(temperature=0.0), stop)
    assert tight.engine.scheduler.stats.preemptions > 0 and any(r.preemptions for r in got)
    assert tight.engine.decode_graphs.launches > 0
    for p, r in zip(prompts, got):
        assert len(r.token_ids) == 40 and r.finish_reason == "length"
        logits = plain_gpt2.forward(cfg, weights, p + r.token_ids)
        slack = 2 * 0.02 * float(np.abs(logits).max())
        for i, token in enumerate(r.token_ids):
            row = logits[len(p) - 1 + i]
            assert row[token] >= row.max() - slack, (i, token)
    tight.engine.cache.assert_clean()


def test_filters_keep_the_twins_support(model_folders):
    from ayaka_py_b200 import LLM, SamplingParams, StopCriteria
    folder, cfg, weights = model_folders["A"]
    prompts = tiny_models.prompts(cfg, [12, 20], seed=24)
    llm = LLM(folder, dtype="float32", page_size=16, kv_pages=64)
    params = [SamplingParams(temperature=1.5, top_k=5, seed=3), SamplingParams(temperature=1.2, top_p=0.5, min_p=0.05, seed=4)]
    out = llm.generate(prompts, params, StopCriteria(max_tokens=20, ignore_eos=True))
    for p, sp, r in zip(prompts, params, out):
        logits = plain_gpt2.forward(cfg, weights, p + r.token_ids)
        for j, token in enumerate(r.token_ids):
            probs = plain_gpt2.filtered_probabilities(logits[len(p) - 1 + j], sp.temperature, sp.top_k, sp.top_p, sp.min_p)
            assert probs[token] > 0, (sp, j, token)


def test_command_line(model_folders, tmp_path):
    folder, cfg, weights = model_folders["A"]
    prompt = tiny_models.prompts(cfg, [9], seed=25)[0]
    proc = subprocess.run(
        [sys.executable, "-m", "ayaka_py_b200", "generate", str(folder), "--dtype", "float32", "--kv-pages", "32",
         "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "8", "--temperature", "0", "--ignore-eos"],
        cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    record = json.loads(proc.stdout.strip().splitlines()[-1])
    assert record["token_ids"] == plain_gpt2.greedy_generate(cfg, weights, prompt, 8)
    assert record["finish_reason"] == "length"


def test_command_line_bench(model_folders):
    folder, cfg, _ = model_folders["D"]
    proc = subprocess.run(
        [sys.executable, "-m", "ayaka_py_b200", "bench", str(folder), "--batch", "3", "--prompt-len", "40", "--steps", "6",
         "--warmup", "3", "--kv-pages", "8"], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    record = json.loads(proc.stdout.strip().splitlines()[-1])
    assert record["batch"] == 3 and record["steps"] == 6 and record["decode_tokens_per_s"] > 0 and record["prompt_tokens_per_s"] > 0


def test_smoke_entry():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__
    __graft_entry__.smoke()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_give_the_same_tokens(model_folders, dtype):
    """Pure-decode steps replayed from CUDA graphs (padded to a bucket) against the eager engine."""
    from ayaka_py_b200 import LLM, SamplingParams, StopCriteria
    folder, cfg, weights = model_folders["B"]
    prompts = tiny_models.prompts(cfg, [3, 20, 41], seed=26)
    stop = [StopCriteria(max_tokens=n, ignore_eos=True) for n in (30, 12, 21)]     # the batch shrinks: 3 -> 2 -> 1
    params = [SamplingParams(temperature=0.0), SamplingParams(temperature=0.7, seed=5), SamplingParams(temperature=0.0)]
    eager = LLM(folder, dtype=dtype, page_size=8, kv_pages=64, batch_tokens=64, prefill_chunk=32, decode_graph=False)
    graphs = LLM(folder, dtype=dtype, page_size=8, kv_pages=64, batch_tokens=64, prefill_chunk=32, decode_graph=True)
    want = [r.token_ids for r in eager.generate(prompts, params, stop)]
    got = [r.token_ids for r in graphs.generate(prompts, params, stop)]
    assert got == want
    assert sorted(graphs.engine.decode_graphs.graphs) == [1, 2, 4]
    assert graphs.engine.decode_graphs.launches > 0
    graphs.engine.cache.assert_clean()


def test_programmatic_dependent_launch_on_and_off_agree(model_folders):
    from ayaka_py_b200 import LLM, SamplingParams, StopCriteria, ops
    folder, cfg, weights = model_folders["A"]
    prompts = tiny_models.prompts(cfg, [11, 30], seed=27)
    stop = StopCriteria(max_tokens=12, ignore_eos=True)
    out = {}
    try:
        for on in (False, True):
            ops.set_pdl(on)
            llm = LLM(folder, dtype="bfloat16", page_size=16, kv_pages=32, decode_graph=on)
            out[on] = [r.token_ids for r in llm.generate(prompts, SamplingParams(temperature=0.0), stop)]
    finally:
        ops.set_pdl(True)
    assert out[False] == out[True]


@pytest.mark.parametrize("graph", [False, True], ids=["eager", "graphs"])
def test_lookahead_gives_the_same_tokens(model_folders, graph):
    """The next decode step launched before this step's tokens are on the host
    (its tokens copied from the sampler's output on the device) against the
    plain loop: same tokens and finish reasons with greedy and seeded sampling,
    requests that stop on a stop id in the middle of a run, and a late arrival."""
    from ayaka_py_b200 import EngineConfig, Request, SamplingParams, StopCriteria
    from ayaka_py_b200.engine.engine import Engine
    from ayaka_py_b200.engine.loading import load_model
    folder, cfg, weights = model_folders["B"]
    prompts = tiny_models.prompts(cfg, [5, 17, 33, 9], seed=31)
    params = [SamplingParams(temperature=0.0), SamplingParams(temperature=0.9, seed=11, top_k=40),
              SamplingParams(temperature=0.0), SamplingParams(temperature=0.8, seed=3)]
    _, model = load_model(folder, "bfloat16", "cuda")

    def run(lookahead, stops):
        config = EngineConfig(dtype="bfloat16", page_size=8, kv_pages=64, batch_tokens=64, prefill_chunk=32,
                              decode_graph=graph, lookahead=lookahead)
        engine = Engine(model, config, eos_token_id=None)
        for i in range(3):
            engine.submit(Request(f"r{i}", prompts[i], params[i], stops[i]))
        steps, ahead = 0, 0
        while engine.has_work():
            if steps == 12:
                engine.submit(Request("r3", prompts[3], params[3], stops[3]))
            engine.step()
            ahead += engine._inflight is not None
            steps += 1
        engine.cache.assert_clean()
        out, engine.finished = engine.finished, {}
        return {k: (v.token_ids, v.finish_reason) for k, v in out.items()}, ahead

    free = [StopCriteria(max_tokens=n, ignore_eos=True) for n in (40, 25, 31, 18)]
    base, _ = run(False, free)
    # stop ids taken from the middle of what two of the requests generate
    stops = [StopCriteria(max_tokens=40, stop_token_ids=(base["r0"][0][13],)), free[1],
             StopCriteria(max_tokens=31, stop_token_ids=(base["r2"][0][20],), min_tokens=4), free[3]]
    want, none_ahead = run(False, stops)
    got, some_ahead = run(True, stops)
    assert none_ahead == 0 and some_ahead > 10
    assert got == want
    assert want["r0"][1] == "stop" and len(want["r0"][0]) <= 14


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lookahead_past_prompt_portions_and_page_pressure(model_folders, dtype):
    """Steps planned ahead that hold prompt portions and newly admitted requests beside the decoding ones,
    in a pool so small that pages run out (the step is then planned when its tokens are known, and requests
    are preempted and recompute): the same tokens as the plain loop, and the same steps."""
    from ayaka_py_b200 import EngineConfig, Request, SamplingParams, StopCriteria
    from ayaka_py_b200.engine.engine import Engine
    from ayaka_py_b200.engine.loading import load_model
    folder, cfg, weights = model_folders["B"]
    lens, news, arrive = [70, 45, 60, 30, 52], [22, 30, 12, 26, 9], [0, 0, 3, 9, 20]
    prompts = tiny_models.prompts(cfg, lens, seed=37)
    _, model = load_model(folder, dtype, "cuda")

    def run(lookahead):
        config = EngineConfig(dtype=dtype, page_size=8, kv_pages=27, batch_tokens=24, prefill_chunk=16, max_requests=4,
                              decode_graph=True, lookahead=lookahead)
        engine = Engine(model, config, eos_token_id=None)
        step, nxt, ahead, kinds = 0, 0, 0, set()
        while engine.has_work() or nxt < len(lens):
            while nxt < len(lens) and arrive[nxt] <= step:
                engine.submit(Request(f"r{nxt}", prompts[nxt], SamplingParams(temperature=0.0),
                                      StopCriteria(max_tokens=news[nxt], ignore_eos=True)))
                nxt += 1
            if engine.has_work():
                engine.step()
                if engine._inflight is not None:
                    ahead += 1
                    plan = engine._inflight.plan
                    kinds.add(("decode" if plan.decode_only else "mixed", bool(plan.token_rows)))
            step += 1
        engine.cache.assert_clean()
        stats = engine.scheduler.stats
        return [engine.finished[f"r{i}"].token_ids for i in range(len(lens))], ahead, kinds, (stats.steps, stats.preemptions)

    want, none_ahead, _, plain_stats = run(False)
    got, some_ahead, kinds, ahead_stats = run(True)
    assert none_ahead == 0 and some_ahead > 20
    assert ("mixed", True) in kinds and ("decode", True) in kinds          # portions beside tokens on their way, and pure decoding
    assert plain_stats[1] > 0 and ahead_stats == plain_stats              # pages ran out, and both loops took the same steps
    assert got == want
    for i in (0, 3):
        assert got[i] == plain_gpt2.greedy_generate(cfg, weights, prompts[i], news[i]) or dtype == "bfloat16"


@pytest.mark.parametrize("graph", [False, True], ids=["eager", "graphs"])
def test_stop_ids_are_banned_until_min_tokens(model_folders, graph):
    """``request/stream.py:130-163``: before ``min_tokens`` the stop ids are masked out of the
    logits (the request produces the best token that is not banned), afterwards the first stop
    id ends it.  Greedy, so every token can be checked against the plain model's logits."""
    from ayaka_py_b200 import LLM, SamplingParams, StopCriteria
    folder, cfg, weights = model_folders["A"]
    prompt = tiny_models.prompts(cfg, [14], seed=41)[0]
    free = plain_gpt2.greedy_generate(cfg, weights, prompt, 12)
    banned = (free[0], free[2], free[5])
    llm = LLM(folder, dtype="float32", page_size=16, kv_pages=32, decode_graph=graph)
    out = llm.generate([prompt, prompt], SamplingParams(temperature=0.0),
                       [StopCriteria(max_tokens=12, min_tokens=7, stop_token_ids=banned),
                        StopCriteria(max_tokens=12, min_tokens=0, stop_token_ids=(free[2],))])
    got = out[0].token_ids
    assert not set(got[:7]) & set(banned) and got[0] != free[0]
    logits = plain_gpt2.forward(cfg, weights, prompt + got)
    for j, token in enumerate(got):
        row = logits[len(prompt) - 1 + j].copy()
        if j < 7:
            row[list(banned)] = -np.inf
        assert token == int(row.argmax()), (j, token)
    assert out[0].finish_reason in ("stop", "length") and (out[0].finish_reason == "length" or got[-1] in banned)
    first = free.index(free[2])                           # no min_tokens: stops at the id's first appearance
    assert out[1].token_ids == free[:first + 1] and out[1].finish_reason == "stop"
    llm.engine.cache.assert_clean()


def test_abort_with_a_step_in_flight(model_folders):
    """``Engine.abort`` while a looked-ahead decode step runs: the step is brought to its end first,
    the request leaves with what it has, the others go on, and every page comes back."""
    from ayaka_py_b200 import EngineConfig, Request, SamplingParams, StopCriteria
    from ayaka_py_b200.engine.engine import Engine
    from ayaka_py_b200.engine.loading import load_model
    folder, cfg, weights = model_folders["A"]
    prompts = tiny_models.prompts(cfg, [9, 21, 5], seed=43)
    _, model = load_model(folder, "float32", "cuda")
    engine = Engine(model, EngineConfig(dtype="float32", page_size=16, kv_pages=32, max_requests=2, lookahead=True),
                    eos_token_id=None)
    def submit(i):
        engine.submit(Request(f"r{i}", prompts[i], SamplingParams(temperature=0.0), StopCriteria(max_tokens=20, ignore_eos=True)))

    submit(0)
    submit(1)
    for _ in range(6):
        engine.step()
    assert engine._inflight is not None                 # a step is on the GPU whose tokens nobody has seen
    submit(2)                                           # both slots are taken: it waits
    engine.abort("r2")                                  # waiting: never ran
    engine.abort("r0")                                  # running, with the step in flight
    assert engine._inflight is None
    assert engine.finished["r0"].finish_reason == "abort" and engine.finished["r2"].token_ids == []
    kept = engine.finished["r0"].token_ids
    assert 5 <= len(kept) <= 8 and kept == plain_gpt2.greedy_generate(cfg, weights, prompts[0], len(kept))
    engine.cache.check_invariants()
    done = engine.run_until_idle()
    assert done["r1"].token_ids == plain_gpt2.greedy_generate(cfg, weights, prompts[1], 20)
    engine.cache.assert_clean()
