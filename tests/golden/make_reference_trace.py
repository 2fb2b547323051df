"""Records a schedule and the per-step logits of the reference's own *paged* engine, once, on the CPU.

Run from the repository root with the reference checkout given:

    python tests/golden/make_reference_trace.py /path/to/ayaka-py

It imports ``ayaka`` from ``<checkout>/python`` and builds what ``ayaka serve`` builds
(``commands/cli.py:112-171``): ``GPT2ForCausalLM(cfg, device="cpu", dtype=float32, backend="torch")``
with the tiny-B weights of these tests copied in (as ``make_golden.py`` does: Conv1D weights transposed,
the query columns of layer i divided by i + 1 because the reference refuses
``scale_attn_by_inverse_layer_idx``), then ``ServingRuntime(model, tokenizer_folder, pages=41,
page_size=8, max_requests=5, batch_tokens=64, prefill_chunk=24, backend="reference")`` and a second
engine from the runtime's own builder (``ServingRuntime._build_tail``; the first one is stepped by the
service's thread).  Five requests (1 / 9 / 33 / 64 / 120 prompt ids, 24 new tokens each, greedy) are
submitted at once; 40 pages of 8 tokens do not hold them all, so the reference's continuous scheduler
(``sched/continuous.py``) cuts prompts into portions beside decoded tokens and preempts with recompute.
``ModelRunner._forward_tail`` (``runner/model_runner.py:175-201``) is wrapped: for every forward step
the slices (request, first position, token count, whether its last row is sampled) and the ``[S, V]``
logits it returned are stored in ``tests/golden/reference_paged_trace.npz``.
``tests/test_gpu_replay.py`` turns the stored schedule into replay records and compares this engine's
logits with the stored ones; it needs no reference checkout.
"""

from __future__ import annotations

import json
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import tiny_models  # noqa: E402

PROMPTS = [1, 9, 33, 64, 120]
NEW_TOKENS = 24
PAGES, PAGE_SIZE, BUDGET, CHUNK = 41, 8, 64, 24        # 40 usable pages of 8 tokens


def write_tokenizer(folder: Path, vocab_size: int) -> None:
    vocab = {f"t{i}": i for i in range(vocab_size)}
    (folder / "tokenizer.json").write_text(json.dumps({
        "version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
        "pre_tokenizer": {"type": "WhitespaceSplit"}, "post_processor": None, "decoder": None,
        "model": {"type": "WordLevel", "vocab": vocab, "unk_token": "t0"}}))
    (folder / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "t0", "model_max_length": 1 << 20}))


def main() -> None:
    checkout = Path(sys.argv[1])
    sys.path.insert(0, str(checkout / "python"))
    sys.dont_write_bytecode = True
    import torch
    from ayaka.models.gpt2 import GPT2Config, GPT2ForCausalLM
    from ayaka.request.schema import Request, StopCriteria
    from ayaka.runtime.serving import ServingConfig, ServingRuntime
    from ayaka.sampling.params import SamplingParams

    cfg = dict(tiny_models.TINY_B)
    weights = {k: v.copy() for k, v in tiny_models.numpy_weights(cfg, 12, scale=4.0, bf16_exact=True).items()}
    d = cfg["n_embd"]
    for i in range(cfg["n_layer"]):
        p = f"transformer.h.{i}.attn.c_attn."
        weights[p + "weight"][:, :d] /= float(i + 1)
        weights[p + "bias"][:d] /= float(i + 1)
    cfg["scale_attn_by_inverse_layer_idx"] = False
    keys = {k: v for k, v in cfg.items() if k not in ("architectures", "model_type")}
    model = GPT2ForCausalLM(GPT2Config.from_dict(keys), device="cpu", dtype=torch.float32, backend="torch")
    params = dict(model.named_parameters())
    with torch.no_grad():
        for name, arr in weights.items():
            t = torch.from_numpy(arr)
            if name.endswith(("c_attn.weight", "c_proj.weight", "c_fc.weight")):
                t = t.t().contiguous()
            if name == "transformer.wte.weight":
                params[name].zero_()
                params[name][: t.shape[0]].copy_(t)
            else:
                params[name].copy_(t)
    model.eval()
    prompts = tiny_models.prompts(tiny_models.TINY_B, PROMPTS, seed=22)

    steps = []
    with tempfile.TemporaryDirectory() as tmp:
        folder = Path(tmp)
        write_tokenizer(folder, cfg["vocab_size"])
        runtime = ServingRuntime(model, folder, config=ServingConfig(model="tiny-b", structured_outputs=False),
                                 pages=PAGES, page_size=PAGE_SIZE, max_requests=len(PROMPTS), batch_tokens=BUDGET,
                                 prefill_chunk=CHUNK, max_model_len=cfg["n_positions"], backend="reference",
                                 tokenizer_workers=0)
        tail = runtime._build_tail(PAGES)
        runner, engine = tail.runner, tail.engine
        inner = runner._forward_tail

        def recording(prepared):
            result = inner(prepared)
            rows = [(str(s.request_id), int(s.query_start), int(s.query_count), bool(s.sample_last_query))
                    for s in prepared.step.slices]
            count = int(result.sampling_count)
            logits = result.logits[:count].detach().float().cpu().numpy().copy() if count else np.zeros((0, cfg["vocab_size"]), np.float32)
            steps.append((rows, logits))
            return result

        runner._forward_tail = recording
        lifecycles = [engine.submit(Request(f"r{i}", tuple(p), SamplingParams(temperature=0.0),
                                            StopCriteria(max_tokens=NEW_TOKENS, ignore_eos=True)))
                      for i, p in enumerate(prompts)]
        spins = 0
        while any(not lc.is_terminal for lc in lifecycles):
            engine.step()
            spins += 1
            assert spins < 100000
        generated = [list(lc.output_token_ids) for lc in lifecycles]
        engine.close()
        tail.resources.close()
        runtime.close()

    # the stored form: one row per slice, and the logits of all steps stacked
    slice_rows, logit_rows, restarts = [], [], 0
    seen_end: dict[str, int] = {}
    for index, (rows, logits) in enumerate(steps):
        sampled = 0
        for rid, start, count, sample in rows:
            if start == 0 and seen_end.get(rid, 0) > 0:
                restarts += 1                              # a preempted request starts over
            seen_end[rid] = start + count
            slice_rows.append((index, int(rid[1:]), start, count, int(sample)))
            sampled += int(sample)
        assert sampled == logits.shape[0], (index, sampled, logits.shape)
        logit_rows.append(logits)
    vocab = cfg["vocab_size"]
    store = {
        "slices": np.asarray(slice_rows, dtype=np.int32),                    # step, request, first position, tokens, sampled
        "logits": np.concatenate(logit_rows).astype(np.float32)[:, :vocab],  # rows in the order of the sampled slices
        "prompts": np.asarray([t for p in prompts for t in p], dtype=np.int32),
        "prompt_lengths": np.asarray(PROMPTS, dtype=np.int32),
        "generated": np.asarray(generated, dtype=np.int32),
        "geometry": np.asarray([PAGES, PAGE_SIZE, BUDGET, CHUNK, NEW_TOKENS], dtype=np.int32),
    }
    np.savez_compressed(HERE / "reference_paged_trace.npz", **store)
    print(f"{len(steps)} forward steps, {restarts} restarts after preemption, {store['logits'].shape[0]} logits rows, "
          f"largest |logit| {np.abs(store['logits']).max():.3f}")


if __name__ == "__main__":
    main()
