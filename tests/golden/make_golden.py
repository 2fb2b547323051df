"""Pins the plain implementation (tests/plain_gpt2.py) to the reference's own
model code, once, on the CPU.

Run from the repository root with the reference checkout given:

    python tests/golden/make_golden.py /path/to/ayaka-py

It imports ``ayaka.models.gpt2`` from ``<checkout>/python``, builds
``GPT2ForCausalLM(cfg, device="cpu", dtype=float32, backend="torch")``, copies
seeded tiny weights into it (Conv1D weights transposed to [out, in], wte into
the first V rows of its padded table) and calls ``forward_dense``.  The
reference refuses ``scale_attn_by_inverse_layer_idx`` (models/gpt2.py:131-132),
so for tiny B the query columns of ``c_attn`` of layer i are divided by (i+1)
and the flag is switched off: the same function in exact arithmetic.  It writes
``tests/golden/reference_logits.npz`` with the reference's logits and the
largest difference from the plain implementation; ``tests/test_plain.py``
reads that file and needs no reference checkout.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import plain_gpt2  # noqa: E402
import tiny_models  # noqa: E402

CASES = {"A": (tiny_models.TINY_A, 11, 24, 4.0), "B": (tiny_models.TINY_B, 12, 21, 4.0),
         # quick_gelu, scores that are not scaled by 1/sqrt(head size), a head that is not the token table
         "E": (tiny_models.TINY_E, 15, 19, 2.0)}


def reference_logits(checkout: Path, cfg: dict, weights: dict, tokens) -> np.ndarray:
    sys.path.insert(0, str(checkout / "python"))
    import torch
    from ayaka.models.gpt2 import GPT2Config, GPT2ForCausalLM

    cfg = dict(cfg)
    weights = {k: v.copy() for k, v in weights.items()}
    if cfg.get("scale_attn_by_inverse_layer_idx"):
        d = cfg["n_embd"]
        for i in range(cfg["n_layer"]):
            p = f"transformer.h.{i}.attn.c_attn."
            weights[p + "weight"][:, :d] /= float(i + 1)
            weights[p + "bias"][:d] /= float(i + 1)
        cfg["scale_attn_by_inverse_layer_idx"] = False
    keys = {k: v for k, v in cfg.items() if k not in ("architectures", "model_type")}
    model = GPT2ForCausalLM(GPT2Config.from_dict(keys), device="cpu", dtype=torch.float32,
                            backend="torch")
    params = dict(model.named_parameters())
    with torch.no_grad():
        for name, arr in weights.items():
            t = torch.from_numpy(arr)
            if name.endswith(("c_attn.weight", "c_proj.weight", "c_fc.weight")):
                t = t.t().contiguous()
            p = params[name]
            if name in ("transformer.wte.weight", "lm_head.weight"):      # tables padded to a multiple of 64 rows
                p.zero_()
                p[: t.shape[0]].copy_(t)
            else:
                p.copy_(t)
        out = model.forward_dense(torch.tensor(tokens, dtype=torch.int64))
    return out.float().numpy()


def main() -> None:
    checkout = Path(sys.argv[1])
    store = {}
    for tag, (cfg, seed, length, scale) in CASES.items():
        weights = tiny_models.numpy_weights(cfg, seed, scale=scale, bf16_exact=False)
        tokens = tiny_models.prompts(cfg, [length], seed + 100)[0]
        ref = reference_logits(checkout, cfg, weights, tokens)
        mine = plain_gpt2.forward(cfg, weights, tokens)
        diff = float(np.abs(ref - mine).max())
        print(f"tiny {tag}: T={length} max|reference - plain| = {diff:.3e}, max|logit| = {np.abs(ref).max():.3f}")
        store[f"{tag}_logits"] = ref.astype(np.float32)
        store[f"{tag}_tokens"] = np.asarray(tokens, dtype=np.int64)
        store[f"{tag}_maxdiff"] = np.float64(diff)
    np.savez_compressed(HERE / "reference_logits.npz", **store)


if __name__ == "__main__":
    main()
