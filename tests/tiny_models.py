"""Tiny GPT-2 configurations and seeded weights for tests (NumPy only).

Two configurations that differ in every size and option.  ``numpy_weights``
draws the tensors with NumPy's legacy ``RandomState`` (stable across NumPy
versions) in HF names and Conv1D ``[in, out]`` layout; ``write_folder`` writes
them with a writer of its own, so that the engine's loader is tested on files
that the engine did not make.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

TINY_A = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 64, "n_head": 4, "n_inner": 256, "vocab_size": 512,
    "n_positions": 128, "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
    "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": True,
}

TINY_B = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 3, "n_embd": 96, "n_head": 2, "n_inner": 320, "vocab_size": 1000,
    "n_positions": 256, "layer_norm_epsilon": 1e-6, "activation_function": "gelu",
    "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": True,
    "tie_word_embeddings": True,
}

# A third one for head size 32 / odd head count / more positions (long decoding).
TINY_C = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 160, "n_head": 5, "n_inner": 200, "vocab_size": 777,
    "n_positions": 640, "layer_norm_epsilon": 3e-5, "activation_function": "gelu_new",
    "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": True,
}


# The options that A and B leave at their defaults: quick_gelu, unscaled scores, a head of its own.
TINY_E = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 48, "n_head": 3, "n_inner": 100, "vocab_size": 130,
    "n_positions": 96, "layer_norm_epsilon": 1e-5, "activation_function": "quick_gelu",
    "scale_attn_weights": False, "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": False,
}


# Head size 64 (the tensor-core attention kernel's), three heads, width 192.
TINY_D = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 192, "n_head": 3, "n_inner": 264, "vocab_size": 300,
    "n_positions": 512, "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
    "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": True,
    "tie_word_embeddings": True,
}


def tensor_shapes(cfg: dict) -> dict[str, tuple]:
    d, L, V = cfg["n_embd"], cfg["n_layer"], cfg["vocab_size"]
    inner = cfg.get("n_inner") or 4 * d
    shapes = {"transformer.wte.weight": (V, d), "transformer.wpe.weight": (cfg["n_positions"], d)}
    for i in range(L):
        p = f"transformer.h.{i}."
        shapes[p + "ln_1.weight"] = (d,)
        shapes[p + "ln_1.bias"] = (d,)
        shapes[p + "attn.c_attn.weight"] = (d, 3 * d)
        shapes[p + "attn.c_attn.bias"] = (3 * d,)
        shapes[p + "attn.c_proj.weight"] = (d, d)
        shapes[p + "attn.c_proj.bias"] = (d,)
        shapes[p + "ln_2.weight"] = (d,)
        shapes[p + "ln_2.bias"] = (d,)
        shapes[p + "mlp.c_fc.weight"] = (d, inner)
        shapes[p + "mlp.c_fc.bias"] = (inner,)
        shapes[p + "mlp.c_proj.weight"] = (inner, d)
        shapes[p + "mlp.c_proj.bias"] = (d,)
    shapes["transformer.ln_f.weight"] = (d,)
    shapes["transformer.ln_f.bias"] = (d,)
    if not cfg.get("tie_word_embeddings", True):
        shapes["lm_head.weight"] = (V, d)
    return shapes


def round_bf16(a: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16 (ties to even), as float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return (u.astype(np.uint32) << 16).view(np.float32).reshape(a.shape)


def numpy_weights(cfg: dict, seed: int, scale: float = 1.0, bf16_exact: bool = True):
    """wte/wpe/c_attn/c_fc ~ N(0, .02); c_proj ~ N(0, .02/sqrt(2L)); biases ~
    N(0, .01); LN gamma = 1 + N(0, .05), beta ~ N(0, .02).  ``scale`` widens
    the matrices so that tiny models have logits that differ visibly.  With
    ``bf16_exact`` every value is representable in bfloat16, so a bf16 engine
    and the fp32 oracle read the same numbers."""
    rs = np.random.RandomState(seed)
    L = cfg["n_layer"]
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        g = rs.standard_normal(shape).astype(np.float32)
        if name.endswith("ln_1.weight") or name.endswith("ln_2.weight") or name.endswith("ln_f.weight"):
            w = 1.0 + 0.05 * g
        elif ".ln_" in name and name.endswith(".bias"):
            w = 0.02 * g
        elif name.endswith(".bias"):
            w = 0.01 * g
        elif name.endswith("c_proj.weight"):
            w = scale * 0.02 / np.sqrt(2.0 * L) * g
        else:
            w = scale * 0.02 * g
        w = w.astype(np.float32)
        out[name] = round_bf16(w) if bf16_exact else w
    return out


def _to_bf16_bytes(a: np.ndarray) -> bytes:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return (u >> 16).astype(np.uint16).tobytes()


def write_safetensors(path, tensors: dict[str, np.ndarray], bf16_names=()):
    header, chunks, off = {}, [], 0
    for name, arr in tensors.items():
        if name in bf16_names:
            raw, dt = _to_bf16_bytes(arr), "BF16"
        else:
            arr = np.ascontiguousarray(arr)
            dt = {np.dtype(np.float32): "F32", np.dtype(np.int32): "I32",
                  np.dtype(np.int64): "I64", np.dtype(np.float16): "F16"}[arr.dtype]
            raw = arr.tobytes()
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        chunks.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for c in chunks:
            f.write(c)


def write_folder(folder, cfg: dict, tensors: dict[str, np.ndarray], matrices_bf16: bool = True):
    """config.json + model.safetensors.  With ``matrices_bf16`` the 2-D tensors
    are stored as BF16 (exact when the values came from ``numpy_weights`` with
    ``bf16_exact``), vectors as F32."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    bf16 = [n for n, a in tensors.items() if matrices_bf16 and a.ndim == 2]
    write_safetensors(folder / "model.safetensors", tensors, bf16_names=bf16)
    return folder


def prompts(cfg: dict, lengths, seed: int):
    rs = np.random.RandomState(seed)
    return [rs.randint(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


def random_config(seed: int) -> tuple[dict, int, list[int]]:
    """A tiny configuration drawn from a seed: head counts 1..7, head sizes 16..128 in steps of 16,
    feed-forward widths that are and are not multiples of 8, odd vocabularies, every activation.
    Returns (config, page size, prompt lengths).  Scores stay scaled (unscaled scores of random
    weights reach the hundreds, where bfloat16 rounding of q and k alone moves a probability by
    tens of per cent)."""
    rs = np.random.RandomState(1000 + seed)
    heads = int(rs.choice([1, 2, 3, 4, 5, 7]))
    head_dim = int(rs.choice([16, 32, 48, 64, 64, 80, 128]))
    inner = int(rs.choice([8 * rs.randint(8, 50), 4 * rs.randint(20, 90), rs.randint(70, 300)]))
    cfg = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": int(rs.randint(1, 4)),
           "n_embd": heads * head_dim, "n_head": heads, "n_inner": inner, "vocab_size": int(rs.randint(40, 1300)),
           "n_positions": int(rs.choice([200, 300, 520, 700])),
           "layer_norm_epsilon": float(rs.choice([1e-5, 1e-6, 3e-4])),
           "activation_function": str(rs.choice(["gelu_new", "gelu", "quick_gelu", "gelu_pytorch_tanh"])),
           "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": bool(rs.rand() < 0.5),
           "tie_word_embeddings": True}
    page = int(rs.choice([8, 16, 32, 64]))
    limit = cfg["n_positions"]
    lengths = [int(x) for x in rs.randint(1, limit, size=rs.randint(2, 5))] + [int(rs.choice([128, 129, 256, limit]))]
    return cfg, page, [min(n, limit) for n in lengths]
