"""A plain, slow GPT-2 for tests: whole sequences, no cache, NumPy only.

It is written from the formulas of the Ayaka reference (file:line given at each
function, paths relative to ``python/ayaka/``) and shares no code with the
engine: it has its own reader for model folders, its own layer functions and
its own sampling twin.  ``tests/golden/make_golden.py`` compares it once with
the reference's own ``forward_dense`` on tiny random models; the stored outputs
are checked by ``tests/test_plain.py``.

Every function takes ``dtype`` through its inputs: pass float64 arrays for a
stricter oracle, float32 arrays for "what a careful fp32 program gives".
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np

# --------------------------------------------------------------------------
# reading a model folder (config.json + model.safetensors), independent reader
# --------------------------------------------------------------------------

_NP_DTYPES = {"F32": np.float32, "F64": np.float64, "F16": np.float16,
              "I32": np.int32, "I64": np.int64}


def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_safetensors(path) -> dict[str, np.ndarray]:
    """safetensors: u64 LE header length, JSON header, payload
    (format as parsed in model_loader/st.py:199-331)."""
    blob = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = blob[base + lo:base + hi]
        shape = tuple(info["shape"])
        if info["dtype"] == "BF16":
            arr = _bf16_to_f32(np.frombuffer(raw, dtype=np.uint16)).reshape(shape)
        else:
            arr = np.frombuffer(raw, dtype=_NP_DTYPES[info["dtype"]]).reshape(shape)
        out[name] = np.array(arr)
    return out


def read_model_folder(folder, dtype=np.float32):
    """Returns (config dict with HF short keys, tensors by HF name as ``dtype``).

    Names without the ``transformer.`` prefix get it (models/gpt2.py:57-61);
    legacy mask buffers ``.attn.bias`` / ``.attn.masked_bias`` are dropped
    (models/gpt2.py:54)."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    tensors = {}
    for name, arr in read_safetensors(folder / "model.safetensors").items():
        if name.endswith(".attn.bias") or name.endswith(".attn.masked_bias"):
            continue
        if name != "lm_head.weight" and not name.startswith("transformer."):
            name = "transformer." + name
        tensors[name] = arr.astype(dtype)
    return config, tensors


# --------------------------------------------------------------------------
# configuration (defaults of models/gpt2.py:91-109)
# --------------------------------------------------------------------------

def resolve_config(config: dict) -> dict:
    c = dict(config)
    out = {
        "vocab_size": c.get("vocab_size", 50257),
        "n_embd": c.get("n_embd", c.get("hidden_size", 768)),
        "n_layer": c.get("n_layer", c.get("num_hidden_layers", 12)),
        "n_head": c.get("n_head", c.get("num_attention_heads", 12)),
        "n_positions": c.get("n_positions", c.get("max_position_embeddings", 1024)),
        "n_inner": c.get("n_inner", c.get("intermediate_size", None)),
        "activation_function": c.get("activation_function", "gelu_new"),
        "layer_norm_epsilon": c.get("layer_norm_epsilon", c.get("layer_norm_eps", 1e-5)),
        "scale_attn_weights": c.get("scale_attn_weights", True),
        "scale_attn_by_inverse_layer_idx": c.get("scale_attn_by_inverse_layer_idx", False),
        "tie_word_embeddings": c.get("tie_word_embeddings", True),
    }
    if out["n_inner"] is None:
        out["n_inner"] = 4 * out["n_embd"]          # models/gpt2.py:140-145
    return out


# --------------------------------------------------------------------------
# one function for each part
# --------------------------------------------------------------------------

def embed(tokens, positions, wte, wpe):
    """x = wte[token] + wpe[position]  (models/gpt2.py:516-517)."""
    return wte[np.asarray(tokens)] + wpe[np.asarray(positions)]


def layer_norm(x, weight, bias, eps):
    """(x - mean) * rsqrt(var + eps) * w + b, biased variance over the last
    dim (layers/norm.py:198-205; kernel/triton/norm.py:327-339)."""
    mean = x.mean(axis=-1, keepdims=True)
    centered = x - mean
    var = (centered * centered).mean(axis=-1, keepdims=True)
    return centered / np.sqrt(var + x.dtype.type(eps)) * weight + bias


def _erf(x):
    return np.vectorize(math.erf, otypes=[np.float64])(x)


def activation(name: str, x):
    """Name map of layers/activation.py:198-203; formulas of
    kernel/triton/activation.py:145-154."""
    t = x.dtype.type
    if name == "gelu":
        return (x * 0.5 * (1.0 + _erf(x.astype(np.float64) * 0.7071067811865475))).astype(x.dtype)
    if name in ("gelu_new", "gelu_fast", "gelu_pytorch_tanh", "gelu_tanh"):
        inner = t(0.7978845608028654) * (x + t(0.044715) * x * x * x)
        return x * t(0.5) * (t(1.0) + np.tanh(inner))
    if name == "quick_gelu":
        return x / (t(1.0) + np.exp(-t(1.702) * x))
    raise ValueError(name)


def linear(x, weight_in_out, bias):
    """Conv1D as the checkpoint stores it: y = x @ W[in,out] + b
    (models/gpt2.py:205-251 transposes W to [out,in] for F.linear; the product
    is the same)."""
    return x @ weight_in_out + bias


def causal_attention(q, k, v, scale, window=None, positions=None):
    """q,k,v: [T, H, Dh].  s_ij = (q_i . k_j) * scale for j <= i; softmax over
    j; o_i = sum_j a_ij v_j  (kernel/triton/paged_attention.py:295-355; dense
    oracle models/_common.py:306-321).  ``window`` (not used by GPT-2) keeps
    only keys with i - j < window."""
    T, H, Dh = q.shape
    pos = np.arange(T) if positions is None else np.asarray(positions)
    out = np.zeros_like(q)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= (pos[:, None] - pos[None, :]) < window
    for h in range(H):
        s = (q[:, h, :] @ k[:, h, :].T) * q.dtype.type(scale)
        s = np.where(allowed, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, h, :] = p @ v[:, h, :]
    return out


def attention_part(h, w_attn, b_attn, w_proj, b_proj, n_head, scale):
    """c_attn, split q|k|v, heads, causal attention, c_proj
    (models/gpt2.py:364-372)."""
    T, d = h.shape
    qkv = linear(h, w_attn, b_attn)
    q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
    dh = d // n_head
    o = causal_attention(q.reshape(T, n_head, dh), k.reshape(T, n_head, dh),
                         v.reshape(T, n_head, dh), scale)
    return linear(o.reshape(T, d), w_proj, b_proj)


def mlp_part(h, w_fc, b_fc, w_proj, b_proj, act):
    """c_fc -> act -> c_proj  (models/gpt2.py:400-403)."""
    return linear(activation(act, linear(h, w_fc, b_fc)), w_proj, b_proj)


def attention_scale(cfg, layer: int) -> float:
    """Dh^-0.5 when scale_attn_weights (models/gpt2.py:147-149); divided by
    (layer+1) when scale_attn_by_inverse_layer_idx — the reference refuses that
    option (models/gpt2.py:131-132); the meaning is the one of the HF key."""
    dh = cfg["n_embd"] // cfg["n_head"]
    s = dh ** -0.5 if cfg["scale_attn_weights"] else 1.0
    if cfg["scale_attn_by_inverse_layer_idx"]:
        s = s / float(layer + 1)
    return s


def block(x, tensors, cfg, layer: int):
    """x += attn(ln_1(x)); x += mlp(ln_2(x))  (models/gpt2.py:435-438)."""
    p = f"transformer.h.{layer}."
    eps = cfg["layer_norm_epsilon"]
    h = layer_norm(x, tensors[p + "ln_1.weight"], tensors[p + "ln_1.bias"], eps)
    x = x + attention_part(h, tensors[p + "attn.c_attn.weight"], tensors[p + "attn.c_attn.bias"],
                           tensors[p + "attn.c_proj.weight"], tensors[p + "attn.c_proj.bias"],
                           cfg["n_head"], attention_scale(cfg, layer))
    h = layer_norm(x, tensors[p + "ln_2.weight"], tensors[p + "ln_2.bias"], eps)
    x = x + mlp_part(h, tensors[p + "mlp.c_fc.weight"], tensors[p + "mlp.c_fc.bias"],
                     tensors[p + "mlp.c_proj.weight"], tensors[p + "mlp.c_proj.bias"],
                     cfg["activation_function"])
    return x


def head(x, tensors, cfg):
    """ln_f then logits = h @ wte[:V]^T, no bias (models/gpt2.py:530;
    models/_common.py:248-253; layers/embedding.py:741-747)."""
    h = layer_norm(x, tensors["transformer.ln_f.weight"], tensors["transformer.ln_f.bias"],
                   cfg["layer_norm_epsilon"])
    if cfg["tie_word_embeddings"] or "lm_head.weight" not in tensors:
        w = tensors["transformer.wte.weight"]
    else:
        w = tensors["lm_head.weight"]
    return h @ w[:cfg["vocab_size"]].T


def forward(config: dict, tensors: dict, tokens) -> np.ndarray:
    """Logits [T, V] of one whole sequence."""
    cfg = resolve_config(config)
    tokens = np.asarray(tokens, dtype=np.int64)
    x = embed(tokens, np.arange(len(tokens)), tensors["transformer.wte.weight"],
              tensors["transformer.wpe.weight"])
    for layer in range(cfg["n_layer"]):
        x = block(x, tensors, cfg, layer)
    return head(x, tensors, cfg)


def greedy_generate(config, tensors, prompt, n_new):
    """Greedy decoding by recomputing the whole sequence each time; the lowest
    index wins ties (sampling/plan.py:353-355: argmax)."""
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(np.argmax(forward(config, tensors, ids)[-1])))
    return ids[len(prompt):]


# --------------------------------------------------------------------------
# sampling twin: Philox4x32-10 and the draws built on it
# --------------------------------------------------------------------------

_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32_10(counter, key):
    """Random123 Philox4x32 with 10 rounds (sampling/rng.py:126-146)."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for r in range(10):
        if r > 0:
            k0 = (k0 + _W0) & 0xFFFFFFFF
            k1 = (k1 + _W1) & 0xFFFFFFFF
        p0 = _M0 * c0
        p1 = _M1 * c2
        hi0, lo0 = p0 >> 32, p0 & 0xFFFFFFFF
        hi1, lo1 = p1 >> 32, p1 & 0xFFFFFFFF
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & 0xFFFFFFFF, lo1, (hi0 ^ c3 ^ k1) & 0xFFFFFFFF, lo0
    return c0, c1, c2, c3


def philox_uniform(seed: int, offset: int) -> float:
    """One 53-bit uniform in [0,1): key = seed, counter = offset >> 1, words
    (w0,w1) for an even offset and (w2,w3) for an odd one
    (sampling/rng.py:149-173)."""
    seed &= 0xFFFFFFFFFFFFFFFF
    ctr = offset >> 1
    w = philox4x32_10((ctr & 0xFFFFFFFF, (ctr >> 32) & 0xFFFFFFFF, 0, 0),
                      (seed & 0xFFFFFFFF, seed >> 32))
    hi, lo = (w[2], w[3]) if offset & 1 else (w[0], w[1])
    return float(((hi << 32) | lo) >> 11) * (1.0 / float(1 << 53))


def splitmix64(x: int) -> int:
    """sampling/rng.py:220-252."""
    m = 0xFFFFFFFFFFFFFFFF
    z = (x + 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)


def derive_seed(request_index: int) -> int:
    """Seed of a request that names none (sampling/rng.py:255-267)."""
    return splitmix64(request_index) & 0x7FFFFFFFFFFFFFFF


def filtered_probabilities(logits, temperature, top_k=-1, top_p=1.0, min_p=0.0):
    """Token-order probabilities after the reference's filters, in its order
    top_k -> renormalise -> top_p -> min_p over the descending sort
    (sampling/ops/sampling.py:473-540), then normalised (:583-585).
    ``scaled = logits / max(T, 1e-6)`` (sampling/plan.py:348-349)."""
    z = np.asarray(logits, dtype=np.float64) / max(float(temperature), 1e-6)
    z = z - z.max()
    p = np.exp(z)
    p = p / p.sum()
    order = np.argsort(-p, kind="stable")
    sp = p[order]
    if top_k is not None and top_k > 0:
        sp[top_k:] = 0.0
        sp = sp / sp.sum()
    if top_p < 1.0:
        cum = np.cumsum(sp)
        drop = (cum - sp) > top_p
        drop[0] = False
        sp[drop] = 0.0
    if min_p > 0.0:
        sp[sp < min_p * sp[0]] = 0.0
    sp = sp / sp.sum()
    out = np.zeros_like(p)
    out[order] = sp
    return out


def sample_token(logits, temperature, seed, offset, top_k=-1, top_p=1.0, min_p=0.0):
    """Greedy when temperature == 0 or top_k == 1 (sampling/params.py:127-134);
    else one inverse-CDF draw with u = philox(seed, offset).  The engine walks
    the cumulative sum in token-id order (the reference walks it in sorted
    order, sampling/ops/sampling.py:587-589: the distribution is the same, the
    token for a given u is not)."""
    if temperature == 0 or top_k == 1:
        return int(np.argmax(logits))
    p = filtered_probabilities(logits, temperature, top_k, top_p, min_p)
    u = philox_uniform(seed, offset)
    cum = np.cumsum(p)
    idx = int(np.searchsorted(cum, u * cum[-1], side="left"))
    idx = min(idx, len(p) - 1)
    while p[idx] == 0.0 and idx > 0:     # never return a filtered token
        idx -= 1
    return idx
