"""Each part alone against the plain functions; the model as data (a layer run
twice, a layer reading another's cache); and a toy architecture with a mixer
that keeps state of its own, registered and stepped from here without touching
the package."""

import json
from dataclasses import dataclass
from types import SimpleNamespace
from typing import ClassVar

import numpy as np
import pytest
import torch

import plain_gpt2
import tiny_models

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def tol(dtype, scale=1.0):
    return (3e-5 if dtype == "float32" else 3e-2) * scale


def context_for(groups, dtype, lengths, page_size=8, vocab=1000, positions=512, starts=None):
    """A cache manager and a step context for whole sequences (or continuations)."""
    from ayaka_py_b200.cache import CacheManager
    from ayaka_py_b200.engine.step import StepEntry, StepRunner

    pages = sum(-(-(n + (starts[i] if starts else 0)) // page_size) for i, n in enumerate(lengths)) + 1
    cache = CacheManager(groups, kv_pages=pages, page_size=page_size, max_requests=len(lengths),
                         max_len=positions, dtype=DT[dtype], device="cuda")
    model = SimpleNamespace(device="cuda", dtype=DT[dtype], max_positions=positions, vocab_size=vocab)
    runner = StepRunner(model, cache, max_tokens=sum(lengths))
    return cache, runner


def run_entries(cache, runner, token_lists, wants=None):
    from ayaka_py_b200.engine.step import StepEntry
    entries = []
    for i, toks in enumerate(token_lists):
        slot = cache.slot_of.get(i)
        if slot is None:
            slot = cache.open(i)
        entries.append(StepEntry(slot, int(cache.length[slot]), toks, wants[i] if wants else []))
    res = cache.reserve([(e.slot, e.start, len(e.tokens)) for e in entries])
    ctx = runner.prepare(entries)
    return ctx, res


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_positions_norm_head(dtype):
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(0)
    V, d, npos = 333, 40, 64
    emb = make_part(PartSpec("token_embedding", {"vocab": V, "width": d}), DT[dtype], "cuda")
    pos = make_part(PartSpec("learned_positions", {"positions": npos, "width": d}), DT[dtype], "cuda")
    norm = make_part(PartSpec("layernorm", {"width": d, "eps": 1e-4}), DT[dtype], "cuda")
    head = make_part(PartSpec("lm_head", {"vocab": V, "width": d}), DT[dtype], "cuda")
    wte, wpe = dev(rs.randn(V, d).astype(np.float32), DT[dtype]), dev(rs.randn(npos, d).astype(np.float32), DT[dtype])
    g, b = rs.randn(d).astype(np.float32), rs.randn(d).astype(np.float32)
    emb.bind({"weight": wte}); pos.bind({"weight": wpe}); head.bind({"weight": wte})
    norm.bind({"weight": dev(g), "bias": dev(b)})
    cache, runner = context_for([], dtype, [7, 3], vocab=V, positions=npos)
    toks = [rs.randint(0, V, 7).tolist(), rs.randint(0, V, 3).tolist()]
    ctx, _ = run_entries(cache, runner, toks, wants=[[6, 0], [2]])
    x = emb.forward(ctx, pos)
    w64, p64 = wte.double().cpu().numpy(), wpe.double().cpu().numpy()
    want_x = np.concatenate([plain_gpt2.embed(t, np.arange(len(t)), w64, p64) for t in toks])
    assert np.abs(x.cpu().numpy() - want_x).max() < 1e-6
    h = norm.forward(x, ctx, rows=ctx.want_rows)
    want_h = plain_gpt2.layer_norm(want_x, g, b, 1e-4)[[6, 0, 9]]
    assert np.abs(h.float().cpu().numpy() - want_h).max() < tol(dtype, 3)
    logits = head.forward(h, ctx)
    assert logits.dtype == torch.float32 and logits.shape == (3, V)
    assert np.abs(logits.cpu().numpy() - h.double().cpu().numpy() @ w64.T).max() < 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("act,name", [("gelu_tanh", "gelu_new"), ("gelu_erf", "gelu"), ("quick_gelu", "quick_gelu")])
def test_mlp_part(dtype, act, name):
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(1)
    d, inner, T = 72, 200, 13
    mlp = make_part(PartSpec("mlp", {"width": d, "inner": inner, "activation": act}), DT[dtype], "cuda")
    up, down = dev(rs.randn(inner, d).astype(np.float32) / 8, DT[dtype]), dev(rs.randn(d, inner).astype(np.float32) / 14, DT[dtype])
    ub, db = rs.randn(inner).astype(np.float32), rs.randn(d).astype(np.float32)
    mlp.bind({"up_weight": up, "down_weight": down, "up_bias": dev(ub), "down_bias": dev(db)})
    h, res = dev(rs.randn(T, d).astype(np.float32), DT[dtype]), rs.randn(T, d).astype(np.float32)
    out = mlp.forward(h, dev(res), None)
    u = plain_gpt2.activation(name, h.double().cpu().numpy() @ up.double().cpu().numpy().T + ub)
    if dtype == "bfloat16":
        u = dev(u.astype(np.float32), torch.bfloat16).double().cpu().numpy()      # the part stores it rounded
    want = res + u @ down.double().cpu().numpy().T + db
    assert out.dtype == torch.float32 and np.abs(out.cpu().numpy() - want).max() < tol(dtype)


def attention_weights(rs, d, H, Hkv, Dh, dtype):
    total = (H + 2 * Hkv) * Dh
    return {"qkv_weight": dev(rs.randn(total, d).astype(np.float32) / np.sqrt(d), DT[dtype]),
            "qkv_bias": dev(rs.randn(total).astype(np.float32) * 0.1),
            "out_weight": dev(rs.randn(d, H * Dh).astype(np.float32) / np.sqrt(H * Dh), DT[dtype]),
            "out_bias": dev(rs.randn(d).astype(np.float32) * 0.1)}


def plain_attention_part(h, w, H, Hkv, Dh, scale, window, dtype):
    """Grouped queries and a window, from the plain functions."""
    f = lambda t: t.double().cpu().numpy()
    qkv = h @ f(w["qkv_weight"]).T + f(w["qkv_bias"])
    if dtype == "bfloat16":
        qkv = f(dev(qkv.astype(np.float32), torch.bfloat16))
    T = h.shape[0]
    q = qkv[:, :H * Dh].reshape(T, H, Dh)
    k = np.repeat(qkv[:, H * Dh:(H + Hkv) * Dh].reshape(T, Hkv, Dh), H // Hkv, axis=1)
    v = np.repeat(qkv[:, (H + Hkv) * Dh:].reshape(T, Hkv, Dh), H // Hkv, axis=1)
    o = plain_gpt2.causal_attention(q, k, v, scale, window=window).reshape(T, H * Dh)
    if dtype == "bfloat16":
        o = f(dev(o.astype(np.float32), torch.bfloat16))
    return o @ f(w["out_weight"]).T + f(w["out_bias"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,Hkv,Dh,window", [(3, 3, 16, None), (4, 2, 48, None), (2, 1, 32, 5)])
def test_attention_part_whole_and_continued(dtype, H, Hkv, Dh, window):
    from ayaka_py_b200.cache import CacheBinding, CacheGroupSpec
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(2)
    d, scale = 56, 0.3
    part = make_part(PartSpec("attention", {"width": d, "num_heads": H, "kv_heads": Hkv, "head_dim": Dh,
                                            "scale": scale, "window": window}), DT[dtype], "cuda")
    w = attention_weights(rs, d, H, Hkv, Dh, dtype)
    part.bind(w)
    lengths = [21, 9]
    cache, runner = context_for([CacheGroupSpec("g", part.cache_need(), 1)], dtype, lengths, page_size=8)
    binding = CacheBinding(0, "g", 0, True)
    hs = [dev(rs.randn(n, d).astype(np.float32), DT[dtype]) for n in lengths]
    want = [plain_attention_part(h.double().cpu().numpy(), w, H, Hkv, Dh, scale, window, dtype) for h in hs]
    # first 13 and 9 rows in one step, then the rest of the first request two rows at a time
    ctx, res = run_entries(cache, runner, [[0] * 13, [0] * 9])
    zero = lambda n: torch.zeros(n, d, device="cuda")
    out = part.forward(torch.cat([hs[0][:13], hs[1]]), zero(22), ctx, binding)
    cache.commit(res)
    got0, got1 = [out[:13].cpu().numpy()], out[13:].cpu().numpy()
    for p in range(13, 21, 2):
        ctx, res = run_entries(cache, runner, [[0, 0]])
        got0.append(part.forward(hs[0][p:p + 2].contiguous(), zero(2), ctx, binding).cpu().numpy())
        cache.commit(res)
    assert np.abs(np.concatenate(got0) - want[0]).max() < tol(dtype)
    assert np.abs(got1 - want[1]).max() < tol(dtype)


def test_block_arrangement_and_run_order():
    """A layer named twice keeps two caches; a run step reading another's cache
    appends nothing and sees the other's keys."""
    from ayaka_py_b200.config.model import GPT2Config
    from ayaka_py_b200.models.gpt2 import gpt2_spec
    from ayaka_py_b200.models.model import Model
    from ayaka_py_b200.parts import RunStep
    import dataclasses

    cfg = GPT2Config.from_dict(tiny_models.TINY_A)
    spec = gpt2_spec(cfg)
    twice = dataclasses.replace(spec, order=(RunStep(0), RunStep(1), RunStep(0), RunStep(1, cache_of=1)))
    model = Model(twice, torch.float32, "cuda")
    assert model.groups[0].layers == 3
    assert [b["mixer"].layer for b in model.bindings] == [0, 1, 2, 1]
    assert [b["mixer"].writes for b in model.bindings] == [True, True, True, False]
    with pytest.raises(ValueError):
        Model(dataclasses.replace(spec, order=(RunStep(0, cache_of=0),)), torch.float32, "cuda")
    with pytest.raises(ValueError):
        Model(dataclasses.replace(spec, order=(RunStep(5),)), torch.float32, "cuda")

    from ayaka_py_b200.cache import CacheManager
    from ayaka_py_b200.engine.step import StepEntry, StepRunner
    from ayaka_py_b200.weights import DictStore, load_weights
    weights = tiny_models.numpy_weights(tiny_models.TINY_A, 3, scale=4.0)
    load_weights(model, DictStore({k: torch.from_numpy(v) for k, v in weights.items()}))
    cache = CacheManager(model.groups, kv_pages=9, page_size=16, max_requests=2, max_len=128,
                         dtype=torch.float32, device="cuda")
    runner = StepRunner(model, cache, max_tokens=64)
    toks = tiny_models.prompts(tiny_models.TINY_A, [19], 1)[0]

    def plain_twice(tokens):
        c = plain_gpt2.resolve_config(tiny_models.TINY_A)
        w = {k: v.astype(np.float64) for k, v in weights.items()}
        d, H = c["n_embd"], c["n_head"]
        x = plain_gpt2.embed(tokens, np.arange(len(tokens)), w["transformer.wte.weight"], w["transformer.wpe.weight"])
        x = plain_gpt2.block(x, w, c, 0)
        entering_second = x
        x = plain_gpt2.block(x, w, c, 1)
        x = plain_gpt2.block(x, w, c, 0)
        # fourth run step: layer 1's weights and queries, keys and values of the SECOND run step
        p, eps, T = "transformer.h.1.", c["layer_norm_epsilon"], len(tokens)
        qkv_now = plain_gpt2.linear(plain_gpt2.layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps),
                                    w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"])
        qkv_then = plain_gpt2.linear(plain_gpt2.layer_norm(entering_second, w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps),
                                     w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"])
        o = plain_gpt2.causal_attention(qkv_now[:, :d].reshape(T, H, -1), qkv_then[:, d:2 * d].reshape(T, H, -1),
                                        qkv_then[:, 2 * d:].reshape(T, H, -1), plain_gpt2.attention_scale(c, 1))
        x = x + plain_gpt2.linear(o.reshape(T, d), w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"])
        x = x + plain_gpt2.mlp_part(plain_gpt2.layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], eps),
                                    w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"], w[p + "mlp.c_proj.weight"],
                                    w[p + "mlp.c_proj.bias"], c["activation_function"])
        return plain_gpt2.head(x, w, c)

    slot = cache.open("r")
    res = cache.reserve([(slot, 0, 12)])
    first = runner.run([StepEntry(slot, 0, toks[:12], list(range(12)))]).cpu().numpy()
    cache.commit(res)
    res = cache.reserve([(slot, 12, 7)])
    second = runner.run([StepEntry(slot, 12, toks[12:], list(range(7)))]).cpu().numpy()
    cache.commit(res)
    # whole, in one step, in a fresh request: cutting must not matter
    other = cache.open("s")
    res = cache.reserve([(other, 0, 19)])
    whole = runner.run([StepEntry(other, 0, toks, list(range(19)))]).cpu().numpy()
    cache.commit(res)
    assert np.abs(np.concatenate([first, second]) - whole).max() < 1e-4
    assert np.abs(whole - plain_twice(toks)).max() < 1e-4


# ------------------------------------------------------------------ toy parts --

@dataclass(frozen=True)
class ToyConfig:
    """Configuration of a toy architecture that exists only in this test."""
    ARCHITECTURE: ClassVar[str] = "ToyRunningMeanLM"
    vocab_size: int = 50
    width: int = 24
    layers: int = 2
    positions: int = 64

    @classmethod
    def from_dict(cls, values):
        return cls(**{k: values[k] for k in ("vocab_size", "width", "layers", "positions") if k in values})

    def to_dict(self):
        return {"architectures": [self.ARCHITECTURE], "vocab_size": self.vocab_size, "width": self.width,
                "layers": self.layers, "positions": self.positions}


def register_toy():
    from ayaka_py_b200.parts import (FeedForward, Init, Mixer, ModelSpec, PartSpec, RunStep, Source,
                                     StateNeed, TensorDecl, pre_norm_layer, register_part)
    from ayaka_py_b200.registry import Architecture, register_architecture

    class RunningMeanMixer(Mixer):
        """mix(h)_t = W . mean(h_0 .. h_t): the running sum is the state it
        keeps per request, in the request's slot."""

        def __init__(self, width, dtype, device):
            self.width, self.dtype = width, dtype
            self.weight = None

        def tensors(self):
            return {"weight": TensorDecl((self.width, self.width), "matrix")}

        def cache_need(self):
            return StateNeed((self.width,), torch.float32)

        def forward(self, h, residual, ctx, cache):
            state = ctx.cache.state_layer(cache.group, cache.layer)       # [slots, width]
            out = torch.empty_like(residual)
            for r in range(ctx.num_requests):
                a, b = int(ctx.host["q_start"][r]), int(ctx.host["q_start"][r + 1])
                slot, start = int(ctx.host["slots"][r]), int(ctx.host["pos0"][r])
                sums = state[slot] + torch.cumsum(h[a:b].float(), dim=0)
                counts = torch.arange(start + 1, start + 1 + (b - a), device=h.device, dtype=torch.float32)
                out[a:b] = residual[a:b] + (sums / counts[:, None]) @ self.weight.float().t()
                state[slot] = sums[-1]
            return out

    class ScaleFeedForward(FeedForward):
        def __init__(self, width, dtype, device):
            self.width = width
            self.gain = None

        def tensors(self):
            return {"gain": TensorDecl((self.width,), "vector")}

        def forward(self, h, residual, ctx):
            return residual + torch.tanh(h.float()) * self.gain

    register_part("toy_running_mean", RunningMeanMixer)
    register_part("toy_scale_ffn", ScaleFeedForward)

    def spec(cfg: ToyConfig) -> ModelSpec:
        d = cfg.width
        norm = lambda name: PartSpec("layernorm", {"width": d, "eps": 1e-5},
                                     {"weight": Source(name + ".g", init=Init(0.1, 1.0)), "bias": Source(name + ".b", init=Init(0.1))})
        layers = tuple(pre_norm_layer(
            norm(f"l{i}.n1"), PartSpec("toy_running_mean", {"width": d}, {"weight": Source(f"l{i}.mix", init=Init(0.3))}),
            norm(f"l{i}.n2"), PartSpec("toy_scale_ffn", {"width": d}, {"gain": Source(f"l{i}.gain", init=Init(0.5))}))
            for i in range(cfg.layers))
        return ModelSpec(cfg.vocab_size, d, cfg.positions,
                         PartSpec("token_embedding", {"vocab": cfg.vocab_size, "width": d}, {"weight": Source("emb", init=Init(1.0))}),
                         PartSpec("no_positions", {}, {}), layers, tuple(RunStep(i) for i in range(cfg.layers)),
                         norm("final"), PartSpec("lm_head", {"vocab": cfg.vocab_size, "width": d}, {"weight": Source("emb", init=Init(1.0))}))

    register_architecture(Architecture("ToyRunningMeanLM", "toy", ToyConfig, spec))


def plain_toy(cfg, t, tokens):
    x = t["emb"][tokens]
    for i in range(cfg.layers):
        h = plain_gpt2.layer_norm(x, t[f"l{i}.n1.g"], t[f"l{i}.n1.b"], 1e-5)
        mean = np.cumsum(h, axis=0) / np.arange(1, len(tokens) + 1)[:, None]
        x = x + mean @ t[f"l{i}.mix"].T
        h = plain_gpt2.layer_norm(x, t[f"l{i}.n2.g"], t[f"l{i}.n2.b"], 1e-5)
        x = x + np.tanh(h) * t[f"l{i}.gain"]
    return plain_gpt2.layer_norm(x, t["final.g"], t["final.b"], 1e-5) @ t["emb"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    import trace_tools
    from ayaka_py_b200.replay import ReplaySession
    from ayaka_py_b200.weights import write_random_model

    register_toy()
    cfg = ToyConfig()
    folder = write_random_model(tmp_path / "toy", cfg, seed=5, dtype="float32")
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyRunningMeanLM"]
    tensors = {k: v.astype(np.float64) for k, v in plain_gpt2.read_safetensors(folder / "model.safetensors").items()}
    rs = np.random.RandomState(0)
    reqs = {f"t{i}": rs.randint(0, cfg.vocab_size, n).tolist() for i, n in enumerate([30, 7, 45, 18])}
    want = {rid: plain_toy(cfg, tensors, toks) for rid, toks in reqs.items()}
    for trace in (trace_tools.whole(reqs), trace_tools.portions(reqs), trace_tools.mixed(reqs, seed=2)):
        session = ReplaySession(folder, "float32", max_tokens=256, page_size=16)
        assert [type(g.need).__name__ for g in session.model.groups] == ["StateNeed"]
        outs = [None if (o := session.step(rec)) is None or o.shape[0] == 0 else o.cpu().numpy() for rec in trace]
        got = trace_tools.collect(trace, outs)
        assert trace_tools.first_difference(got, want, 1e-4) is None
        session.cache.assert_clean()


# ------------------------------------- toy parts: rotating positions, routing --

@dataclass(frozen=True)
class ToyMixedConfig:
    """A second toy architecture: layer 0 is the framework's attention (2 query
    heads on 1 key/value head, a window) with a rotating position encoding and a
    routed feed-forward that are defined here; layer 1 is the running-mean mixer
    of the first toy with the framework's MLP.  Two cache groups come out of it:
    pages for layer 0, state slots for layer 1."""
    ARCHITECTURE: ClassVar[str] = "ToyMixedLM"
    vocab_size: int = 61
    width: int = 32
    head_dim: int = 16
    experts: int = 3
    window: int = 21
    positions: int = 96

    @classmethod
    def from_dict(cls, values):
        names = ("vocab_size", "width", "head_dim", "experts", "window", "positions")
        return cls(**{k: values[k] for k in names if k in values})

    def to_dict(self):
        return {"architectures": [self.ARCHITECTURE], **{k: getattr(self, k) for k in
                ("vocab_size", "width", "head_dim", "experts", "window", "positions")}}


def register_toy_mixed():
    from ayaka_py_b200.parts import (FeedForward, Init, ModelSpec, PartSpec, PositionEncoding, RunStep,
                                     Source, TensorDecl, pre_norm_layer, register_part)
    from ayaka_py_b200.registry import Architecture, register_architecture
    register_toy()                               # the running-mean mixer

    class TurningPositions(PositionEncoding):
        """No table: queries and keys are turned, pair (2i, 2i+1) of every head by
        the angle position * base^(-i / pairs) (32-bit), in place."""

        def __init__(self, head_dim, base, dtype, device):
            self.head_dim, self.base = head_dim, float(base)

        def tensors(self):
            return {}

        def rotate_qk(self, q, k, heads, kv_heads, head_dim, ctx):
            pairs = head_dim // 2
            freq = self.base ** (-torch.arange(pairs, device=q.device, dtype=torch.float32) / pairs)
            angle = ctx.positions.float()[:, None] * freq[None, :]
            cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            for x, n in ((q, heads), (k, kv_heads)):
                v = x.unflatten(1, (n, head_dim)).float()
                a, b = v[..., 0::2], v[..., 1::2]
                turned = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2)
                x.copy_(turned.flatten(1).to(x.dtype))

    class RoutedFeedForward(FeedForward):
        """Each row goes to the expert its router likes best (32-bit logits): out =
        residual + p_e * tanh(h) * gain_e, p = softmax over the experts."""

        def __init__(self, width, experts, dtype, device):
            self.width, self.experts = width, experts
            self.router = self.gain = None

        def tensors(self):
            return {"router": TensorDecl((self.experts, self.width), "vector"),
                    "gain": TensorDecl((self.experts, self.width), "vector")}

        def forward(self, h, residual, ctx):
            logits = h.float() @ self.router.t()
            p = torch.softmax(logits, dim=-1)
            e = torch.argmax(logits, dim=-1)
            return residual + p.gather(1, e[:, None]) * torch.tanh(h.float()) * self.gain[e]

    register_part("toy_turning_positions", TurningPositions)
    register_part("toy_routed_ffn", RoutedFeedForward)

    def spec(cfg: ToyMixedConfig) -> ModelSpec:
        d, H, Dh = cfg.width, 2, cfg.head_dim
        norm = lambda name: PartSpec("layernorm", {"width": d, "eps": 1e-5},
                                     {"weight": Source(name + ".g", init=Init(0.1, 1.0)), "bias": Source(name + ".b", init=Init(0.1))})
        attention = PartSpec("attention", {"width": d, "num_heads": H, "kv_heads": 1, "head_dim": Dh, "scale": Dh ** -0.5,
                                           "window": cfg.window, "bias": False},
                             {"qkv_weight": Source("l0.qkv", init=Init(0.4)), "out_weight": Source("l0.out", init=Init(0.3))})
        routed = PartSpec("toy_routed_ffn", {"width": d, "experts": cfg.experts},
                          {"router": Source("l0.router", init=Init(0.5)), "gain": Source("l0.gain", init=Init(0.5))})
        mean = PartSpec("toy_running_mean", {"width": d}, {"weight": Source("l1.mix", init=Init(0.3))})
        mlp = PartSpec("mlp", {"width": d, "inner": 40, "activation": "gelu_erf", "bias": True},
                       {"up_weight": Source("l1.up", init=Init(0.3)), "up_bias": Source("l1.up_b", init=Init(0.1)),
                        "down_weight": Source("l1.down", init=Init(0.3)), "down_bias": Source("l1.down_b", init=Init(0.1))})
        layers = (pre_norm_layer(norm("l0.n1"), attention, norm("l0.n2"), routed),
                  pre_norm_layer(norm("l1.n1"), mean, norm("l1.n2"), mlp))
        return ModelSpec(cfg.vocab_size, d, cfg.positions,
                         PartSpec("token_embedding", {"vocab": cfg.vocab_size, "width": d}, {"weight": Source("emb", init=Init(1.0))}),
                         PartSpec("toy_turning_positions", {"head_dim": Dh, "base": 50.0}, {}),
                         layers, (RunStep(0), RunStep(1)), norm("final"),
                         PartSpec("lm_head", {"vocab": cfg.vocab_size, "width": d}, {"weight": Source("head", init=Init(0.3))}))

    register_architecture(Architecture("ToyMixedLM", "toy_mixed", ToyMixedConfig, spec))


def plain_toy_mixed(cfg, t, tokens):
    """Whole sequence, float64, no cache."""
    T, d, H, Dh = len(tokens), cfg.width, 2, cfg.head_dim
    x = t["emb"][tokens]
    # layer 0: windowed attention of 2 heads over one key/value head, turned by position
    h = plain_gpt2.layer_norm(x, t["l0.n1.g"], t["l0.n1.b"], 1e-5)
    qkv = h @ t["l0.qkv"].T
    q, k, v = qkv[:, :H * Dh].reshape(T, H, Dh), qkv[:, H * Dh:H * Dh + Dh], qkv[:, H * Dh + Dh:]
    pairs = Dh // 2
    angle = np.arange(T)[:, None] * 50.0 ** (-np.arange(pairs) / pairs)[None, :]

    def turn(a):                                  # [T, ..., Dh]
        out = np.empty_like(a)
        c, s = np.cos(angle), np.sin(angle)
        if a.ndim == 3:
            c, s = c[:, None, :], s[:, None, :]
        out[..., 0::2] = a[..., 0::2] * c - a[..., 1::2] * s
        out[..., 1::2] = a[..., 0::2] * s + a[..., 1::2] * c
        return out

    q, k = turn(q), turn(k)
    o = np.zeros((T, H, Dh))
    for i in range(T):
        lo = max(0, i - cfg.window + 1)
        for hd in range(H):
            s = k[lo:i + 1] @ q[i, hd] * Dh ** -0.5
            p = np.exp(s - s.max())
            o[i, hd] = (p / p.sum()) @ v[lo:i + 1]
    x = x + o.reshape(T, H * Dh) @ t["l0.out"].T
    h = plain_gpt2.layer_norm(x, t["l0.n2.g"], t["l0.n2.b"], 1e-5)
    logits = h @ t["l0.router"].T
    p = np.exp(logits - logits.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    e = logits.argmax(-1)
    x = x + p[np.arange(T), e][:, None] * np.tanh(h) * t["l0.gain"][e]
    # layer 1: running mean, then the MLP
    h = plain_gpt2.layer_norm(x, t["l1.n1.g"], t["l1.n1.b"], 1e-5)
    x = x + (np.cumsum(h, axis=0) / np.arange(1, T + 1)[:, None]) @ t["l1.mix"].T
    h = plain_gpt2.layer_norm(x, t["l1.n2.g"], t["l1.n2.b"], 1e-5)
    x = x + plain_gpt2.activation("gelu", h @ t["l1.up"].T + t["l1.up_b"]) @ t["l1.down"].T + t["l1.down_b"]
    return plain_gpt2.layer_norm(x, t["final.g"], t["final.b"], 1e-5) @ t["head"].T


def test_toy_positions_routing_and_mixed_layers_without_touching_the_framework(tmp_path):
    """Another position encoding (through the attention part's rotate_qk hook), a
    feed-forward with routing, and layers of different kinds in one model, all
    registered from this file: built, given random weights, and replayed whole,
    in portions and mixed with few pages, against the plain formulas."""
    import trace_tools
    from ayaka_py_b200.parts.base import KVNeed, StateNeed
    from ayaka_py_b200.replay import ReplaySession
    from ayaka_py_b200.weights import write_random_model

    register_toy_mixed()
    cfg = ToyMixedConfig()
    folder = write_random_model(tmp_path / "mixed", cfg, seed=9, dtype="float32")
    tensors = {k: v.astype(np.float64) for k, v in plain_gpt2.read_safetensors(folder / "model.safetensors").items()}
    rs = np.random.RandomState(3)
    reqs = {f"m{i}": rs.randint(0, cfg.vocab_size, n).tolist() for i, n in enumerate([50, 9, 64, 27])}
    want = {rid: plain_toy_mixed(cfg, tensors, toks) for rid, toks in reqs.items()}
    for trace in (trace_tools.whole(reqs), trace_tools.tail_decoded(reqs, tail=8), trace_tools.portions(reqs),
                  trace_tools.mixed(reqs, seed=4)):
        session = ReplaySession(folder, "float32", max_tokens=256, page_size=8)
        needs = sorted(type(g.need).__name__ for g in session.model.groups)
        assert needs == ["KVNeed", "StateNeed"]
        kv = [g.need for g in session.model.groups if isinstance(g.need, KVNeed)][0]
        assert (kv.kv_heads, kv.head_dim, kv.window) == (1, cfg.head_dim, cfg.window)
        outs = [None if (o := session.step(rec)) is None or o.shape[0] == 0 else o.cpu().numpy() for rec in trace]
        got = trace_tools.collect(trace, outs)
        assert trace_tools.first_difference(got, want, 2e-4) is None
        session.cache.assert_clean()


# ------------------------------- toy arrangement: one norm, two parallel branches --

@dataclass(frozen=True)
class ToyParallelConfig:
    """A third toy architecture: every layer has ONE norm whose output feeds the framework's
    attention and the framework's MLP side by side, x += attention(norm(x)) + mlp(norm(x)); the last
    layer has no feed-forward at all.  Only the arrangement is new, and it is defined here."""
    ARCHITECTURE: ClassVar[str] = "ToyParallelLM"
    vocab_size: int = 83
    width: int = 64
    heads: int = 2
    inner: int = 88
    layers: int = 3
    positions: int = 160

    @classmethod
    def from_dict(cls, values):
        names = ("vocab_size", "width", "heads", "inner", "layers", "positions")
        return cls(**{k: values[k] for k in names if k in values})

    def to_dict(self):
        return {"architectures": [self.ARCHITECTURE], **{k: getattr(self, k) for k in
                ("vocab_size", "width", "heads", "inner", "layers", "positions")}}


def register_toy_parallel():
    from ayaka_py_b200.parts import Block, Init, LayerSpec, ModelSpec, PartSpec, RunStep, Source, register_block
    from ayaka_py_b200.registry import Architecture, register_architecture

    class ParallelBlock(Block):
        KIND = "toy_parallel"
        PARTS = ("norm", "mixer", "ffn")

        def forward(self, x, ctx, caches):
            h = self.norm.forward(x, ctx)
            x = self.mixer.forward(h, x, ctx, caches["mixer"])        # x + mix(h), summed in the projection's epilogue
            return self.ffn.forward(h, x, ctx)                         # ... + ffn(h), the same h

    class MixerOnlyBlock(Block):
        KIND = "toy_mixer_only"
        PARTS = ("norm", "mixer")

        def forward(self, x, ctx, caches):
            return self.mixer.forward(self.norm.forward(x, ctx), x, ctx, caches["mixer"])

    register_block(ParallelBlock.KIND, ParallelBlock)
    register_block(MixerOnlyBlock.KIND, MixerOnlyBlock)

    def spec(cfg: ToyParallelConfig) -> ModelSpec:
        d, H = cfg.width, cfg.heads
        Dh = d // H
        norm = lambda name: PartSpec("layernorm", {"width": d, "eps": 1e-5},
                                     {"weight": Source(name + ".g", init=Init(0.1, 1.0)), "bias": Source(name + ".b", init=Init(0.1))})
        layers = []
        for i in range(cfg.layers):
            attention = PartSpec("attention", {"width": d, "num_heads": H, "kv_heads": H, "head_dim": Dh,
                                               "scale": Dh ** -0.5, "window": None, "bias": True},
                                 {"qkv_weight": Source(f"l{i}.qkv", init=Init(0.2)), "qkv_bias": Source(f"l{i}.qkv_b", init=Init(0.1)),
                                  "out_weight": Source(f"l{i}.out", init=Init(0.2)), "out_bias": Source(f"l{i}.out_b", init=Init(0.1))})
            mlp = PartSpec("mlp", {"width": d, "inner": cfg.inner, "activation": "gelu_tanh", "bias": True},
                           {"up_weight": Source(f"l{i}.up", init=Init(0.2)), "up_bias": Source(f"l{i}.up_b", init=Init(0.1)),
                            "down_weight": Source(f"l{i}.down", init=Init(0.2)), "down_bias": Source(f"l{i}.down_b", init=Init(0.1))})
            if i < cfg.layers - 1:
                layers.append(LayerSpec((("norm", norm(f"l{i}.n")), ("mixer", attention), ("ffn", mlp)), "toy_parallel"))
            else:
                layers.append(LayerSpec((("norm", norm(f"l{i}.n")), ("mixer", attention)), "toy_mixer_only"))
        return ModelSpec(cfg.vocab_size, d, cfg.positions,
                         PartSpec("token_embedding", {"vocab": cfg.vocab_size, "width": d}, {"weight": Source("emb", init=Init(1.0))}),
                         PartSpec("learned_positions", {"positions": cfg.positions, "width": d}, {"weight": Source("pos", init=Init(0.5))}),
                         tuple(layers), tuple(RunStep(i) for i in range(cfg.layers)), norm("final"),
                         PartSpec("lm_head", {"vocab": cfg.vocab_size, "width": d}, {"weight": Source("emb", init=Init(1.0))}))

    register_architecture(Architecture("ToyParallelLM", "toy_parallel", ToyParallelConfig, spec))


def plain_toy_parallel(cfg, t, tokens, round_to=None):
    T, d, H = len(tokens), cfg.width, cfg.heads
    Dh = d // H
    x = t["emb"][tokens] + t["pos"][:T]
    for i in range(cfg.layers):
        h = plain_gpt2.layer_norm(x, t[f"l{i}.n.g"], t[f"l{i}.n.b"], 1e-5)
        qkv = h @ t[f"l{i}.qkv"].T + t[f"l{i}.qkv_b"]
        q, k, v = (qkv[:, j * d:(j + 1) * d].reshape(T, H, Dh) for j in range(3))
        o = plain_gpt2.causal_attention(q, k, v, Dh ** -0.5).reshape(T, d)
        branch = o @ t[f"l{i}.out"].T + t[f"l{i}.out_b"]
        if i < cfg.layers - 1:
            branch = branch + plain_gpt2.activation("gelu_new", h @ t[f"l{i}.up"].T + t[f"l{i}.up_b"]) @ t[f"l{i}.down"].T + t[f"l{i}.down_b"]
        x = x + branch
    return plain_gpt2.layer_norm(x, t["final.g"], t["final.b"], 1e-5) @ t["emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_arrangement_one_norm_two_branches_and_a_layer_without_feed_forward(tmp_path, dtype):
    """Two arrangements that are not the framework's (a norm shared by a mixer and a feed-forward that run
    side by side; a layer that is a mixer only), registered from this file with the framework's own parts,
    through the loader, the cache manager, the step function and the replay program, nothing of which
    changes.  In bfloat16 the prompt steps run the tensor-core kernels (head size 32 and width 64)."""
    import trace_tools
    from ayaka_py_b200.replay import ReplaySession
    from ayaka_py_b200.weights import write_random_model

    register_toy_parallel()
    cfg = ToyParallelConfig()
    folder = write_random_model(tmp_path / "parallel", cfg, seed=11, dtype="bfloat16")
    tensors = {k: v.astype(np.float64) for k, v in plain_gpt2.read_safetensors(folder / "model.safetensors").items()}
    rs = np.random.RandomState(7)
    reqs = {f"p{i}": rs.randint(0, cfg.vocab_size, n).tolist() for i, n in enumerate([70, 9, 140, 33])}
    want = {rid: plain_toy_parallel(cfg, tensors, toks) for rid, toks in reqs.items()}
    limit = 2e-4 if dtype == "float32" else 0.02 * max(float(np.abs(w).max()) for w in want.values())
    for trace in (trace_tools.whole(reqs), trace_tools.tail_decoded(reqs, tail=8), trace_tools.mixed(reqs, seed=6)):
        session = ReplaySession(folder, dtype, max_tokens=trace_tools.tokens_needed(trace), page_size=16)
        assert [len(b) for b in session.model.bindings] == [1, 1, 1] and session.model.groups[0].layers == 3
        assert [type(b).KIND for b in session.model.blocks] == ["toy_parallel", "toy_parallel", "toy_mixer_only"]
        outs = [None if (o := session.step(rec)) is None or o.shape[0] == 0 else o.cpu().numpy() for rec in trace]
        got = trace_tools.collect(trace, outs)
        bad = trace_tools.first_difference(got, want, limit)
        assert bad is None, f"first wrong place: request {bad[0]} position {bad[1]} |diff| {bad[2]:.3e}"
        session.cache.assert_clean()
