"""The plain implementation against the stored outputs of the reference's own
model code (tests/golden/make_golden.py made them), and its parts against
direct formulas."""

from pathlib import Path

import numpy as np

import plain_gpt2
import tiny_models

GOLDEN = np.load(Path(__file__).parent / "golden" / "reference_logits.npz")


def test_golden_file_records_agreement():
    assert all(float(GOLDEN[f"{tag}_maxdiff"]) < 1e-5 for tag in "ABE")


def _check(tag, cfg, seed, scale=4.0):
    weights = tiny_models.numpy_weights(cfg, seed, scale=scale, bf16_exact=False)
    tokens = GOLDEN[f"{tag}_tokens"].tolist()
    mine = plain_gpt2.forward(cfg, weights, tokens)
    assert mine.shape == GOLDEN[f"{tag}_logits"].shape
    assert np.abs(mine - GOLDEN[f"{tag}_logits"]).max() < 1e-5


def test_plain_matches_reference_tiny_a():
    _check("A", tiny_models.TINY_A, 11)


def test_plain_matches_reference_tiny_b_inverse_layer_scaling():
    _check("B", tiny_models.TINY_B, 12)


def test_plain_matches_reference_tiny_e_quick_gelu_unscaled_scores_untied_head():
    """The options that A and B leave at their defaults, which the reference accepts
    (``models/gpt2.py:64-66``, ``:147-149``, ``:253-254``)."""
    _check("E", tiny_models.TINY_E, 15, scale=2.0)
    cfg, weights = tiny_models.TINY_E, tiny_models.numpy_weights(tiny_models.TINY_E, 15, scale=2.0, bf16_exact=False)
    tokens = GOLDEN["E_tokens"].tolist()
    tied = plain_gpt2.forward({**cfg, "tie_word_embeddings": True}, weights, tokens)
    scaled = plain_gpt2.forward({**cfg, "scale_attn_weights": True}, weights, tokens)
    gelu = plain_gpt2.forward({**cfg, "activation_function": "gelu_new"}, weights, tokens)
    for other in (tied, scaled, gelu):                         # each option moves the logits: none is ignored
        assert np.abs(other - GOLDEN["E_logits"]).max() > 1e-3


def test_float64_and_float32_agree():
    cfg = tiny_models.TINY_B
    w32 = tiny_models.numpy_weights(cfg, 5, scale=4.0)
    w64 = {k: v.astype(np.float64) for k, v in w32.items()}
    tokens = tiny_models.prompts(cfg, [30], 1)[0]
    assert np.abs(plain_gpt2.forward(cfg, w32, tokens) - plain_gpt2.forward(cfg, w64, tokens)).max() < 2e-5


def test_layer_norm_formula():
    x = np.random.RandomState(0).randn(3, 10).astype(np.float64)
    y = plain_gpt2.layer_norm(x, np.ones(10), np.zeros(10), 1e-5)
    assert np.allclose(y.mean(-1), 0, atol=1e-12)
    assert np.allclose((y * y).mean(-1), x.var(-1) / (x.var(-1) + 1e-5))


def test_attention_is_causal_and_windowed():
    rs = np.random.RandomState(1)
    q, k, v = (rs.randn(6, 2, 4) for _ in range(3))
    full = plain_gpt2.causal_attention(q, k, v, 0.5)
    k2, v2 = k.copy(), v.copy()
    k2[4:], v2[4:] = 9.0, 9.0                      # the future must not matter
    assert np.allclose(full[:4], plain_gpt2.causal_attention(q, k2, v2, 0.5)[:4])
    assert np.allclose(full[0], v[0])              # one visible key
    win = plain_gpt2.causal_attention(q, k, v, 0.5, window=1)
    assert np.allclose(win, v)                     # only the own key is visible


def test_activations():
    x = np.linspace(-3, 3, 13).astype(np.float64)
    assert np.allclose(plain_gpt2.activation("gelu", x)[6], 0.0)
    assert abs(plain_gpt2.activation("gelu", x)[-1] - 3 * 0.9986501019683699) < 1e-12
    assert np.abs(plain_gpt2.activation("gelu_new", x) - plain_gpt2.activation("gelu", x)).max() < 3e-3
    assert np.allclose(plain_gpt2.activation("quick_gelu", x), x / (1 + np.exp(-1.702 * x)))


def test_philox_known_answers():
    # Random123 known-answer vectors for philox4x32-10.
    assert plain_gpt2.philox4x32_10((0, 0, 0, 0), (0, 0)) == (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)
    assert plain_gpt2.philox4x32_10((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2) == (
        0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)
    assert plain_gpt2.philox4x32_10((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344),
                                    (0xA4093822, 0x299F31D0)) == (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)
    u = [plain_gpt2.philox_uniform(7, i) for i in range(1000)]
    assert 0 <= min(u) and max(u) < 1 and abs(np.mean(u) - 0.5) < 0.05


def test_sampling_twin_distribution():
    logits = np.array([0.0, 1.0, 2.0, -1.0])
    p = plain_gpt2.filtered_probabilities(logits, 1.0)
    draws = [plain_gpt2.sample_token(logits, 1.0, 123, i) for i in range(4000)]
    freq = np.bincount(draws, minlength=4) / 4000
    assert np.abs(freq - p).max() < 0.03
    assert plain_gpt2.sample_token(logits, 0.0, 1, 0) == 2
    assert set(plain_gpt2.sample_token(logits, 1.0, 5, i, top_k=2) for i in range(200)) <= {1, 2}
    p_top = plain_gpt2.filtered_probabilities(logits, 1.0, top_p=0.6)
    assert p_top[2] > 0 and p_top[3] == 0 and abs(p_top.sum() - 1) < 1e-12
