"""Each kernel alone against a plain reference, at other sizes than the engine's."""

import numpy as np
import pytest
import torch

import plain_gpt2

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == "float32" else 2e-2) * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(0)
    wte, wpe = rs.randn(301, 72).astype(np.float32), rs.randn(50, 72).astype(np.float32)
    tok, pos = rs.randint(0, 301, 23).astype(np.int32), rs.randint(0, 50, 23).astype(np.int32)
    a, b = dev(wte, DTYPES[dtype]), dev(wpe, DTYPES[dtype])
    out = ops.embed(dev(tok), dev(pos), a, b).cpu().numpy()
    want = a.float().cpu().numpy()[tok] + b.float().cpu().numpy()[pos]
    assert np.abs(out - want).max() < 1e-6
    only = ops.embed(dev(tok), dev(pos), a, None).cpu().numpy()
    assert np.array_equal(only, a.float().cpu().numpy()[tok])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,eps", [(72, 1e-5), (1600, 1e-6), (1000, 3e-2), (8, 1e-5), (2050, 1e-5), (4096, 1e-5), (2048, 1e-5)])
def test_layernorm(dtype, width, eps):
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(1)
    x = (rs.randn(19, width) * 3 + 1.5).astype(np.float32)
    g, b = rs.randn(width).astype(np.float32), rs.randn(width).astype(np.float32)
    want = plain_gpt2.layer_norm(x.astype(np.float64), g, b, eps)
    out = ops.layernorm(dev(x), dev(g), dev(b), eps, DTYPES[dtype]).float().cpu().numpy()
    assert np.abs(out - want).max() < tol(dtype, 4.0)
    rows = np.array([18, 0, 7], dtype=np.int32)
    picked = ops.layernorm(dev(x), dev(g), dev(b), eps, DTYPES[dtype], rows=dev(rows)).float().cpu().numpy()
    assert np.abs(picked - want[rows]).max() < tol(dtype, 4.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 50, 24), (7, 257, 1000), (130, 96, 72), (64, 64, 16), (33, 1003, 330)])
@pytest.mark.parametrize("act", ["none", "gelu_tanh", "gelu_erf", "quick_gelu"])
def test_gemm_simt(dtype, M, N, K, act):
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(2)
    a, w = rs.randn(M, K).astype(np.float32), (rs.randn(N, K) / np.sqrt(K)).astype(np.float32)
    bias, res = rs.randn(N).astype(np.float32), rs.randn(M, N).astype(np.float32)
    A, W = dev(a, DTYPES[dtype]), dev(w, DTYPES[dtype])
    a64, w64 = A.double().cpu().numpy(), W.double().cpu().numpy()
    names = {"none": None, "gelu_tanh": "gelu_new", "gelu_erf": "gelu", "quick_gelu": "quick_gelu"}
    y = a64 @ w64.T + bias
    if names[act]:
        y = plain_gpt2.activation(names[act], y)
    want = y + res
    out = ops.gemm_simt(A, W, dev(bias), act, dev(res), out_dtype=torch.float32).cpu().numpy()
    assert np.abs(out - want).max() < 2e-5
    plain = ops.gemm_simt(A, W, None, "none", None).float().cpu().numpy()
    assert np.abs(plain - a64 @ w64.T).max() < tol(dtype, 4.0)
    R = dev(res)
    ops.gemm_simt(A, W, dev(bias), act, R, out_dtype=torch.float32, out=R)        # in place on the residual
    assert np.abs(R.cpu().numpy() - want).max() < 2e-5


def paged_case(rs, lens_q, lens_ctx, H, Hkv, Dh, P, dtype, pages=None, sharp=None):
    """Random requests: request r brings lens_q[r] rows after lens_ctx[r] cached
    tokens.  Returns kernel inputs and the plain result."""
    R = len(lens_q)
    total = [c + q for c, q in zip(lens_ctx, lens_q)]
    C = max(-(-t // P) for t in total)
    n_pages = pages or (sum(-(-t // P) for t in total) + 1)
    order = rs.permutation(np.arange(1, n_pages))
    table = np.zeros((R, C), dtype=np.int32)
    kc = rs.randn(n_pages, P, Hkv, Dh).astype(np.float32)     # garbage where nothing lives
    vc = rs.randn(n_pages, P, Hkv, Dh).astype(np.float32)
    qs, ks, vs, rows, k_new, v_new, pos, row_req = [], [], [], [], [], [], [], []
    used = 0
    for r in range(R):
        T = total[r]
        q = rs.randn(T, H, Dh).astype(np.float32)
        k = rs.randn(T, Hkv, Dh).astype(np.float32)
        v = rs.randn(T, Hkv, Dh).astype(np.float32)
        if sharp is not None and r == sharp[0]:
            _, qpos, kpos = sharp                 # one far key stands out for one query
            for hh in range(H):
                key = k[kpos, hh // (H // Hkv)]
                q[qpos, hh] = key * (30.0 / float(key @ key))
        qs.append(q); ks.append(k); vs.append(v)
        for j in range(-(-T // P)):
            table[r, j] = order[used]; used += 1
        for p in range(lens_ctx[r]):              # the cached prefix is in the pages already
            kc[table[r, p // P], p % P] = k[p]
            vc[table[r, p // P], p % P] = v[p]
        for p in range(lens_ctx[r], T):
            rows.append(q[p].reshape(-1)); k_new.append(k[p].reshape(-1)); v_new.append(v[p].reshape(-1))
            pos.append(p); row_req.append(r)
    q_start = np.concatenate([[0], np.cumsum(lens_q)]).astype(np.int32)
    t = DTYPES[dtype]
    inputs = dict(q=dev(np.stack(rows), t), k=dev(np.stack(k_new), t), v=dev(np.stack(v_new), t),
                  kc=dev(kc, t), vc=dev(vc, t), table=dev(table), q_start=dev(q_start),
                  pos0=dev(np.asarray(lens_ctx, dtype=np.int32)), pos=dev(np.asarray(pos, dtype=np.int32)),
                  row_req=dev(np.asarray(row_req, dtype=np.int32)))

    def rounded(a):
        return dev(a, t).double().cpu().numpy()

    def plain(scale, window):
        out = []
        for r in range(R):
            kk = np.repeat(rounded(ks[r]), H // Hkv, axis=1)
            vv = np.repeat(rounded(vs[r]), H // Hkv, axis=1)
            o = plain_gpt2.causal_attention(rounded(qs[r]), kk, vv, scale, window=window)
            out.append(o[lens_ctx[r]:].reshape(lens_q[r], H * Dh))
        return np.concatenate(out)

    return inputs, plain


ATTENTION_CASES = [
    # lens_q, lens_ctx, H, Hkv, Dh, P, window
    ([5, 1, 40], [0, 17, 3], 4, 4, 16, 16, None),
    ([1, 1, 1, 1], [0, 15, 16, 130], 2, 2, 48, 8, None),
    ([33, 2, 64], [31, 0, 65], 6, 2, 80, 16, None),        # grouped queries, head size 80
    ([70], [200], 1, 1, 256, 32, None),
    ([9, 1, 50], [40, 99, 0], 4, 2, 32, 4, 24),            # window
    ([1, 3], [63, 64], 5, 5, 64, 64, 7),
    ([7, 1, 35], [0, 40, 3], 3, 3, 20, 8, None),           # head sizes that are no multiple of 16, of 4, of 2
    ([40, 2], [0, 70], 4, 2, 36, 16, 30),
    ([33, 1], [5, 64], 6, 3, 5, 4, None),
    ([1, 1, 9], [99, 0, 12], 2, 2, 6, 16, None),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ATTENTION_CASES)
def test_append_then_attention(dtype, case):
    from ayaka_py_b200 import ops
    lens_q, lens_ctx, H, Hkv, Dh, P, window = case
    rs = np.random.RandomState(3)
    x, plain = paged_case(rs, lens_q, lens_ctx, H, Hkv, Dh, P, dtype)
    scale = 0.7 / np.sqrt(Dh)
    ops.kv_append(x["kc"], x["vc"], x["k"], x["v"], x["row_req"], x["pos"], x["table"])
    out = ops.attention_simt(x["q"], x["kc"], x["vc"], x["table"], x["q_start"], x["pos0"], sum(lens_q), H,
                             scale, window).float().cpu().numpy()
    assert np.abs(out - plain(scale, window)).max() < tol(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("qpos,kpos", [(299, 0), (299, 15), (299, 16), (255, 127), (256, 128)])
def test_far_key_stands_out(dtype, qpos, kpos):
    """One query's score for one far key (at a page's edge) is made large, so
    that losing that key changes the result by far more than the tolerance."""
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(4)
    x, plain = paged_case(rs, [300, 1], [0, 20], 2, 2, 32, 16, dtype, sharp=(0, qpos, kpos))
    ops.kv_append(x["kc"], x["vc"], x["k"], x["v"], x["row_req"], x["pos"], x["table"])
    out = ops.attention_simt(x["q"], x["kc"], x["vc"], x["table"], x["q_start"], x["pos0"], 301, 2, 1.0).float().cpu().numpy()
    want = plain(1.0, None)
    uniform = plain(0.0, None)
    assert np.abs(want[qpos] - uniform[qpos]).max() > 0.5      # the far key matters
    assert np.abs(out - want).max() < tol(dtype)


def test_greedy_ties_take_the_lowest_index():
    from ayaka_py_b200 import ops
    logits = np.zeros((3, 1000), dtype=np.float32)
    logits[0, [700, 12, 999]] = 5.0
    logits[1, 999] = 1.0
    logits[2] = -np.inf
    out = ops.sample(dev(logits)).cpu().numpy()
    assert out.tolist() == [12, 999, 0]


def test_temperature_draws_fall_in_the_twins_interval_and_are_batch_independent():
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(5)
    V, S = 1237, 64
    logits = (rs.randn(S, V) * 2).astype(np.float32)
    temp = np.full(S, 0.8, dtype=np.float32)
    temp[5] = 0.0
    seed = rs.randint(0, 2 ** 62, S).astype(np.int64)
    offset = rs.randint(0, 1000, S).astype(np.int64)
    out = ops.sample(dev(logits), dev(temp), dev(seed), dev(offset)).cpu().numpy()
    for r in range(S):
        if temp[r] == 0:
            assert out[r] == int(np.argmax(logits[r]))
            continue
        p = plain_gpt2.filtered_probabilities(logits[r], temp[r])
        cum = np.cumsum(p)
        u = plain_gpt2.philox_uniform(int(seed[r]), int(offset[r]))
        lo = cum[out[r] - 1] if out[r] > 0 else 0.0
        assert lo - 1e-5 <= u <= cum[out[r]] + 1e-5, (r, out[r], lo, u, cum[out[r]])
    alone = ops.sample(dev(logits[9:10]), dev(temp[9:10]), dev(seed[9:10]), dev(offset[9:10])).cpu().numpy()
    assert alone[0] == out[9]


def test_filters_that_keep_the_maximum_only():
    """min_p = 1 and top_k = 1 leave the most likely token alone, whatever the temperature: the
    maximum's own weight exp(z - zmax) has to come out as 1 exactly (with logit / T and the
    subtraction fused it came out as 1 +- 4e-6, and nothing or the wrong token was kept).  A row
    without a finite logit gives token 0, as greedy does."""
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(12)
    for V in (11, 1971, 50257):
        S = 48
        logits = (rs.randn(S, V) * 6).astype(np.float32)
        logits[7] = -np.inf
        temp = rs.choice([0.3, 0.8, 1.7], size=S).astype(np.float32)
        seed = rs.randint(0, 2 ** 62, S).astype(np.int64)
        offset = rs.randint(0, 5000, S).astype(np.int64)
        want = np.argmax(logits, axis=1)
        want[7] = 0
        ones = np.ones(S, dtype=np.float32)
        only_max = ops.sample(dev(logits), dev(temp), dev(seed), dev(offset), None, None, dev(ones)).cpu().numpy()
        assert only_max.tolist() == want.tolist()
        top_one = ops.sample(dev(logits), dev(temp), dev(seed), dev(offset), dev(np.ones(S, dtype=np.int64)), None, None).cpu().numpy()
        assert top_one.tolist() == want.tolist()
        tiny_nucleus = ops.sample(dev(logits), dev(temp), dev(seed), dev(offset), None, dev(np.full(S, 1e-6, dtype=np.float32)), None)
        assert tiny_nucleus.cpu().numpy().tolist() == want.tolist()


def test_temperature_distribution():
    from ayaka_py_b200 import ops
    logits = np.tile(np.array([[0.0, 1.0, 2.0, -1.0, 0.5]], dtype=np.float32), (20000, 1))
    n = logits.shape[0]
    out = ops.sample(dev(logits), dev(np.full(n, 1.3, dtype=np.float32)), dev(np.full(n, 77, dtype=np.int64)),
                     dev(np.arange(n, dtype=np.int64))).cpu().numpy()
    p = plain_gpt2.filtered_probabilities(logits[0], 1.3)
    freq = np.bincount(out, minlength=5) / n
    chi2 = float((n * (freq - p) ** 2 / p).sum())
    assert chi2 < 18.5        # 4 degrees of freedom, p = 0.001


def test_kernels_refuse_what_they_cannot_do():
    from ayaka_py_b200 import ops
    with pytest.raises(ops.KernelError):
        ops.layernorm(torch.zeros(2, 20000, device="cuda"), torch.ones(20000, device="cuda"), None, 1e-5, torch.float32)
    with pytest.raises(ops.KernelError):
        ops.gemm_simt(torch.zeros(2, 8, device="cuda"), torch.zeros(3, 9, device="cuda"))
    with pytest.raises(ops.KernelError):
        ops.embed(torch.zeros(2, dtype=torch.int64, device="cuda"), torch.zeros(2, dtype=torch.int32, device="cuda"),
                  torch.zeros(4, 4, device="cuda"), None)


TC_CASES = [
    # M, N, K, splits
    (1, 128, 64, 1), (5, 50, 72, 1), (16, 257, 200, 1), (17, 384, 1000, 1), (64, 96, 320, 1),
    (100, 1003, 328, 1), (300, 200, 1600, 1), (8, 1600, 1600, None), (64, 1600, 6400, None),
    (3, 130, 512, 4), (40, 300, 1000, 7), (8, 64, 64, 3),
    (16, 300, 1600, 8), (1, 1600, 6400, 2), (5, 257, 520, 8), (9, 50257 // 16, 128, 2),      # splits as one cluster
    (64, 1600, 6400, 8), (33, 4800, 1600, 4), (17, 200, 328, 2), (32, 130, 256, 4), (50, 6400, 1600, 2),
    (8, 1600, 6400, 16), (1, 300, 1104, 16), (24, 257, 2048, 16), (64, 1000, 4104, 16),         # clusters of 16
]


@pytest.mark.parametrize("M,N,K,splits", TC_CASES)
@pytest.mark.parametrize("act,out_dtype", [("none", "float32"), ("gelu_tanh", "bfloat16")])
def test_gemm_tcgen05(M, N, K, splits, act, out_dtype):
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(6)
    a, w = rs.randn(M, K).astype(np.float32), (rs.randn(N, K) / np.sqrt(K)).astype(np.float32)
    bias, res = rs.randn(N).astype(np.float32), rs.randn(M, N).astype(np.float32)
    A, W = dev(a, torch.bfloat16), dev(w, torch.bfloat16)
    y = A.double().cpu().numpy() @ W.double().cpu().numpy().T + bias
    if act != "none":
        y = plain_gpt2.activation("gelu_new", y)
    want = y + res
    out = ops.gemm_tc(A, W, dev(bias), act, dev(res), out_dtype=DTYPES[out_dtype], splits=splits, static_weight=False)
    torch.cuda.synchronize()
    assert ops.tc_error() == 0
    err = np.abs(out.float().cpu().numpy() - want).max()
    # The tensor core adds K products of ~unit size in 32-bit: the rounding error grows like sqrt(K).
    assert err < (2e-5 * max(1.0, K / 1600.0) ** 0.5 if out_dtype == "float32" else 4e-2), err
    if out_dtype == "float32":
        R = dev(res)
        again = ops.gemm_tc(A, W, dev(bias), act, R, out_dtype=torch.float32, out=R, splits=splits, static_weight=False)
        assert torch.equal(again, out)                      # in place on the residual, and the same bits again
        assert ops.tc_error() == 0


def test_gemm_tcgen05_rows_do_not_depend_on_the_batch():
    """A row's result is the same alone, among 7 and among 200 rows (same split)."""
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(7)
    a, w = rs.randn(200, 640).astype(np.float32), rs.randn(320, 640).astype(np.float32) / 25
    A, W = dev(a, torch.bfloat16), dev(w, torch.bfloat16)
    full = ops.gemm_tc(A, W, out_dtype=torch.float32, splits=1)
    for m in (1, 7, 64):
        part = ops.gemm_tc(A[:m].contiguous(), W, out_dtype=torch.float32, splits=1)
        assert torch.equal(part, full[:m])
    assert ops.tc_error() == 0


def test_gemm_tcgen05_refuses_odd_k():
    from ayaka_py_b200 import ops
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.gemm_tc(torch.zeros(2, 12, device="cuda", dtype=torch.bfloat16), torch.zeros(4, 12, device="cuda", dtype=torch.bfloat16))
    out = ops.linear(torch.ones(2, 12, device="cuda", dtype=torch.bfloat16), torch.ones(4, 12, device="cuda", dtype=torch.bfloat16))
    assert float(out.float().max()) == 12.0      # the dispatcher takes the FP32-pipe kernel instead


DECODE_CASES = [
    # contexts (tokens cached before the row), H, Hkv, Dh, P, window
    ([0, 17, 127, 128, 300], 4, 4, 64, 16, None),
    ([5, 255, 256, 640], 25, 25, 64, 16, None),
    ([1, 129, 400], 6, 2, 48, 8, None),
    ([700], 2, 1, 256, 32, None),
    ([3, 130, 500], 4, 2, 32, 16, 40),
    ([63, 64, 200], 5, 5, 16, 64, 129),
    ([9, 200, 333], 20, 2, 128, 4, None),      # groups of 10 heads: two passes of rows; small pages
    ([150, 31, 0], 8, 1, 64, 64, 70),          # 8 heads on one key/value head; a page larger than a warp's keys
    ([1000, 513], 3, 3, 32, 32, None),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", DECODE_CASES)
@pytest.mark.parametrize("max_context", [1024, 2048], ids=["8_parts", "16_parts"])
def test_decode_attention_split_and_merge(dtype, case, max_context):
    from ayaka_py_b200 import ops
    ctxs, H, Hkv, Dh, P, window = case
    rs = np.random.RandomState(8)
    x, plain = paged_case(rs, [1] * len(ctxs), ctxs, H, Hkv, Dh, P, dtype)
    scale = 1.3 / np.sqrt(Dh)
    kc2, vc2 = x["kc"].clone(), x["vc"].clone()
    ops.kv_append(x["kc"], x["vc"], x["k"], x["v"], x["row_req"], x["pos"], x["table"])
    out = ops.attention_decode(x["q"], x["kc"], x["vc"], x["table"], x["pos0"], H, scale, window, max_context)
    assert np.abs(out.float().cpu().numpy() - plain(scale, window)).max() < tol(dtype)
    general = ops.attention_simt(x["q"], x["kc"], x["vc"], x["table"], x["q_start"], x["pos0"], len(ctxs), H, scale, window)
    assert np.abs(out.float().cpu().numpy() - general.float().cpu().numpy()).max() < tol(dtype)
    # the same with the step's keys and values filed by the attention call itself
    fused = ops.attention_decode(x["q"], kc2, vc2, x["table"], x["pos0"], H, scale, window, max_context,
                                 append=(x["k"], x["v"], x["row_req"]))
    assert torch.equal(fused, out)
    assert torch.equal(kc2, x["kc"]) and torch.equal(vc2, x["vc"])
    # the same when the caller vouches that the rows of earlier steps are complete (they are: nothing
    # that wrote them is still running), so that their copies may start before the kernel's wait
    torch.cuda.synchronize()
    kc3, vc3 = x["kc"].clone(), x["vc"].clone()
    early = ops.attention_decode(x["q"], kc3, vc3, x["table"], x["pos0"], H, scale, window, max_context,
                                 append=(x["k"], x["v"], x["row_req"]), settled=True)
    assert torch.equal(early, out)
    assert torch.equal(ops.attention_decode(x["q"], kc3, vc3, x["table"], x["pos0"], H, scale, window, max_context,
                                            settled=True), out)


@pytest.mark.parametrize("kpos", [0, 127, 128, 383, 384])
def test_decode_attention_far_key_at_a_partition_edge(kpos):
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(9)
    x, plain = paged_case(rs, [1, 1], [500, 9], 2, 2, 64, 16, "bfloat16", sharp=(0, 500, kpos))
    ops.kv_append(x["kc"], x["vc"], x["k"], x["v"], x["row_req"], x["pos"], x["table"])
    out = ops.attention_decode(x["q"], x["kc"], x["vc"], x["table"], x["pos0"], 2, 1.0, None, 1024).float().cpu().numpy()
    want = plain(1.0, None)
    assert np.abs(want[0] - plain(0.0, None)[0]).max() > 0.5
    assert np.abs(out - want).max() < tol("bfloat16")


TC_ATTENTION_CASES = [
    # lens_q, lens_ctx, H, Hkv, P, window
    ([5, 1, 40], [0, 17, 3], 2, 2, 16, None),
    ([128, 129, 1], [0, 0, 300], 3, 3, 16, None),
    ([300], [0], 2, 1, 8, None),
    ([70, 200], [250, 57], 4, 2, 64, None),
    ([33, 260], [100, 0], 2, 2, 128, None),
    ([150, 9], [140, 300], 2, 2, 16, 100),
    # 40 requests (two groups of 32 in the kernel's search for its tile), tiles of very different length
    ([3] * 20 + [130, 260] + [5] * 17 + [129], [0] * 20 + [40, 0] + [7] * 17 + [200], 2, 1, 16, None),
]


@pytest.mark.parametrize("case", TC_ATTENTION_CASES)
def test_attention_tcgen05(case):
    from ayaka_py_b200 import ops
    lens_q, lens_ctx, H, Hkv, P, window = case
    rs = np.random.RandomState(10)
    x, plain = paged_case(rs, lens_q, lens_ctx, H, Hkv, 64, P, "bfloat16")
    scale = 0.9 / 8.0
    ops.kv_append(x["kc"], x["vc"], x["k"], x["v"], x["row_req"], x["pos"], x["table"])
    assert ops.attention_tc_takes(x["q"], x["kc"])
    out = ops.attention_tc(x["q"], x["kc"], x["vc"], x["table"], x["q_start"], x["pos0"], sum(lens_q), H, scale, window)
    torch.cuda.synchronize()
    assert ops.tc_error() == 0
    assert np.abs(out.float().cpu().numpy() - plain(scale, window)).max() < tol("bfloat16")


@pytest.mark.parametrize("qpos,kpos", [(299, 0), (299, 127), (299, 128), (255, 15), (256, 16), (130, 129)])
def test_attention_tcgen05_far_key_stands_out(qpos, kpos):
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(11)
    x, plain = paged_case(rs, [300, 2], [0, 20], 2, 2, 64, 16, "bfloat16", sharp=(0, qpos, kpos))
    ops.kv_append(x["kc"], x["vc"], x["k"], x["v"], x["row_req"], x["pos"], x["table"])
    out = ops.attention_tc(x["q"], x["kc"], x["vc"], x["table"], x["q_start"], x["pos0"], 302, 2, 1.0).float().cpu().numpy()
    torch.cuda.synchronize()
    assert ops.tc_error() == 0
    want = plain(1.0, None)
    assert np.abs(want[qpos] - plain(0.0, None)[qpos]).max() > 0.5
    assert np.abs(out - want).max() < tol("bfloat16")


PREFILL_GEMM_CASES = [
    # M, N, K, tile_n (0: chosen by the library)
    (129, 64, 64, 0), (300, 200, 1600, 0), (2048, 1600, 1600, 0), (2048, 4800, 1600, 192), (1000, 1003, 328, 96),
    (513, 6400, 256, 256), (640, 1600, 6400, 128), (257, 330, 72, 160), (4096, 264, 192, 64), (150, 1000, 1000, 224),
]


@pytest.mark.parametrize("pair", [False, True], ids=["one_sm", "two_sms"])
@pytest.mark.parametrize("lens_q,lens_ctx,H,Hkv,Dh,P,K,tile_n", [
    ([130, 7, 200], [0, 50, 13], 4, 4, 64, 16, 256, 0),       # q | k | v of 256 columns each
    ([300], [5], 6, 2, 32, 8, 136, 96),                       # grouped heads: 192 | 64 | 64, tiles that straddle the parts
    ([129, 140], [0, 0], 3, 1, 24, 16, 64, 64),               # 72 | 24 | 24 = 120 columns: a ragged last chunk
])
def test_gemm_prefill_files_keys_and_values(lens_q, lens_ctx, H, Hkv, Dh, P, K, tile_n, pair):
    """The many-row product as a q | k | v projection that also stores the key and value columns into
    the paged cache: the same output as without, and the same cache as the append kernel leaves."""
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(21)
    x, _ = paged_case(rs, lens_q, lens_ctx, H, Hkv, Dh, P, "bfloat16")
    T, qw, kvw = sum(lens_q), H * Dh, Hkv * Dh
    N = qw + 2 * kvw
    a = dev(rs.randn(T, K).astype(np.float32), torch.bfloat16)
    w = dev((rs.randn(N, K) / np.sqrt(K)).astype(np.float32), torch.bfloat16)
    bias = dev(rs.randn(N).astype(np.float32))
    plain_out = ops.gemm_tc_prefill(a, w, bias, out_dtype=torch.bfloat16, tile_n=tile_n, pair=pair)
    kc1, vc1 = x["kc"].clone(), x["vc"].clone()
    ops.kv_append(kc1, vc1, plain_out[:, qw:qw + kvw], plain_out[:, qw + kvw:], x["row_req"], x["pos"], x["table"])
    kc2, vc2 = x["kc"].clone(), x["vc"].clone()
    filing = ops.KVAppend(kc2, vc2, x["row_req"], x["pos"], x["table"], qw, kvw)
    out = ops.gemm_tc_prefill(a, w, bias, out_dtype=torch.bfloat16, tile_n=tile_n, pair=pair, kv=filing)
    torch.cuda.synchronize()
    assert ops.tc_error() == 0 and filing.done
    assert torch.equal(out, plain_out)
    assert torch.equal(kc2, kc1) and torch.equal(vc2, vc1)
    assert not torch.equal(kc2, x["kc"])
    # through the dispatcher, which takes this path for many rows
    kc3, vc3 = x["kc"].clone(), x["vc"].clone()
    filing = ops.KVAppend(kc3, vc3, x["row_req"], x["pos"], x["table"], qw, kvw)
    again = ops.linear(a, w, bias, out_dtype=torch.bfloat16, kv=filing)
    if filing.done:
        assert torch.equal(kc3, kc1) and torch.equal(vc3, vc1)
    assert filing.done == (T > ops.PREFILL_ROWS)      # the dispatcher takes the filing product for many rows
    assert torch.equal(again, plain_out)


@pytest.mark.parametrize("M,N,K,tile_n", PREFILL_GEMM_CASES)
@pytest.mark.parametrize("act,out_dtype", [("none", "float32"), ("gelu_tanh", "bfloat16")])
@pytest.mark.parametrize("pair", [False, True], ids=["one_sm", "two_sms"])
def test_gemm_tcgen05_many_rows(M, N, K, tile_n, act, out_dtype, pair):
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(12)
    a, w = rs.randn(M, K).astype(np.float32), (rs.randn(N, K) / np.sqrt(K)).astype(np.float32)
    bias, res = rs.randn(N).astype(np.float32), rs.randn(M, N).astype(np.float32)
    A, W = dev(a, torch.bfloat16), dev(w, torch.bfloat16)
    y = (A.float() @ W.float().t()).double().cpu().numpy() + bias            # float32 products are exact for bf16 operands
    if act != "none":
        y = plain_gpt2.activation("gelu_new", y)
    want = y + res
    R = dev(res)
    out = ops.gemm_tc_prefill(A, W, dev(bias), act, R, out_dtype=DTYPES[out_dtype], tile_n=tile_n, pair=pair)
    torch.cuda.synchronize()
    assert ops.tc_error() == 0
    err = np.abs(out.float().cpu().numpy() - want).max()
    assert err < (1e-3 if out_dtype == "float32" else 5e-2), err
    if out_dtype == "float32":
        again = ops.gemm_tc_prefill(A, W, dev(bias), act, R, out_dtype=torch.float32, out=R, tile_n=tile_n, pair=pair)   # in place
        assert torch.equal(again, out) and ops.tc_error() == 0
        few = ops.gemm_tc(A[:64].contiguous(), W, dev(bias), act, dev(res[:64]), out_dtype=torch.float32, splits=1)
        assert float((few - out[:64]).abs().max()) < 1e-4                     # the few-row kernel agrees


SPLIT_GEMM_CASES = [
    # M, N, K, tile_n, parts: the tiles' clusters all run at once, the tile width is a multiple of 16 * parts
    (128, 1600, 6400, 128, 8), (300, 200, 1600, 64, 4), (130, 328, 1000, 96, 2), (512, 1600, 6400, 256, 4),
    (129, 72, 4096, 32, 2), (1024, 264, 712, 128, 2), (200, 768, 3072, 128, 8), (70, 1600, 6400, 128, 8), (17, 64, 512, 64, 4),
    (1024, 1600, 6400, 192, 2),
]


@pytest.mark.parametrize("M,N,K,tile_n,parts", SPLIT_GEMM_CASES)
@pytest.mark.parametrize("act,out_dtype", [("none", "float32"), ("gelu_tanh", "bfloat16")])
def test_gemm_tcgen05_many_rows_split_along_k(M, N, K, tile_n, parts, act, out_dtype):
    """The many-row product with the K blocks of a tile split over a cluster of 2, 4 or 8 CTAs (sums
    exchanged through shared memory, each CTA finishing its share of the columns): the plain float32
    product, the unsplit kernel to rounding of the sums, the same bits in a second run (sums added in a
    fixed order), in place over the residual, and the library's own choice."""
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(31)
    a, w = rs.randn(M, K).astype(np.float32), (rs.randn(N, K) / np.sqrt(K)).astype(np.float32)
    bias, res = rs.randn(N).astype(np.float32), rs.randn(M, N).astype(np.float32)
    A, W = dev(a, torch.bfloat16), dev(w, torch.bfloat16)
    y = (A.float() @ W.float().t()).double().cpu().numpy() + bias
    if act != "none":
        y = plain_gpt2.activation("gelu_new", y)
    want = y + res
    R = dev(res)
    try:
        ops.set_split(0)
        whole = ops.gemm_tc_prefill(A, W, dev(bias), act, R, out_dtype=DTYPES[out_dtype], tile_n=tile_n, pair=False)
        ops.set_split(parts)
        before = ops.launches
        out = ops.gemm_tc_prefill(A, W, dev(bias), act, R, out_dtype=DTYPES[out_dtype], tile_n=tile_n, pair=False)
        assert ops.last_split() == parts
        again = ops.gemm_tc_prefill(A, W, dev(bias), act, R, out_dtype=DTYPES[out_dtype], tile_n=tile_n, pair=False)
        assert ops.launches == before + 2
        torch.cuda.synchronize()
        assert ops.tc_error() == 0
        err = np.abs(out.float().cpu().numpy() - want).max()
        assert err < (1e-3 if out_dtype == "float32" else 5e-2), err
        assert torch.equal(out, again)
        assert float((out.float() - whole.float()).abs().max()) < (1e-4 if out_dtype == "float32" else 5e-2)
        if out_dtype == "float32":
            R2 = dev(res)
            in_place = ops.gemm_tc_prefill(A, W, dev(bias), act, R2, out_dtype=torch.float32, out=R2, tile_n=tile_n, pair=False)
            assert torch.equal(in_place, out)
        ops.set_split(None)
        chosen = ops.gemm_tc_prefill(A, W, dev(bias), act, R, out_dtype=DTYPES[out_dtype], pair=False)
        torch.cuda.synchronize()
        assert ops.tc_error() == 0
        assert np.abs(chosen.float().cpu().numpy() - want).max() < (1e-3 if out_dtype == "float32" else 5e-2)
    finally:
        ops.set_split(None)


@pytest.mark.parametrize("M,N,K,tile_n", [(2048, 1600, 1600, 192), (640, 1600, 6400, 128), (300, 1000, 328, 64),
                                          (129, 72, 64, 64), (1000, 1608, 712, 192), (131, 6400, 128, 128)])
@pytest.mark.parametrize("in_place", [False, True], ids=["apart", "in_place"])
def test_gemm_tcgen05_many_rows_staged_residual(M, N, K, tile_n, in_place):
    """The residual epilogue through shared memory by TMA (rows that end inside a tile, columns that end inside
    a chunk, the residual apart from the output or the output itself): the same bits as the epilogue in which
    a thread owns a row, and the plain float32 product."""
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(41)
    a, w = rs.randn(M, K).astype(np.float32), (rs.randn(N, K) / np.sqrt(K)).astype(np.float32)
    bias, res = rs.randn(N).astype(np.float32), rs.randn(M, N).astype(np.float32)
    A, W = dev(a, torch.bfloat16), dev(w, torch.bfloat16)
    want = (A.float() @ W.float().t()).double().cpu().numpy() + bias + res
    try:
        ops.set_split(0)
        outs = []
        for staged in (False, True):
            ops.set_staged(staged)
            R = dev(res)
            out = ops.gemm_tc_prefill(A, W, dev(bias), "none", R, out_dtype=torch.float32, out=R if in_place else None,
                                      tile_n=tile_n, pair=False)
            torch.cuda.synchronize()
            assert ops.tc_error() == 0
            assert in_place or torch.equal(R, dev(res))        # the residual is only read
            assert (ops.last_staged() > 0) == (staged and M >= 128)
            outs.append(out.clone())
        assert np.abs(outs[1].cpu().numpy() - want).max() < 1e-3
        assert torch.equal(outs[0], outs[1])
    finally:
        ops.set_staged(True)
        ops.set_split(None)


@pytest.mark.parametrize("M,N,K,tile_n", [(200, 50257, 64, 0), (129, 331, 72, 96), (1000, 1003, 328, 160), (65, 77, 200, 32),
                                          (300, 4802, 1600, 0)])
@pytest.mark.parametrize("act,out_dtype", [("none", "float32"), ("gelu_tanh", "bfloat16")])
def test_gemm_tcgen05_many_rows_of_odd_width(M, N, K, tile_n, act, out_dtype):
    """Output rows that are no whole 16-byte pieces (an LM head's 50,257 columns) and no residual: the epilogue
    that turns a warp's 32 x 32 block in shared memory and stores it a row at a time gives the bits of the
    epilogue that stores element by element, and the plain float32 product."""
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(51)
    a, w = rs.randn(M, K).astype(np.float32), (rs.randn(N, K) / np.sqrt(K)).astype(np.float32)
    bias = rs.randn(N).astype(np.float32)
    A, W = dev(a, torch.bfloat16), dev(w, torch.bfloat16)
    y = (A.float() @ W.float().t()).double() + dev(bias).double()
    want = (torch.nn.functional.gelu(y, approximate="tanh") if act != "none" else y).cpu().numpy()
    try:
        outs = []
        for turned in (False, True):
            ops.set_staged(turned)
            out = ops.gemm_tc_prefill(A, W, dev(bias), act, None, out_dtype=DTYPES[out_dtype], tile_n=tile_n, pair=False)
            torch.cuda.synchronize()
            assert ops.tc_error() == 0
            outs.append(out)
        err = np.abs(outs[1].float().cpu().numpy() - want).max()
        assert err < (1e-3 if out_dtype == "float32" else 5e-2), err
        assert torch.equal(outs[0], outs[1])
    finally:
        ops.set_staged(True)


def test_gemm_prefill_split_files_keys_and_values():
    """The split form as a q | k | v projection: the CTA that finishes a share of the columns also stores
    the keys and values among them into the paged cache."""
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(22)
    lens_q, lens_ctx, H, Hkv, Dh, P, K = [130, 70], [3, 40], 4, 2, 32, 16, 2048
    x, _ = paged_case(rs, lens_q, lens_ctx, H, Hkv, Dh, P, "bfloat16")
    T, qw, kvw = sum(lens_q), H * Dh, Hkv * Dh
    N = qw + 2 * kvw
    a = dev(rs.randn(T, K).astype(np.float32), torch.bfloat16)
    w = dev((rs.randn(N, K) / np.sqrt(K)).astype(np.float32), torch.bfloat16)
    bias = dev(rs.randn(N).astype(np.float32))
    try:
        ops.set_split(0)
        plain_out = ops.gemm_tc_prefill(a, w, bias, out_dtype=torch.bfloat16, tile_n=64, pair=False)
        kc1, vc1 = x["kc"].clone(), x["vc"].clone()
        ops.kv_append(kc1, vc1, plain_out[:, qw:qw + kvw], plain_out[:, qw + kvw:], x["row_req"], x["pos"], x["table"])
        ops.set_split(4)
        kc2, vc2 = x["kc"].clone(), x["vc"].clone()
        filing = ops.KVAppend(kc2, vc2, x["row_req"], x["pos"], x["table"], qw, kvw)
        out = ops.gemm_tc_prefill(a, w, bias, out_dtype=torch.bfloat16, tile_n=64, pair=False, kv=filing)
        torch.cuda.synchronize()
        assert ops.tc_error() == 0 and filing.done and ops.last_split() == 4
        assert float((out.float() - plain_out.float()).abs().max()) < 5e-2
        # the cache holds what the output holds
        kc3, vc3 = x["kc"].clone(), x["vc"].clone()
        ops.kv_append(kc3, vc3, out[:, qw:qw + kvw], out[:, qw + kvw:], x["row_req"], x["pos"], x["table"])
        assert torch.equal(kc2, kc3) and torch.equal(vc2, vc3)
        assert not torch.equal(kc2, x["kc"])
    finally:
        ops.set_split(None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [64, 1600, 2048])
def test_layernorm_many_rows(dtype, width):
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(13)
    x = (rs.randn(777, width) * 2 - 0.5).astype(np.float32)
    g, b = rs.randn(width).astype(np.float32), rs.randn(width).astype(np.float32)
    want = plain_gpt2.layer_norm(x.astype(np.float64), g, b, 1e-5)
    out = ops.layernorm(dev(x), dev(g), dev(b), 1e-5, DTYPES[dtype]).float().cpu().numpy()
    assert np.abs(out - want).max() < tol(dtype, 4.0)
    rows = np.arange(776, -1, -1).astype(np.int32)
    picked = ops.layernorm(dev(x), dev(g), None, 1e-5, DTYPES[dtype], rows=dev(rows)).float().cpu().numpy()
    assert np.abs(picked - (want[rows] - b)).max() < tol(dtype, 4.0)


@pytest.mark.parametrize("singles,portions,ctx_singles,ctx_portions,window", [
    (60, [300], "long", [77], None),                 # 60 decoded tokens beside one 300-row portion
    (3, [130, 2, 257], "short", [0, 510, 64], None),
    (17, [129], "long", [900], 200),                 # window
])
def test_mixed_step_runs_decode_rows_and_portions_through_their_own_kernels(singles, portions, ctx_singles,
                                                                            ctx_portions, window):
    """``ops.attention`` on a step whose first requests bring one row each: those rows take the
    split-context decode kernels, the prompt portions the tiled tensor-core kernel, over one block
    table; the result is the plain attention of every row, and equal to the tiled kernel alone."""
    from types import SimpleNamespace

    from ayaka_py_b200 import ops
    rs = np.random.RandomState(31)
    H, Hkv, P = 5, 5, 16
    ctx_s = [int(c) for c in (rs.randint(600, 1000, singles) if ctx_singles == "long" else rs.randint(0, 40, singles))]
    lens_q = [1] * singles + portions
    lens_ctx = ctx_s + ctx_portions
    x, plain = paged_case(rs, lens_q, lens_ctx, H, Hkv, 64, P, "bfloat16")
    scale = 1.1 / 8.0
    ops.kv_append(x["kc"], x["vc"], x["k"], x["v"], x["row_req"], x["pos"], x["table"])
    T, R = sum(lens_q), len(lens_q)
    ctx = SimpleNamespace(max_q_len=max(lens_q), num_single=singles, num_requests=R, num_rows=T,
                          req_q_start=x["q_start"], req_pos0=x["pos0"], row_req=x["row_req"], positions=x["pos"],
                          cache=SimpleNamespace(max_len=1024), earlier_rows_settled=False)
    before = ops.launches
    out = ops.attention(x["q"], x["kc"], x["vc"], x["table"], ctx, H, scale, window)
    assert ops.launches - before == 3                # partitions, merge, tiled kernel
    alone = ops.attention_tc(x["q"], x["kc"], x["vc"], x["table"], x["q_start"], x["pos0"], T, H, scale, window)
    torch.cuda.synchronize()
    assert ops.tc_error() == 0
    want = plain(scale, window)
    got = out.float().cpu().numpy()
    assert np.abs(got - want).max() < tol("bfloat16")
    assert np.abs(got[:singles] - want[:singles]).max() < tol("bfloat16")
    assert np.abs(got - alone.float().cpu().numpy()).max() < tol("bfloat16")
