"""Python face of the CUDA library: one function per kernel, torch tensors in.

The library is built by ``csrc/build.py`` (at the first call if it is missing
or stale) and loaded with ctypes.  There is no fallback: when the library
cannot be built or loaded, or a tensor does not live on a CUDA device, the call
raises.  Every function launches on torch's current stream.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_TAG = {torch.float32: F32, torch.bfloat16: BF16}
ACTIVATIONS = {"none": 0, "gelu_erf": 1, "gelu_tanh": 2, "quick_gelu": 3}

_lib = None
_lock = threading.Lock()


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


def library():
    """The loaded library; builds it first if needed."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.build()
                lib = ctypes.CDLL(str(path))
                lib.ayk_last_error.restype = ctypes.c_char_p
                _lib = lib
    return _lib


def library_file() -> str:
    return str(_build.library_path())


_initialised = False


def _ready():
    global _initialised
    lib = library()
    if not _initialised:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this package runs its kernels on a B200 and has no CPU path")
        _check(lib.ayk_init(ctypes.c_int(torch.cuda.current_device())))
        lib.ayk_set_pdl(ctypes.c_int(0 if os.environ.get("AYAKA_B200_PDL", "1") == "0" else 1))
        _initialised = True
    return lib


def set_pdl(on: bool) -> None:
    """Launch kernels with programmatic stream serialization (the default; the
    environment variable AYAKA_B200_PDL=0 switches it off): a kernel may be
    scheduled while its predecessor still runs and waits, on the device, for
    the predecessor's results before it touches them."""
    _ready().ayk_set_pdl(ctypes.c_int(1 if on else 0))


def set_split(parts: int | None) -> None:
    """Split along K in the product for many rows (``gemm_tc_prefill``, one-SM form): when the tiles
    alone would leave most SMs idle, the 2, 4 or 8 CTAs of a cluster share a tile, each with an equal
    part of its K blocks; they exchange their sums through shared memory and each finishes a share of
    the tile's columns.  None: the
    library decides per product (the default); 0: never; 2, 4, 8: wherever the tiles allow it."""
    _ready().ayk_gemm_tc_prefill_split(ctypes.c_int(-1 if parts is None else int(parts)))


def set_staged(on: bool) -> None:
    """The staged residual epilogue of ``gemm_tc_prefill`` (float32 out over a float32 residual: both
    through shared memory by TMA, whole lines at a time) where it applies (the default), or never."""
    _ready().ayk_gemm_tc_prefill_staged(ctypes.c_int(1 if on else 0))


def prefill_plan(M: int, N: int, K: int, sms: int = 148, wide_rows: bool = False) -> tuple[int, int]:
    """(tile width, parts of K per tile) that ``gemm_tc_prefill`` picks for an [M, K] x [N, K]^T product
    on ``sms`` SMs; ``wide_rows``: the epilogue reads or writes 32-bit rows.  Host arithmetic from the
    kernel's fitted time model: works without a GPU."""
    tile, parts = ctypes.c_int(0), ctypes.c_int(0)
    library().ayk_gemm_tc_prefill_plan(ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(sms),
                                       ctypes.c_int(1 if wide_rows else 0), ctypes.byref(tile), ctypes.byref(parts))
    return tile.value, parts.value


def last_staged() -> int:
    """Buffers per half through which the last ``gemm_tc_prefill`` staged its residual (0: it did not)."""
    return int(_ready().ayk_gemm_tc_prefill_last_staged())


def last_split() -> int:
    """Into how many parts the last ``gemm_tc_prefill`` (one-SM form) split the K blocks of its tiles."""
    return int(_ready().ayk_gemm_tc_prefill_last_split())


def _check(code: int) -> None:
    if code != 0:
        raise KernelError(library().ayk_last_error().decode("utf-8", "replace"))


launches = 0      # kernels of this library launched so far (graph replays are counted by their owner)


def _launch(code: int) -> None:
    global launches
    launches += 1
    _check(code)


def _ptr(t: torch.Tensor | None):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("tensor is not on a CUDA device")
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _tag(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_TAG[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported (float32 or bfloat16)") from None


def _i32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return t


# ---------------------------------------------------------------- kernels --

def embed(tokens: torch.Tensor, positions: torch.Tensor, table: torch.Tensor,
          position_table: torch.Tensor | None, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[tokens[t]] (+ position_table[positions[t]]), float32 [T, d]."""
    lib = _ready()
    T, d = tokens.numel(), table.shape[1]
    if out is None:
        out = torch.empty((T, d), dtype=torch.float32, device=table.device)
    if position_table is not None and (position_table.dtype != table.dtype or position_table.shape[1] != d):
        raise KernelError("position table must match the token table in dtype and width")
    if not table.is_contiguous() or (position_table is not None and not position_table.is_contiguous()):
        raise KernelError("embedding tables must be contiguous")
    _launch(lib.ayk_embed(_ptr(out), _ptr(_i32(tokens, "tokens")), _ptr(_i32(positions, "positions")),
                         _ptr(table), _ptr(position_table), ctypes.c_int(T), ctypes.c_int(d),
                         ctypes.c_int(_tag(table.dtype)), _stream()))
    return out


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor | None, eps: float,
              out_dtype: torch.dtype, rows: torch.Tensor | None = None,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """LayerNorm of float32 rows (of ``x[rows]`` when rows is given), result as out_dtype."""
    lib = _ready()
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("layernorm input must be contiguous float32")
    d = x.shape[-1]
    n = x.shape[0] if rows is None else rows.numel()
    if gamma.dtype != torch.float32 or gamma.numel() != d or (beta is not None and (beta.dtype != torch.float32 or beta.numel() != d)):
        raise KernelError("layernorm weight and bias must be float32 of the row width")
    if out is None:
        out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    _launch(lib.ayk_layernorm(_ptr(out), _ptr(x), _ptr(gamma), _ptr(beta),
                             _ptr(None if rows is None else _i32(rows, "rows")), ctypes.c_int(n),
                             ctypes.c_int(d), ctypes.c_float(eps), ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
              activation: str = "none", residual: torch.Tensor | None = None,
              out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """act(a[M,K] @ w[N,K]^T + bias) (+ residual) on the FP32 pipes."""
    lib = _ready()
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or a.dtype != w.dtype or not a.is_contiguous() or not w.is_contiguous():
        raise KernelError(f"gemm operands do not fit: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    for name, t in (("bias", bias), ("residual", residual)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"{name} must be contiguous float32")
    if residual is not None and tuple(residual.shape) != (M, N):
        raise KernelError("residual must have the output's shape")
    _launch(lib.ayk_gemm_simt(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), ctypes.c_int(M),
                             ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(ACTIVATIONS[activation]),
                             ctypes.c_int(_tag(a.dtype)), ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def kv_append(kcache: torch.Tensor, vcache: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              row_req: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> None:
    """cache[page, pos % P] = k/v row; k and v are column slices [T, Hkv*Dh] of one matrix."""
    lib = _ready()
    T, width = k.shape
    pages, P, Hkv, Dh = kcache.shape
    if width != Hkv * Dh or v.shape != k.shape or k.stride(1) != 1 or v.stride(1) != 1 or k.stride(0) != v.stride(0):
        raise KernelError("kv_append: keys and values must be [T, kv_heads*head_dim] slices with one row stride")
    if k.dtype != kcache.dtype or not kcache.is_contiguous() or not vcache.is_contiguous():
        raise KernelError("kv_append: cache must be contiguous and of the rows' dtype")
    _launch(lib.ayk_kv_append(_ptr(kcache), _ptr(vcache), _ptr(k), _ptr(v), ctypes.c_int(k.stride(0)),
                             _ptr(_i32(row_req, "row_req")), _ptr(_i32(positions, "positions")),
                             _ptr(_i32(table, "table")), ctypes.c_int(table.stride(0)), ctypes.c_int(P),
                             ctypes.c_int(T), ctypes.c_int(width), ctypes.c_int(_tag(k.dtype)), _stream()))


def attention_simt(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, table: torch.Tensor,
                   req_q_start: torch.Tensor, req_pos0: torch.Tensor, total_rows: int, num_heads: int,
                   scale: float, window: int | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of the step's rows over the paged cache.  q: [T, H*Dh] slice."""
    lib = _ready()
    pages, P, Hkv, Dh = kcache.shape
    T = q.shape[0]
    if q.shape[1] != num_heads * Dh or q.stride(1) != 1 or q.dtype != kcache.dtype:
        raise KernelError("attention: q must be a [T, heads*head_dim] slice of the cache's dtype")
    if total_rows != T:
        raise KernelError(f"attention: {total_rows} rows named, q has {T} (rows beyond the count would stay unwritten)")
    if out is None:
        out = torch.empty((T, num_heads * Dh), dtype=q.dtype, device=q.device)
    R = req_pos0.numel()
    _launch(lib.ayk_attention_simt(_ptr(out), _ptr(q), ctypes.c_int(q.stride(0)), _ptr(kcache), _ptr(vcache),
                                  _ptr(_i32(table, "table")), ctypes.c_int(table.stride(0)),
                                  _ptr(_i32(req_q_start, "req_q_start")), _ptr(_i32(req_pos0, "req_pos0")),
                                  ctypes.c_int(R), ctypes.c_int(total_rows), ctypes.c_int(num_heads),
                                  ctypes.c_int(Hkv), ctypes.c_int(Dh), ctypes.c_int(P), ctypes.c_float(scale),
                                  ctypes.c_int(window or 0), ctypes.c_int(_tag(q.dtype)), _stream()))
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor | None = None,
           seed: torch.Tensor | None = None, offset: torch.Tensor | None = None,
           top_k: torch.Tensor | None = None, top_p: torch.Tensor | None = None,
           min_p: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of float32 logits: greedy where temperature is 0 or
    absent; else a draw after the top_k / top_p / min_p filters (null: off)."""
    lib = _ready()
    if logits.dtype != torch.float32 or not logits.is_contiguous() or logits.dim() != 2:
        raise KernelError("sample: logits must be contiguous float32 [S, V]")
    S, V = logits.shape
    out = torch.empty((S,), dtype=torch.int32, device=logits.device)
    if temperature is not None:
        if temperature.dtype != torch.float32 or seed.dtype != torch.int64 or offset.dtype != torch.int64:
            raise KernelError("sample: temperature float32, seed and offset int64")
    for name, t, dt in (("top_k", top_k, torch.int64), ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32)):
        if t is not None and (t.dtype != dt or t.numel() != S or not t.is_contiguous()):
            raise KernelError(f"sample: {name} must be a contiguous {dt} tensor with one value per row")
    _launch(lib.ayk_sample(_ptr(out), _ptr(logits), ctypes.c_int(S), ctypes.c_int(V), _ptr(temperature),
                          _ptr(seed), _ptr(offset), _ptr(top_k), _ptr(top_p), _ptr(min_p), _stream()))
    return out


def ban_tokens(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor) -> None:
    """logits[rows[i], tokens[i]] = -inf, in place (int32 index tensors on the device)."""
    lib = _ready()
    if logits.dtype != torch.float32 or not logits.is_contiguous() or logits.dim() != 2:
        raise KernelError("ban_tokens: logits must be contiguous float32 [S, V]")
    if rows.numel() != tokens.numel():
        raise KernelError("ban_tokens: one row index per token id")
    S, V = logits.shape
    _launch(lib.ayk_ban_tokens(_ptr(logits), _ptr(_i32(rows, "rows")), _ptr(_i32(tokens, "tokens")),
                               ctypes.c_int(rows.numel()), ctypes.c_int(S), ctypes.c_int(V), _stream()))


# ------------------------------------------------------------- dispatchers --

_tc_scratch: dict = {}
_tc_retired: list = []          # a captured CUDA graph may still write to an outgrown buffer
_sm_count = 0


def sm_count() -> int:
    """Streaming multiprocessors of the current device, asked of the driver once (148 on a B200)."""
    global _sm_count
    if _sm_count == 0:
        _sm_count = int(_ready().ayk_device_sm_count())
    return _sm_count


def _tc_workspace(device, floats: int):
    ws = _tc_scratch.get(device)
    if ws is None or ws[0].numel() < floats:
        if ws is not None:
            _tc_retired.append(ws[0])
        partials = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
        counters = ws[1] if ws is not None else torch.zeros(8192, dtype=torch.int32, device=device)
        ws = (partials, counters)
        _tc_scratch[device] = ws
    return ws


CLUSTER_ROWS = 64        # up to this many rows the splits of a tile exchange their sums inside a cluster


def tc_splits(M: int, N: int, K: int) -> int:
    """Split-K factor of the tensor-core product: skinny products (few output
    tiles) are cut along K so that about one CTA per SM streams the weight.
    Up to 64 rows the factor is 1, 2, 4, 8 or 16: those splits form a cluster.  16 (beyond the
    portable cluster size) only where each split still has four K blocks: a product of 13
    tiles and K = 6400 streamed at 3.6 TB/s from 104 CTAs, which do not keep enough
    bytes in flight, and at the copy rate from 200.  (The rule itself lives in the library,
    where the native step program uses it too.)"""
    return int(_ready().ayk_tc_splits(ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K)))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
            activation: str = "none", residual: torch.Tensor | None = None,
            out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None,
            splits: int | None = None, static_weight: bool = True, cluster: bool | None = None) -> torch.Tensor:
    """act(a[M,K] @ w[N,K]^T + bias) (+ residual), bfloat16 operands, on tcgen05.
    ``splits``: CTAs along K per output tile (default: chosen by shape).  ``cluster``:
    the splits exchange their sums through shared memory of a thread-block cluster
    instead of scratch in global memory (default where it applies: up to 64 rows,
    2, 4, 8 or 16 splits)."""
    lib = _ready()
    M, K = a.shape
    N = w.shape[0]
    if (w.shape[1] != K or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16
            or not a.is_contiguous() or not w.is_contiguous()):
        raise KernelError(f"gemm_tc operands do not fit: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    for name, t in (("bias", bias), ("residual", residual)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"{name} must be contiguous float32")
    if residual is not None and tuple(residual.shape) != (M, N):
        raise KernelError("residual must have the output's shape")
    if splits is None:
        splits = tc_splits(M, N, K)
    can_cluster = M <= CLUSTER_ROWS and splits in (2, 4, 8, 16) and -(-K // 64) >= splits
    if cluster is None:
        cluster = can_cluster
    elif cluster and not can_cluster:
        raise KernelError(f"gemm_tc: the cluster form takes up to {CLUSTER_ROWS} rows and 2, 4, 8 or 16 splits (rows {M}, splits {splits})")
    partials = counters = None
    if splits > 1 and not cluster:
        tiles = -(-N // 128) * -(-M // 16)
        partials, counters = _tc_workspace(a.device, splits * M * N)
        if tiles > counters.numel():
            raise KernelError("gemm_tc: too many output tiles for split-K")
    _launch(lib.ayk_gemm_tc(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), ctypes.c_int(M),
                           ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(ACTIVATIONS[activation]),
                           ctypes.c_int(_tag(out_dtype)), ctypes.c_int(splits), _ptr(partials), _ptr(counters),
                           ctypes.c_int(1 if static_weight else 0), ctypes.c_int(1 if cluster else 0), _stream()))
    return out


PREFILL_ROWS = 16        # more rows than this: the kernel with 128-row tiles and no split along K


class KVAppend:
    """Where the key and value columns of a fused q | k | v projection belong in the paged
    cache: ``linear`` hands this to the product that can file them itself (the many-row
    tensor-core kernel, in its epilogue) and sets ``done``; the caller appends them with
    ``kv_append`` otherwise."""

    def __init__(self, kcache: torch.Tensor, vcache: torch.Tensor, row_req: torch.Tensor, positions: torch.Tensor,
                 table: torch.Tensor, col0: int, width: int):
        self.kcache, self.vcache, self.row_req, self.positions, self.table = kcache, vcache, row_req, positions, table
        self.col0, self.width = col0, width
        self.done = False

    def fits(self, n_out: int, out_dtype) -> bool:
        pages, P, Hkv, Dh = self.kcache.shape
        return (out_dtype == torch.bfloat16 and self.kcache.dtype == torch.bfloat16 and self.width == Hkv * Dh
                and self.col0 % 8 == 0 and self.width % 8 == 0 and n_out == self.col0 + 2 * self.width
                and self.kcache.is_contiguous() and self.vcache.is_contiguous())


def gemm_tc_prefill(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                    activation: str = "none", residual: torch.Tensor | None = None,
                    out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None,
                    tile_n: int = 0, pair: bool | None = None, kv: KVAppend | None = None) -> torch.Tensor:
    """act(a[M,K] @ w[N,K]^T + bias) (+ residual) for many rows: persistent tcgen05
    kernel, epilogue of a tile under the main loop of the next.  ``pair``: two SMs
    on a 256-row tile (tcgen05 cta_group::2) or one SM on a 128-row tile (the default;
    AYAKA_B200_GEMM_PAIR=1 makes pairs the default from 129 rows on).  ``kv``: the product is a
    q | k | v projection whose key and value columns also go into the paged cache."""
    lib = _ready()
    M, K = a.shape
    N = w.shape[0]
    if (w.shape[1] != K or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16
            or not a.is_contiguous() or not w.is_contiguous()):
        raise KernelError(f"gemm_tc_prefill operands do not fit: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    for name, t in (("bias", bias), ("residual", residual)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"{name} must be contiguous float32")
    if residual is not None and tuple(residual.shape) != (M, N):
        raise KernelError("residual must have the output's shape")
    if kv is not None:
        if activation != "none" or residual is not None or not kv.fits(N, out_dtype):
            raise KernelError("gemm_tc_prefill: keys and values are filed only by a plain bfloat16 q | k | v projection")
        P = kv.kcache.shape[1]
        _launch(lib.ayk_gemm_tc_prefill_kv(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), ctypes.c_int(M), ctypes.c_int(N),
                                           ctypes.c_int(K), ctypes.c_int(tile_n), ctypes.c_int(sm_count()),
                                           ctypes.c_int(-1 if pair is None else int(pair)), _ptr(kv.kcache), _ptr(kv.vcache),
                                           _ptr(_i32(kv.row_req, "row_req")), _ptr(_i32(kv.positions, "positions")),
                                           _ptr(_i32(kv.table, "table")), ctypes.c_int(kv.table.stride(0)), ctypes.c_int(P),
                                           ctypes.c_int(kv.col0), ctypes.c_int(kv.width), _stream()))
        kv.done = True
        return out
    _launch(lib.ayk_gemm_tc_prefill(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), ctypes.c_int(M),
                                    ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(ACTIVATIONS[activation]),
                                    ctypes.c_int(_tag(out_dtype)), ctypes.c_int(tile_n), ctypes.c_int(sm_count()),
                                    ctypes.c_int(-1 if pair is None else int(pair)), _stream()))
    return out


class _KvTarget(ctypes.Structure):
    _fields_ = [("kcache", ctypes.c_void_p), ("vcache", ctypes.c_void_p), ("row_req", ctypes.c_void_p),
                ("positions", ctypes.c_void_p), ("table", ctypes.c_void_p), ("table_stride", ctypes.c_int32),
                ("page_size", ctypes.c_int32), ("col0", ctypes.c_int32), ("width", ctypes.c_int32),
                ("dtype", ctypes.c_int32)]


def linear(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           activation: str = "none", residual: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None,
           kv: KVAppend | None = None) -> torch.Tensor:
    """act(a @ w^T + bias) (+ residual).  float32 operands run on the FP32
    pipes (true 32-bit); bfloat16 operands on the tensor cores (tcgen05) when
    K is a multiple of 8, else on the FP32 pipes with 32-bit accumulation: up to 16 rows,
    and up to 64 rows with few output tiles, the kernel whose CTAs split K inside a cluster;
    above, the persistent kernel with 128-row tiles.  The choice is made in the library
    (``ayk_linear``), by the same code that the native step program runs.
    ``kv``: see KVAppend; ``kv.done`` tells whether the product filed the rows."""
    lib = _ready()
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or a.dtype != w.dtype or not a.is_contiguous() or not w.is_contiguous():
        raise KernelError(f"linear: operands do not fit: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    elif tuple(out.shape) != (M, N) or out.dtype != out_dtype or not out.is_contiguous():
        raise KernelError("linear: out must be a contiguous [M, N] tensor of the output dtype")
    for name, t in (("bias", bias), ("residual", residual)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"{name} must be contiguous float32")
    if residual is not None and tuple(residual.shape) != (M, N):
        raise KernelError("residual must have the output's shape")
    target, filed = None, ctypes.c_int(0)
    if kv is not None and kv.fits(N, out_dtype):
        target = _KvTarget(kv.kcache.data_ptr(), kv.vcache.data_ptr(), _i32(kv.row_req, "row_req").data_ptr(),
                           _i32(kv.positions, "positions").data_ptr(), _i32(kv.table, "table").data_ptr(),
                           kv.table.stride(0), kv.kcache.shape[1], kv.col0, kv.width, _tag(kv.kcache.dtype))
    _launch(lib.ayk_linear(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), ctypes.c_int(M), ctypes.c_int(N),
                           ctypes.c_int(K), ctypes.c_int(ACTIVATIONS[activation]), ctypes.c_int(_tag(a.dtype)),
                           ctypes.c_int(_tag(out_dtype)), ctypes.byref(target) if target is not None else None,
                           ctypes.byref(filed), _stream()))
    if kv is not None and filed.value:
        kv.done = True
    return out


DECODE_PART = 128
_decode_scratch: dict = {}      # device -> partials; outgrown buffers stay alive below
_decode_retired: list = []      # a captured CUDA graph may still write to an outgrown buffer


def _decode_buffer(device, floats: int) -> torch.Tensor:
    have = _decode_scratch.get(device)
    if have is None or have.numel() < floats:
        if have is not None:
            _decode_retired.append(have)
        have = torch.empty(max(floats, 1 << 21), dtype=torch.float32, device=device)
        _decode_scratch[device] = have
    return have


def attention_decode(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, table: torch.Tensor,
                     req_pos0: torch.Tensor, num_heads: int, scale: float, window: int | None,
                     max_context: int, out: torch.Tensor | None = None,
                     append: tuple | None = None, settled: bool = False) -> torch.Tensor:
    """One query row per request over its pages, split along the context and
    merged.  ``max_context``: the longest context the engine allows (fixes the grid).
    ``append`` = (k, v, row_req): this step's key and value rows, not yet in the
    cache; they are stored at each request's position on the way (inside the
    attention kernel where it can, else by the append kernel first).  ``settled``:
    the cache rows before the requests' positions were written by work that is
    complete (an earlier step); the kernel may then read them while the kernels
    launched just before it still run."""
    lib = _ready()
    pages, P, Hkv, Dh = kcache.shape
    R = q.shape[0]
    if q.shape[1] != num_heads * Dh or q.stride(1) != 1 or q.dtype != kcache.dtype:
        raise KernelError("attention_decode: q must be a [R, heads*head_dim] slice of the cache's dtype")
    if req_pos0.numel() != R:
        raise KernelError("attention_decode: one row per request")
    parts = -(-max_context // DECODE_PART)
    scratch = _decode_buffer(q.device, R * num_heads * parts * (Dh + 2))
    if out is None:
        out = torch.empty((R, num_heads * Dh), dtype=q.dtype, device=q.device)
    k_new = v_new = row_req = None
    new_stride = 0
    if append is not None:
        k_new, v_new, row_req = append
        if (k_new.shape != (R, Hkv * Dh) or v_new.shape != k_new.shape or k_new.stride(1) != 1 or v_new.stride(1) != 1
                or k_new.stride(0) != v_new.stride(0) or k_new.dtype != kcache.dtype or v_new.dtype != kcache.dtype):
            raise KernelError("attention_decode: new keys and values must be [R, kv_heads*head_dim] slices of one matrix")
        new_stride = k_new.stride(0)
    _launch(lib.ayk_attention_decode(_ptr(out), _ptr(q), ctypes.c_int(q.stride(0)), _ptr(kcache), _ptr(vcache),
                                     _ptr(_i32(table, "table")), ctypes.c_int(table.stride(0)),
                                     _ptr(_i32(req_pos0, "req_pos0")), ctypes.c_int(R), ctypes.c_int(num_heads),
                                     ctypes.c_int(Hkv), ctypes.c_int(Dh), ctypes.c_int(P), ctypes.c_float(scale),
                                     ctypes.c_int(window or 0), ctypes.c_int(parts), _ptr(scratch),
                                     _ptr(k_new), _ptr(v_new), ctypes.c_int(new_stride),
                                     _ptr(_i32(row_req, "row_req") if row_req is not None else None),
                                     ctypes.c_longlong(pages), ctypes.c_int(1 if settled else 0),
                                     ctypes.c_int(_tag(q.dtype)), _stream()))
    global launches
    launches += 1            # the call launches two kernels (partitions, merge)
    return out


def attention_tc_takes(q: torch.Tensor, kcache: torch.Tensor) -> bool:
    """Whether the tensor-core attention kernel takes this geometry: bfloat16,
    head size 64, pages of 8 to 128 tokens, 16-byte aligned query rows."""
    pages, P, Hkv, Dh = kcache.shape
    return (q.dtype == torch.bfloat16 and Dh == 64 and 8 <= P <= 128 and P & (P - 1) == 0
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def attention_tc(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, table: torch.Tensor,
                 req_q_start: torch.Tensor, req_pos0: torch.Tensor, total_rows: int, num_heads: int,
                 scale: float, window: int | None = None, out: torch.Tensor | None = None,
                 first_row: int = 0) -> torch.Tensor:
    """Causal attention of prompt portions over the paged cache on tcgen05 (bfloat16, head size 64).
    ``first_row``: the requests named here cover rows first_row .. T of ``q`` and ``out`` (their
    ``req_q_start`` holds absolute row numbers); earlier rows are left to another kernel."""
    lib = _ready()
    pages, P, Hkv, Dh = kcache.shape
    T = q.shape[0]
    if q.shape[1] != num_heads * Dh or q.stride(1) != 1 or q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16:
        raise KernelError("attention_tc: q must be a bfloat16 [T, heads*head_dim] slice, the cache bfloat16")
    if total_rows + first_row != T:
        raise KernelError(f"attention_tc: rows {first_row} .. {first_row + total_rows} named, q has {T} "
                          f"(rows beyond the count would stay unwritten)")
    if not kcache.is_contiguous() or not vcache.is_contiguous():
        raise KernelError("attention_tc: the cache must be contiguous")
    if out is None:
        out = torch.empty((T, num_heads * Dh), dtype=q.dtype, device=q.device)
    R = req_pos0.numel()
    _launch(lib.ayk_attention_tc(_ptr(out), _ptr(q), ctypes.c_int(q.stride(0)), ctypes.c_int(T), ctypes.c_int(total_rows),
                                 _ptr(kcache), _ptr(vcache), ctypes.c_int(pages), _ptr(_i32(table, "table")),
                                 ctypes.c_int(table.stride(0)), _ptr(_i32(req_q_start, "req_q_start")),
                                 _ptr(_i32(req_pos0, "req_pos0")), ctypes.c_int(R), ctypes.c_int(num_heads),
                                 ctypes.c_int(Hkv), ctypes.c_int(Dh), ctypes.c_int(P), ctypes.c_float(scale),
                                 ctypes.c_int(window or 0), _stream()))
    return out


MIXED_DECODE_MIN = 1     # single-token requests in a mixed step from which they take the decode kernels


def tc_error() -> int:
    """0, or the code of the bounded wait that ran out in a tensor-core kernel
    (1-4: matrix product, 11-17: attention)."""
    lib = library()
    return (int(lib.ayk_gemm_tc_error()) or int(lib.ayk_attention_tc_error())
            or int(lib.ayk_gemm_tc_prefill_error()))


def attention(q, kcache, vcache, table, ctx, num_heads: int, scale: float,
              window: int | None = None, append: tuple | None = None) -> torch.Tensor:
    """Attention of the step's rows (``ctx`` gives the rows of each request): the
    split-context decode kernels when every request brings one row (head sizes in
    steps of 16); the tensor-core kernel for prompt portions in bfloat16 with head
    size 64, beside the decode kernels for the single rows of a mixed step; else
    the general kernel, which takes every head size up to 256.  ``append`` = (k, v): the rows' keys and values, which
    go into the cache first (in a decode step, inside the attention kernel)."""
    # Head sizes that are no multiple of 16 are taken by the general kernel alone (the decode kernels
    # read keys in 16-byte pieces and refuse them).
    if ctx.max_q_len == 1 and kcache.shape[3] % 16 == 0:
        return attention_decode(q, kcache, vcache, table, ctx.req_pos0, num_heads, scale, window,
                                ctx.cache.max_len,
                                append=(append[0], append[1], ctx.row_req) if append is not None else None,
                                settled=getattr(ctx, "earlier_rows_settled", False))
    if append is not None:
        kv_append(kcache, vcache, append[0], append[1], ctx.row_req, ctx.positions, table)
    if attention_tc_takes(q, kcache):
        # A mixed step: its single-token requests are its first rows (the step runner packs them
        # first).  They go through the split-context decode kernels, one row per request, and the
        # prompt portions through the tiled kernel: two launches on disjoint row ranges over one
        # block table.  (As rows of the tiled kernel each would be a 128-row tile with one live row.)
        D = getattr(ctx, "num_single", 0)
        if D >= MIXED_DECODE_MIN and D < ctx.num_requests:
            out = torch.empty((ctx.num_rows, q.shape[1]), dtype=q.dtype, device=q.device)
            attention_decode(q[:D], kcache, vcache, table[:D], ctx.req_pos0[:D], num_heads, scale, window,
                             ctx.cache.max_len, out=out[:D], settled=getattr(ctx, "earlier_rows_settled", False))
            return attention_tc(q, kcache, vcache, table[D:], ctx.req_q_start[D:], ctx.req_pos0[D:],
                                ctx.num_rows - D, num_heads, scale, window, out=out, first_row=D)
        return attention_tc(q, kcache, vcache, table, ctx.req_q_start, ctx.req_pos0, ctx.num_rows,
                            num_heads, scale, window)
    return attention_simt(q, kcache, vcache, table, ctx.req_q_start, ctx.req_pos0, ctx.num_rows,
                          num_heads, scale, window)
