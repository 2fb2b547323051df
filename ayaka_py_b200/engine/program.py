"""A model's step as a program for the native executor (``csrc/step_program.cu``).

Every part may say, once, what it launches in a step: ``lower(builder, ...)`` records
operations over symbolic buffers (rows of the step times a fixed width) instead of
launching kernels.  When every part of a model can, the model's step becomes one list
of operations, and a step is then one call into the library, which lays the buffers out
in a workspace for the step's row counts, picks each kernel by the rules of
``ops.linear`` / ``ops.attention`` and launches it.  The kernels, their arguments and
their order are those of ``Model.forward``; only the interpreter is out of the loop
(about 20 us per launch from Python against 2 us from native code, which is what
bounds prompt and mixed steps of small models).

A part without ``lower`` (a toy part of a test, an attention with a position encoding
that turns queries and keys on the host's side) keeps the whole model on
``Model.forward``; nothing else changes for it.  ``AYAKA_B200_NATIVE_STEP=0`` does the
same for every model.
"""

from __future__ import annotations

import ctypes
import os

import torch

from .. import ops
from ..parts.base import KVNeed, NotLowered

OP_EMBED, OP_LAYERNORM, OP_LINEAR, OP_ATTENTION = 0, 1, 2, 3
ROWS_ALL, ROWS_WANTED = 0, 1
LOGITS = -2
MAX_BUFFERS, MAX_GROUPS = 64, 8


class _Buffer(ctypes.Structure):
    _fields_ = [("rows_kind", ctypes.c_int32), ("row_bytes", ctypes.c_int32)]


class _Op(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("src", ctypes.c_int32), ("src2", ctypes.c_int32), ("out", ctypes.c_int32),
                ("i", ctypes.c_int32 * 16), ("f", ctypes.c_float * 2), ("p", ctypes.c_void_p * 4)]


class _Step(ctypes.Structure):
    _fields_ = [("T", ctypes.c_int32), ("R", ctypes.c_int32), ("S", ctypes.c_int32), ("num_single", ctypes.c_int32),
                ("max_q_len", ctypes.c_int32), ("max_context", ctypes.c_int32), ("settled", ctypes.c_int32),
                ("pad_", ctypes.c_int32),
                ("tokens", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("row_req", ctypes.c_void_p),
                ("want_rows", ctypes.c_void_p), ("req_q_start", ctypes.c_void_p), ("req_pos0", ctypes.c_void_p),
                ("tables", ctypes.c_void_p * MAX_GROUPS), ("table_stride", ctypes.c_int32 * MAX_GROUPS),
                ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_longlong), ("logits", ctypes.c_void_p),
                ("decode_scratch", ctypes.c_void_p), ("decode_scratch_floats", ctypes.c_longlong)]


def _bytes(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


class ProgramBuilder:
    """What parts record into.  A buffer is named by a small integer; ``release`` gives it back
    for reuse by a later buffer of the same shape (the layers of a model repeat their shapes, so a
    model needs a handful of buffers whatever its depth)."""

    def __init__(self, cache, dtype: torch.dtype):
        self.cache, self.dtype = cache, dtype
        self.buffers: list[tuple[int, int]] = []          # rows kind, bytes per row
        self.free: dict[tuple[int, int], list[int]] = {}
        self.ops: list[_Op] = []
        self.keep: list[torch.Tensor] = []                # tensors whose addresses the operations hold
        self.filed_slots = 0
        self.decode_floats_per_request = 0                # largest heads * (head size + 2) among the attention layers

    # ------------------------------------------------------------- buffers --
    def buffer(self, width: int, dtype: torch.dtype, wanted: bool = False) -> int:
        key = (ROWS_WANTED if wanted else ROWS_ALL, width * _bytes(dtype))
        spare = self.free.get(key)
        if spare:
            return spare.pop()
        if len(self.buffers) >= MAX_BUFFERS:
            raise NotLowered(f"a step of this model needs more than {MAX_BUFFERS} buffers at once")
        self.buffers.append(key)
        return len(self.buffers) - 1

    def release(self, buf: int) -> None:
        if buf >= 0:
            self.free.setdefault(self.buffers[buf], []).append(buf)

    def _ptr(self, t: torch.Tensor | None) -> int:
        if t is None:
            return 0
        if not t.is_contiguous():
            raise NotLowered("a tensor of a part is not contiguous")
        self.keep.append(t)
        return t.data_ptr()

    def _op(self, kind: int, src: int, src2: int, out: int, ints=(), floats=(), ptrs=()) -> None:
        op = _Op()
        op.kind, op.src, op.src2, op.out = kind, src, src2, out
        for n, v in enumerate(ints):
            op.i[n] = int(v)
        for n, v in enumerate(floats):
            op.f[n] = float(v)
        for n, v in enumerate(ptrs):
            op.p[n] = v or None
        self.ops.append(op)

    # ---------------------------------------------------------- operations --
    def embed(self, table: torch.Tensor, position_table: torch.Tensor | None) -> int:
        """wte[tokens] (+ wpe[positions]) as the float32 residual stream."""
        width = table.shape[1]
        out = self.buffer(width, torch.float32)
        self._op(OP_EMBED, -1, -1, out, ints=(width, ops._tag(table.dtype)),
                 ptrs=(self._ptr(table), self._ptr(position_table)))
        return out

    def layernorm(self, x: int, weight: torch.Tensor, bias: torch.Tensor | None, eps: float, width: int,
                  out_dtype: torch.dtype, wanted: bool = False) -> int:
        """LayerNorm of the float32 rows of ``x`` (of the wanted rows only with ``wanted``)."""
        out = self.buffer(width, out_dtype, wanted)
        self._op(OP_LAYERNORM, x, -1, out, ints=(width, ops._tag(out_dtype), 1 if wanted else 0), floats=(eps,),
                 ptrs=(self._ptr(weight), self._ptr(bias)))
        return out

    def linear(self, x: int, weight: torch.Tensor, bias: torch.Tensor | None, *, activation: str = "none",
               residual: int | None = None, out_dtype: torch.dtype, out: int | None = None, wanted: bool = False,
               filing=None) -> int:
        """act(x @ weight^T + bias) (+ residual).  ``out``: an existing buffer (the residual
        stream, in place), ``LOGITS``, or None for a new one.  ``filing`` = (cache binding,
        first key column, key width): the product is a q | k | v projection that may store the
        key and value columns of prompt rows into the pages itself; returns then (buffer, slot)
        where ``slot`` names the flag that tells the attention whether it did."""
        N, K = weight.shape
        if out is None:
            out = self.buffer(N, out_dtype, wanted)
        ints = [N, K, ops.ACTIVATIONS[activation], ops._tag(weight.dtype), ops._tag(out_dtype),
                ROWS_WANTED if wanted else ROWS_ALL, 0, 0, 0, 0, 0, 0, 0]
        ptrs = [self._ptr(weight), self._ptr(bias), 0, 0]
        slot = -1
        if filing is not None:
            binding, col0, width = filing
            kcache, vcache = self.cache.kv_layer(binding.group, binding.layer)
            slot = self.filed_slots
            self.filed_slots += 1
            ints[6:13] = [1, binding.group, col0, width, self.cache.page_size, ops._tag(kcache.dtype), slot]
            ptrs[2], ptrs[3] = self._ptr(kcache), self._ptr(vcache)
        self._op(OP_LINEAR, x, -1 if residual is None else residual, out, ints=ints, ptrs=ptrs)
        return (out, slot) if filing is not None else out

    def attention(self, qkv: int, binding, *, heads: int, kv_heads: int, head_dim: int, scale: float,
                  window: int | None, dtype: torch.dtype, filed_slot: int = -1) -> int:
        """Attention of the step's rows over the pages of ``binding``; q | k | v are the columns of
        ``qkv``.  The rows' keys and values are stored first unless the projection did (``filed_slot``)
        or the run step only reads another's cache."""
        kcache, vcache = self.cache.kv_layer(binding.group, binding.layer)
        if binding.group >= MAX_GROUPS:
            raise NotLowered(f"more than {MAX_GROUPS} cache groups")
        pages, page_size = kcache.shape[0], kcache.shape[1]
        out = self.buffer(heads * head_dim, dtype)
        self._op(OP_ATTENTION, qkv, -1, out,
                 ints=(heads, kv_heads, head_dim, page_size, window or 0, ops._tag(dtype), binding.group,
                       heads * head_dim, kv_heads * head_dim, 1 if binding.writes else 0, filed_slot),
                 floats=(scale,), ptrs=(self._ptr(kcache), self._ptr(vcache), pages))
        self.decode_floats_per_request = max(self.decode_floats_per_request, heads * (head_dim + 2))
        return out


class StepProgram:
    """The recorded operations of a model, runnable for a ``StepContext``."""

    def __init__(self, builder: ProgramBuilder, vocab_size: int, device):
        self.lib = ops._ready()
        self.n_ops, self.n_buffers = len(builder.ops), len(builder.buffers)
        self.ops = (_Op * self.n_ops)(*builder.ops)
        self.buffers = (_Buffer * max(1, self.n_buffers))(*[_Buffer(k, b) for k, b in builder.buffers])
        self.keep = builder.keep
        self.cache = builder.cache
        self.vocab_size, self.device = vocab_size, device
        self.decode_floats_per_request = builder.decode_floats_per_request
        self.kv_groups = [g for g, spec in enumerate(self.cache.groups) if isinstance(spec.need, KVNeed)]
        self.workspace = torch.empty(1 << 20, dtype=torch.uint8, device=device)
        self.retired: list[torch.Tensor] = []             # a captured CUDA graph may still write to an outgrown workspace
        self.lib.ayk_program_workspace_bytes.restype = ctypes.c_longlong
        self._step = _Step()
        self._launched = ctypes.c_int(0)

    def run(self, ctx) -> torch.Tensor:
        """Logits [S, V] float32 of the step that ``ctx`` describes."""
        T, S = ctx.num_rows, ctx.num_wanted
        need = int(self.lib.ayk_program_workspace_bytes(self.buffers, self.n_buffers, T, S))
        if need > self.workspace.numel():
            self.retired.append(self.workspace)
            self.workspace = torch.empty(max(need, 2 * self.workspace.numel()), dtype=torch.uint8, device=self.device)
        logits = torch.empty((S, self.vocab_size), dtype=torch.float32, device=self.device)
        step = self._step
        step.T, step.R, step.S = T, ctx.num_requests, S
        step.num_single, step.max_q_len = ctx.num_single, ctx.max_q_len
        step.max_context = self.cache.max_len
        step.settled = 1 if ctx.earlier_rows_settled else 0
        step.tokens, step.positions, step.row_req = ctx.tokens.data_ptr(), ctx.positions.data_ptr(), ctx.row_req.data_ptr()
        step.want_rows, step.req_q_start, step.req_pos0 = (ctx.want_rows.data_ptr(), ctx.req_q_start.data_ptr(),
                                                           ctx.req_pos0.data_ptr())
        for g in self.kv_groups:
            table = ctx.tables[g]
            step.tables[g], step.table_stride[g] = table.data_ptr(), table.stride(0)
        step.workspace, step.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        step.logits = logits.data_ptr()
        if self.decode_floats_per_request:
            parts = -(-self.cache.max_len // ops.DECODE_PART)
            scratch = ops._decode_buffer(self.device, ctx.num_requests * self.decode_floats_per_request * parts)
            step.decode_scratch, step.decode_scratch_floats = scratch.data_ptr(), scratch.numel()
        code = self.lib.ayk_program_run(self.ops, self.n_ops, self.buffers, self.n_buffers, ctypes.byref(step),
                                        ctypes.byref(self._launched), ops._stream())
        ops.launches += self._launched.value
        ops._check(code)
        return logits


def lower_model(model, cache) -> StepProgram | None:
    """The model's step as a program, or None when a part of it cannot be lowered (then
    ``Model.forward`` runs the step) or AYAKA_B200_NATIVE_STEP=0 asks for the Python path."""
    if os.environ.get("AYAKA_B200_NATIVE_STEP", "1") == "0" or not str(model.device).startswith("cuda"):
        return None
    builder = ProgramBuilder(cache, model.dtype)
    try:
        x = model.embedding.lower(builder, model.position)
        for step, caches in zip(model.spec.order, model.bindings):
            x = model.blocks[step.layer].lower(builder, x, caches)
        h = model.final_norm.lower(builder, x, wanted=True)
        model.head.lower(builder, h)
    except NotLowered:
        return None
    return StepProgram(builder, model.vocab_size, model.device)
