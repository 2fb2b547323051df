"""A small safetensors reader and writer.

File: u64 little-endian header length, a JSON header (name -> dtype, shape,
data_offsets), then the payload.  The reader makes the checks the reference's
own parser makes (``model_loader/st.py:38-48``, ``:98-331``): header length
bounded and inside the file, valid UTF-8 JSON without duplicate keys, known
dtype, non-negative shapes, ordered offsets inside the payload, byte count equal
to numel * itemsize, no overlap.  Tensors are read one at a time through a
memory map; bfloat16 is handed out as a ``torch.bfloat16`` tensor.
"""

from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

MAX_HEADER_BYTES = 64 << 20

_ITEMSIZE = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2,
             "I8": 1, "U8": 1, "BOOL": 1}
_TORCH = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
          "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
          "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}
_NUMPY = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16,
          "I64": np.int64, "I32": np.int32, "I16": np.int16, "I8": np.int8,
          "U8": np.uint8, "BOOL": np.bool_}
_TOKEN_OF = {v: k for k, v in _TORCH.items()}


class CheckpointCorruptError(ValueError):
    """The file is not a well-formed safetensors file."""


class UnsupportedWeightFormatError(ValueError):
    """The file is well formed but stores tensors in a format this engine has
    no path for: sub-byte and 8-bit float dtypes (packed or quantized weights).
    A refusal rather than a silent reinterpretation (``exceptions.py:53-60``,
    ``model_loader/st.py:98-131`` in the reference)."""


# dtype tokens of the safetensors format that are known but not readable here
_UNSUPPORTED_TOKENS = {"I4", "U4", "F4", "F6_E2M3", "F6_E3M2", "F8_E4M3", "F8_E5M2", "F8_E8M0"}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str                 # safetensors token, e.g. "BF16"
    shape: tuple[int, ...]
    begin: int                 # byte offsets inside the payload
    end: int

    @property
    def torch_dtype(self) -> torch.dtype:
        return _TORCH[self.dtype]


def _no_duplicates(pairs):
    seen = {}
    for key, value in pairs:
        if key in seen:
            raise CheckpointCorruptError(f"duplicate key in header: {key!r}")
        seen[key] = value
    return seen


class SafetensorsFile:
    """An open file: ``entries`` by name and ``read(name)``."""

    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise CheckpointCorruptError(f"{self.path}: shorter than its 8-byte length field")
        self._fh = open(self.path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > MAX_HEADER_BYTES:
            raise CheckpointCorruptError(f"{self.path}: header of {hlen} bytes exceeds {MAX_HEADER_BYTES}")
        if 8 + hlen > size:
            raise CheckpointCorruptError(f"{self.path}: header of {hlen} bytes runs past the file end")
        raw = self._fh.read(hlen)
        try:
            header = json.loads(raw.decode("utf-8"), object_pairs_hook=_no_duplicates)
        except UnicodeDecodeError as exc:
            raise CheckpointCorruptError(f"{self.path}: header is not UTF-8") from exc
        except json.JSONDecodeError as exc:
            raise CheckpointCorruptError(f"{self.path}: header is not JSON: {exc}") from exc
        if not isinstance(header, dict):
            raise CheckpointCorruptError(f"{self.path}: header must be a JSON object")
        self.payload_start = 8 + hlen
        payload = size - self.payload_start
        self.metadata = header.pop("__metadata__", None)
        self.entries: dict[str, TensorEntry] = {}
        spans = []
        for name, info in header.items():
            if not isinstance(info, dict) or not {"dtype", "shape", "data_offsets"} <= set(info):
                raise CheckpointCorruptError(f"{self.path}: entry {name!r} lacks dtype, shape or data_offsets")
            token = info["dtype"]
            if isinstance(token, str) and token in _UNSUPPORTED_TOKENS:
                raise UnsupportedWeightFormatError(
                    f"{self.path}: entry {name!r} is stored as {token}: packed and quantized weight formats "
                    f"are not supported (readable: {sorted(_ITEMSIZE)})")
            if not isinstance(token, str) or token not in _ITEMSIZE:
                raise CheckpointCorruptError(f"{self.path}: entry {name!r} has unsupported dtype {token!r}")
            shape = info["shape"]
            if not isinstance(shape, list) or any(isinstance(s, bool) or not isinstance(s, int) or s < 0 for s in shape):
                raise CheckpointCorruptError(f"{self.path}: entry {name!r} has a bad shape {shape!r}")
            offs = info["data_offsets"]
            if (not isinstance(offs, list) or len(offs) != 2
                    or any(isinstance(o, bool) or not isinstance(o, int) for o in offs)):
                raise CheckpointCorruptError(f"{self.path}: entry {name!r} has bad data_offsets {offs!r}")
            begin, end = offs
            if not 0 <= begin <= end <= payload:
                raise CheckpointCorruptError(
                    f"{self.path}: entry {name!r} spans [{begin}, {end}) outside a payload of {payload} bytes")
            numel = 1
            for s in shape:
                numel *= s
            if end - begin != numel * _ITEMSIZE[token]:
                raise CheckpointCorruptError(
                    f"{self.path}: entry {name!r} holds {end - begin} bytes, "
                    f"shape {shape} of {token} needs {numel * _ITEMSIZE[token]}")
            self.entries[name] = TensorEntry(name, token, tuple(shape), begin, end)
            if end > begin:
                spans.append((begin, end, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise CheckpointCorruptError(f"{self.path}: entries {n0!r} and {n1!r} overlap")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def read(self, name: str) -> torch.Tensor:
        """A fresh CPU tensor (its own memory) with the stored dtype and shape."""
        e = self.entries[name]
        lo = self.payload_start + e.begin
        count = (e.end - e.begin) // _ITEMSIZE[e.dtype]
        arr = np.frombuffer(self._map, dtype=_NUMPY[e.dtype], count=count, offset=lo).copy()
        t = torch.from_numpy(arr)
        if e.dtype == "BF16":
            t = t.view(torch.bfloat16)
        return t.reshape(e.shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Writes CPU tensors in the order given; offsets are contiguous."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _TOKEN_OF:
            raise ValueError(f"{name}: dtype {t.dtype} cannot be stored")
        raw = (t.view(torch.uint16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _TOKEN_OF[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for raw in blobs:
            fh.write(raw)
