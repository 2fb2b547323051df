"""Binding checkpoint tensors to the parts of a model, by name.

The model lists the tensors its parts hold and where each comes from
(``Model.tensor_rows``).  The loader compares that list with what the
checkpoint offers and raises ONE ``WeightMismatchError`` that lists every
missing tensor, every unexpected tensor and every wrong shape or dtype (the
reference reports per category too, ``model_loader/validate.py:55-173``).  Then
it reads one tensor at a time, brings it into the part's layout (transpose of
Conv1D weights) and dtype, and binds it.  Two parts that name the same source
share one tensor on the device (a tied head).

Dtypes: ``matrix`` tensors are kept in the compute dtype (bfloat16 or
float32), ``vector`` tensors in float32, ``int`` tables in int32.  A stored
dtype may feed a target dtype when they are equal, when float32 is narrowed to
bfloat16 (the deliberate downcast, ``model_loader/validate.py:83-95``), or when
bfloat16 / float16 is widened to float32 (exact; this is what lets the 32-bit
engine read a bfloat16 checkpoint, which the reference would refuse).  Anything
else (float16 read as bfloat16, float64 into anything) is listed as a wrong dtype:
it would produce no shape complaint and wrong values.  A shard that holds
tensors which its index does not list is reported too: they are unexpected.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Protocol

import torch

from .safetensors import CheckpointCorruptError, SafetensorsFile, UnsupportedWeightFormatError  # noqa: F401

_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def dtype_feeds(stored: torch.dtype, target: torch.dtype) -> bool:
    """Whether a stored floating dtype may be converted into ``target``."""
    if stored == target:
        return True
    if target == torch.bfloat16:
        return stored == torch.float32                       # narrowing, on purpose
    if target == torch.float32:
        return stored in (torch.bfloat16, torch.float16)     # widening, exact
    return False


class WeightMismatchError(ValueError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and
    ``wrong`` (shape or dtype) list every problem."""

    def __init__(self, missing, unexpected, wrong):
        self.missing, self.unexpected, self.wrong = list(missing), list(unexpected), list(wrong)
        lines = ["checkpoint does not fit the model:"]

        def section(title, items):
            if items:
                lines.append(f"  {title} ({len(items)}):")
                lines.extend(f"    {item}" for item in items[:40])
                if len(items) > 40:
                    lines.append(f"    ... and {len(items) - 40} more")

        section("missing tensors", self.missing)
        section("unexpected tensors", self.unexpected)
        section("wrong shape or dtype", self.wrong)
        super().__init__("\n".join(lines))


class TensorStore(Protocol):
    def names(self) -> list[str]: ...
    def describe(self, name: str) -> tuple[torch.dtype, tuple[int, ...]]: ...
    def read(self, name: str) -> torch.Tensor: ...


class FolderStore:
    """``model.safetensors``, or the shards that ``model.safetensors.index.json`` names."""

    def __init__(self, folder):
        folder = Path(folder)
        index = folder / "model.safetensors.index.json"
        self.files: list[SafetensorsFile] = []
        self.where: dict[str, SafetensorsFile] = {}
        if index.is_file():
            try:
                weight_map = json.loads(index.read_text(encoding="utf-8"))["weight_map"]
            except (KeyError, json.JSONDecodeError) as exc:
                raise CheckpointCorruptError(f"{index}: not a shard index") from exc
            opened = {}
            for name, shard in weight_map.items():
                if shard not in opened:
                    opened[shard] = SafetensorsFile(folder / shard)
                    self.files.append(opened[shard])
                if name not in opened[shard].entries:
                    raise CheckpointCorruptError(f"{index}: {name!r} is not in shard {shard}")
                self.where[name] = opened[shard]
            # Tensors that a shard holds but the index does not list are offered all the same, so
            # that the check against the model reports them as unexpected instead of passing over them.
            for shard, f in opened.items():
                for name in f.entries:
                    if name not in self.where:
                        self.where[name] = f
                    elif self.where[name] is not f:
                        raise CheckpointCorruptError(f"{index}: {name!r} is stored in more than one shard")
        else:
            single = folder / "model.safetensors"
            if not single.is_file():
                raise FileNotFoundError(f"{folder} holds neither model.safetensors nor an index")
            f = SafetensorsFile(single)
            self.files.append(f)
            self.where = {name: f for name in f.entries}

    def names(self):
        return list(self.where)

    def describe(self, name):
        e = self.where[name].entries[name]
        return e.torch_dtype, e.shape

    def read(self, name):
        return self.where[name].read(name)

    def close(self):
        for f in self.files:
            f.close()


class DictStore:
    """Tensors in memory, by checkpoint name."""

    def __init__(self, tensors: dict[str, torch.Tensor]):
        self.tensors = tensors

    def names(self):
        return list(self.tensors)

    def describe(self, name):
        t = self.tensors[name]
        return t.dtype, tuple(t.shape)

    def read(self, name):
        return self.tensors[name]

    def close(self):
        pass


def _target_dtype(kind: str, compute: torch.dtype) -> torch.dtype:
    if kind == "matrix":
        return compute
    if kind == "vector":
        return torch.float32
    if kind == "int":
        return torch.int32
    raise ValueError(f"unknown tensor kind {kind!r}")


def load_weights(model, store: TensorStore, normalize_name=None, config=None) -> dict:
    """Checks, reads, converts and binds.  Returns a small report."""
    normalize_name = normalize_name or (lambda name, config: name)
    offered: dict[str, str] = {}              # canonical name -> name in the store
    wrong: list[str] = []
    for raw in store.names():
        canon = normalize_name(raw, config)
        if canon is None:
            continue
        if canon in offered:
            wrong.append(f"{canon}: offered twice (as {offered[canon]!r} and {raw!r})")
            continue
        offered[canon] = raw

    rows = model.tensor_rows()
    missing: list[str] = []
    used: set[str] = set()
    for row in rows:
        src = row.source
        if src.name not in offered:
            if src.name not in missing:
                missing.append(src.name)
            continue
        used.add(src.name)
        dtype, shape = store.describe(offered[src.name])
        expect = tuple(reversed(row.decl.shape)) if src.transposed else tuple(row.decl.shape)
        if src.transposed and len(row.decl.shape) != 2:
            wrong.append(f"{src.name}: a transposed source must be a matrix")
        elif tuple(shape) != expect:
            wrong.append(f"{src.name}: shape {tuple(shape)}, the model expects {expect}")
        target = _target_dtype(row.decl.kind, model.dtype)
        if row.decl.kind == "int":
            if dtype not in _INTS:
                wrong.append(f"{src.name}: dtype {dtype}, the model expects an integer table")
        elif not dtype_feeds(dtype, target):
            wrong.append(f"{src.name}: dtype {dtype} cannot feed {target} (allowed: the same dtype, "
                         f"float32 -> bfloat16, bfloat16 or float16 -> float32)")
    unexpected = sorted(name for name in offered if name not in used)
    if missing or unexpected or wrong:
        raise WeightMismatchError(sorted(missing), unexpected, wrong)

    shared: dict[tuple, torch.Tensor] = {}
    per_part: dict[int, tuple[object, dict[str, torch.Tensor]]] = {}
    for row in rows:
        src = row.source
        target = _target_dtype(row.decl.kind, model.dtype)
        key = (src.name, src.transposed, target)
        if key not in shared:
            t = store.read(offered[src.name])
            if src.transposed:
                t = t.t()
            shared[key] = t.to(device=model.device, dtype=target).contiguous()
        per_part.setdefault(id(row.part), (row.part, {}))[1][row.name] = shared[key]
    for part, tensors in per_part.values():
        part.bind(tensors)
    if str(model.device).startswith("cuda"):
        torch.cuda.synchronize()
    model.loaded = True
    return {"tensors": len(shared), "bytes": sum(t.numel() * t.element_size() for t in shared.values())}
