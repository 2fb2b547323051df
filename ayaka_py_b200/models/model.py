"""The model that a ``ModelSpec`` describes: parts, run order, cache bindings.

Nothing here knows GPT-2.  The model instantiates the parts the spec names,
lists the tensors they hold (for the loader), derives the cache groups from
what the mixers declare, and runs one step: embedding, the run order, final
norm and head on the wanted rows only.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.spec import CacheBinding, CacheGroupSpec
from ..parts.base import (KVNeed, ModelSpec, Part, Source, StateNeed, TensorDecl,
                          make_block, make_part)


@dataclass(frozen=True)
class TensorRow:
    """One tensor of one part and where it comes from."""
    part: Part
    name: str
    decl: TensorDecl
    source: Source


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device="cuda"):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self._rows: list[TensorRow] = []

        def build(part_spec):
            part = make_part(part_spec, dtype, device)
            declared = part.tensors()
            missing = set(declared) - set(part_spec.sources)
            extra = set(part_spec.sources) - set(declared)
            if missing or extra:
                raise ValueError(
                    f"part {part_spec.kind!r}: tensors without a source {sorted(missing)}, "
                    f"sources without a tensor {sorted(extra)}")
            for name, decl in declared.items():
                self._rows.append(TensorRow(part, name, decl, part_spec.sources[name]))
            return part

        self.embedding = build(spec.embedding)
        self.position = build(spec.position)
        self.blocks = []
        for layer in spec.layers:
            names = [name for name, _ in layer.parts]
            if len(set(names)) != len(names):
                raise ValueError(f"a layer names a part twice: {names}")
            parts = {name: build(part_spec) for name, part_spec in layer.parts}
            for part in parts.values():
                part.set_position(self.position)
            self.blocks.append(make_block(layer.block, parts))
        self.final_norm = build(spec.final_norm)
        self.head = build(spec.head)

        # Cache groups: parts (of any run step) that declare the same need share a group (one
        # namespace of pages and one block table, or one region of state slots); each keeps its
        # own layer index inside the group.  ``bindings[i]``: part name -> binding, for run step i.
        self.groups: list[CacheGroupSpec] = []
        self.bindings: list[dict[str, CacheBinding]] = []
        counts: list[int] = []
        for index, step in enumerate(spec.order):
            if not 0 <= step.layer < len(self.blocks):
                raise ValueError(f"run step {index} names layer {step.layer}, the model has {len(self.blocks)}")
            needs = {name: part.cache_need() for name, part in self.blocks[step.layer].parts.items()}
            needs = {name: need for name, need in needs.items() if need is not None}
            if step.cache_of is not None:
                if not 0 <= step.cache_of < index or not self.bindings[step.cache_of]:
                    raise ValueError(f"run step {index}: cache_of must name an earlier run step with a cache")
                theirs = self.bindings[step.cache_of]
                if set(theirs) != set(needs) or any(self.groups[theirs[n].group].need != needs[n] for n in needs):
                    raise ValueError(f"run step {index} reads a cache of another geometry")
                self.bindings.append({n: CacheBinding(b.group, b.name, b.layer, writes=False) for n, b in theirs.items()})
                continue
            mine: dict[str, CacheBinding] = {}
            for name, need in needs.items():
                if not isinstance(need, (KVNeed, StateNeed)):
                    raise TypeError(f"cache_need() of {type(self.blocks[step.layer].parts[name]).__name__} "
                                    f"must be KVNeed, StateNeed or None")
                for g, group in enumerate(self.groups):
                    if group.need == need:
                        break
                else:
                    g = len(self.groups)
                    self.groups.append(CacheGroupSpec(name=f"group{g}", need=need, layers=0))
                    counts.append(0)
                mine[name] = CacheBinding(g, self.groups[g].name, counts[g], writes=True)
                counts[g] += 1
            self.bindings.append(mine)
        self.groups = [CacheGroupSpec(g.name, g.need, counts[i]) for i, g in enumerate(self.groups)]
        self.loaded = False

    # ---------------------------------------------------------------- facts --
    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    @property
    def max_positions(self) -> int:
        return self.spec.max_positions

    def tensor_rows(self) -> list[TensorRow]:
        return list(self._rows)

    def parts(self):
        seen = []
        for row in self._rows:
            if all(row.part is not p for p in seen):
                seen.append(row.part)
        return seen

    def weight_bytes(self) -> int:
        """Bytes of every distinct bound tensor (a tied table counts once)."""
        seen, total = set(), 0
        for row in self._rows:
            t = getattr(row.part, row.name.replace(".", "_"), None)
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ run --
    def forward(self, ctx) -> torch.Tensor:
        """One step.  Returns logits [S, V] float32 at ``ctx.want_rows``."""
        if not self.loaded:
            raise RuntimeError("the model has no weights yet")
        x = self.embedding.forward(ctx, self.position)
        for step, caches in zip(self.spec.order, self.bindings):
            x = self.blocks[step.layer].forward(x, ctx, caches)
        if ctx.num_wanted == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=x.device)
        h = self.final_norm.forward(x, ctx, rows=ctx.want_rows)
        return self.head.forward(h, ctx)
