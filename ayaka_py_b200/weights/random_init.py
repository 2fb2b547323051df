"""The random-weights mode: tensors drawn from a configuration and a seed.

Every distinct source tensor of the model is drawn in checkpoint layout, in the
order in which the model lists it, from one seeded CPU generator:
``mean + std * N(0, 1)`` with the ``Init`` that the architecture attached to the
source.  ``write_random_model`` writes ``config.json`` and ``model.safetensors``;
loading that folder goes through the ordinary loader.  (The reference's writer
draws every tensor as ``randn * 0.02``, ``models/_common.py:383-427``.)
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config.model import ModelConfig
from ..models.model import Model
from ..registry import Architecture, architecture_for
from .safetensors import write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(arch: Architecture, config: ModelConfig, seed: int,
                   dtype: str = "bfloat16", device="cpu") -> dict[str, torch.Tensor]:
    """Checkpoint name -> tensor.  Matrices in ``dtype``, vectors in float32,
    integer tables int32.  With ``device`` a CUDA device the values are drawn
    there (another stream of numbers than on the CPU, same distributions)."""
    store_dtype = _DTYPES[dtype]
    model = Model(arch.build_spec(config), store_dtype, device="meta")
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for row in model.tensor_rows():
        src = row.source
        if src.name in out:
            continue
        shape = tuple(reversed(row.decl.shape)) if src.transposed else tuple(row.decl.shape)
        if row.decl.kind == "int":
            out[src.name] = torch.zeros(shape, dtype=torch.int32, device=device)
            continue
        t = torch.randn(shape, generator=gen, dtype=torch.float32, device=device)
        t.mul_(src.init.std).add_(src.init.mean)
        out[src.name] = t.to(store_dtype) if row.decl.kind == "matrix" else t
    return out


def write_random_model(folder, config: ModelConfig, seed: int, dtype: str = "bfloat16") -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    document = config.to_dict()
    document["torch_dtype"] = dtype
    arch = architecture_for(document)
    (folder / "config.json").write_text(json.dumps(document, indent=2), encoding="utf-8")
    write_safetensors(folder / "model.safetensors", random_tensors(arch, config, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
