"""From a model folder (or a configuration and a seed) to a model with weights."""

from __future__ import annotations

import torch

from .. import models  # noqa: F401  (registers the architectures)
from .. import parts  # noqa: F401   (registers the part kinds)
from ..config.model import ModelConfig
from ..models.model import Model
from ..registry import architecture_for, read_config
from ..weights.loader import DictStore, FolderStore, load_weights
from ..weights.random_init import random_tensors

TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def load_model(folder, dtype: str = "bfloat16", device="cuda") -> tuple[ModelConfig, Model]:
    """The model class is chosen by ``config.json``; weights come from
    ``model.safetensors`` by tensor name."""
    arch, config = read_config(folder)
    model = Model(arch.build_spec(config), TORCH_DTYPES[dtype], device)
    store = FolderStore(folder)
    try:
        load_weights(model, store, arch.normalize_name, config)
    finally:
        store.close()
    return config, model


def random_model(config: ModelConfig, seed: int, dtype: str = "bfloat16", device="cuda",
                 generate_on_device: bool = False) -> Model:
    """The random-weights mode without files: the same tensors that
    ``write_random_model`` writes (when generated on the CPU), bound directly."""
    arch = architecture_for(config.to_dict())
    model = Model(arch.build_spec(config), TORCH_DTYPES[dtype], device)
    tensors = random_tensors(arch, config, seed, dtype="bfloat16" if dtype == "bfloat16" else "float32",
                             device=device if generate_on_device else "cpu")
    load_weights(model, DictStore(tensors), arch.normalize_name, config)
    return model
