"""Position encodings.  GPT-2 uses a learned table of absolute positions that
is added to the token embedding; ``NoPositions`` adds nothing."""

from __future__ import annotations

import torch

from .base import PositionEncoding, TensorDecl, register_part


class LearnedPositions(PositionEncoding):
    KIND = "learned_positions"

    def __init__(self, positions: int, width: int, dtype=torch.float32, device="cuda"):
        self.positions, self.width = positions, width
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.positions, self.width), "matrix")}

    def embedding_table(self):
        return self.weight

    def max_positions(self):
        return self.positions


class NoPositions(PositionEncoding):
    KIND = "no_positions"

    def __init__(self, dtype=torch.float32, device="cuda"):
        pass


register_part(LearnedPositions.KIND, LearnedPositions)
register_part(NoPositions.KIND, NoPositions)
