"""From logits rows to tokens: packs the rows' options and calls the kernel.

Stage order of the reference (``sampling/plan.py:274-377``) for the options kept
here: scale by temperature, all-greedy batches take the argmax, other batches
draw per row with greedy rows overridden.  The uniform of a draw is a function
of the request's seed and of how many tokens it has sampled so far, so a
request's tokens do not depend on what else is in the batch.
"""

from __future__ import annotations

from typing import Sequence

import torch

from .. import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device="cuda", max_rows: int = 256):
        self.device = device
        self._allocate(max_rows)

    def _allocate(self, rows: int) -> None:
        pin = torch.cuda.is_available()
        self.rows = rows
        # Two sets, used in turn: the engine may pack the options of the next step while the
        # upload of this step's options still waits in the stream behind this step's kernels.
        self._sets = [(torch.zeros((3, rows), dtype=torch.float32, pin_memory=pin),   # temperature, top_p, min_p
                       torch.zeros((3, rows), dtype=torch.int64, pin_memory=pin),     # seed, offset, top_k
                       torch.zeros((3, rows), dtype=torch.float32, device=self.device),
                       torch.zeros((3, rows), dtype=torch.int64, device=self.device)) for _ in range(2)]
        self._uploaded = [None, None]
        self._turn = 0

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               offsets: Sequence[int], banned: Sequence[tuple[int, int]] = ()) -> torch.Tensor:
        """logits [S, V] float32 (device) -> tokens [S] int32 (device).
        ``banned``: (row, token id) pairs that must not be produced in this step (stop ids
        before a request's ``min_tokens``, ``request/stream.py:130-136``): their logits are
        set to -inf first, for greedy rows and draws alike."""
        S = logits.shape[0]
        if not (len(params) == len(seeds) == len(offsets) == S):
            raise ValueError("one set of options per logits row")
        if banned:
            pairs = torch.tensor(list(banned), dtype=torch.int32).t().contiguous().to(logits.device)
            ops.ban_tokens(logits, pairs[0], pairs[1])
        if all(p.greedy for p in params):
            return ops.sample(logits)
        if S > self.rows:
            self._allocate(max(S, 2 * self.rows))
        self._turn ^= 1
        h_float, h_long, d_float, d_long = self._sets[self._turn]
        if self._uploaded[self._turn] is not None:
            self._uploaded[self._turn].synchronize()       # this set's last upload (two calls ago) has left the host
        for i, p in enumerate(params):
            h_float[0, i] = 0.0 if p.greedy else p.temperature
            h_float[1, i] = p.top_p
            h_float[2, i] = p.min_p
            h_long[0, i] = seeds[i]
            h_long[1, i] = offsets[i]
            h_long[2, i] = p.top_k if p.top_k > 0 else 0
        d_float.copy_(h_float, non_blocking=True)
        d_long.copy_(h_long, non_blocking=True)
        if d_float.is_cuda:
            self._uploaded[self._turn] = torch.cuda.Event()
            self._uploaded[self._turn].record()
        filtered = any(p.filtered and not p.greedy for p in params)
        return ops.sample(logits, d_float[0, :S], d_long[0, :S], d_long[1, :S],
                          top_k=d_long[2, :S] if filtered else None,
                          top_p=d_float[1, :S] if filtered else None,
                          min_p=d_float[2, :S] if filtered else None)
