"""A learned blend of every row with the row of the token before it."""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import StateSpec
from ..weights.spec import VECTOR, TensorSpec
from .base import Part


class TokenShift(Part):
    """h[t] <- h[t] + (h[t - 1] - h[t]) * weight, channel by channel, with the rows as they came in; the row before a
    sequence's first token is zero.  The last incoming row of a sequence is kept as the per-sequence state `state_name`
    of the layer's cache entry (zeroed when the slot is released), so a step continues where the one before ended.
    32-bit arithmetic; the result is rounded once to the type the next product reads."""

    state_name = "shift_prev"

    def __init__(self, width: int):
        self.width = width

    def specs(self):
        return {"weight": TensorSpec((self.width,), VECTOR, ("normal", 0.3))}

    def states(self) -> tuple[StateSpec, ...]:
        return (StateSpec(self.state_name, (self.width,), torch.float32),)

    def forward(self, ctx, x32, out, entry: int) -> None:
        kernels.token_shift(x32, self.t_weight, ctx.cache.state(entry, self.state_name), ctx.slots, ctx.seq_start,
                            ctx.token_seq, out, n_rows=ctx.n_tokens)
