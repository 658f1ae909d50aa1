"""A selective state-space layer: a per-channel recurrence whose step size and in/out vectors depend on the token."""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import CacheNeed, StateSpec
from ..errors import ShapeError
from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .base import Mixer
from .linear import linear


def _round_up(n: int, to: int) -> int:
    return -(-n // to) * to


class SelectiveScan(Mixer):
    """Per channel c of `inner` and state index n of `n_state` a 32-bit state S (zero for a new sequence):

        [x | z] = W_in h
        x = silu(conv(x) + b_conv)                       a causal convolution per channel over `taps` tokens
        [r | B | C] = W_x x                              r: dt_rank numbers, B and C: n_state each
        dt = softplus(W_dt r + b_dt)                     one step size a channel
        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,   A = -exp(A_log)
        y_c = sum_n S[c, n] C_n + D_c x_c,   then y * silu(z), W_o, times `out_scale`

    Step sizes, decays, the state and every sum of the recurrence are 32-bit (csrc/selective_scan.cu); the convolution
    keeps the last taps - 1 projected rows of a sequence (csrc/short_conv.cu).  The cache: states "scan"
    (inner, n_state) and "x_taps" (taps - 1, inner).

    Tensors: `in.weight` [2 * inner, width]; `conv.weight` [inner, taps], `conv.bias` [inner]; `x.weight`
    [dt_rank + 2 * n_state rounded up to a multiple of 8 (zero rows), inner]; `dt.weight` [inner, dt_rank], `dt.bias`
    [inner]; `A_log` [inner, n_state]; `D` [inner]; `out.weight` [width, inner].
    """

    accepts_lazy_norm = True
    MAX_TAPS = 16

    def __init__(self, width: int, inner: int, n_state: int, dt_rank: int, taps: int, *, out_scale: float = 1.0,
                 init_std: float = 0.02, out_init_std: float | None = None):
        if min(width, inner, n_state, dt_rank) <= 0:
            raise ShapeError("selective scan: sizes must be positive")
        if n_state > 512 or dt_rank > 160:
            raise ShapeError(f"selective scan: {n_state} state indices (at most 512) and a step-size rank of {dt_rank} "
                             f"(at most 160) are what its kernels take")
        if not 1 <= taps <= self.MAX_TAPS:
            raise ShapeError(f"short convolution: {taps} taps are outside 1..{self.MAX_TAPS}")
        self.width, self.inner, self.n_state, self.dt_rank, self.taps = width, inner, n_state, dt_rank, taps
        self.out_scale = float(out_scale)
        self.low_width = _round_up(dt_rank + 2 * n_state, 8)
        self.init_std = init_std
        self.out_init_std = init_std if out_init_std is None else out_init_std

    def specs(self):
        inner = self.inner
        return {"in.weight": TensorSpec((2 * inner, self.width), MATRIX, ("normal", self.init_std)),
                "conv.weight": TensorSpec((inner, self.taps), VECTOR, ("normal", self.taps ** -0.5)),
                "conv.bias": TensorSpec((inner,), VECTOR, ("normal", 0.1)),
                "x.weight": TensorSpec((self.low_width, inner), MATRIX, ("normal", inner ** -0.5)),
                "dt.weight": TensorSpec((inner, self.dt_rank), VECTOR, ("normal", self.dt_rank ** -0.5)),
                "dt.bias": TensorSpec((inner,), VECTOR, ("normal", 0.5)),
                "A_log": TensorSpec((inner, self.n_state), VECTOR, ("normal", 0.5)),
                "D": TensorSpec((inner,), VECTOR, ("ones",)),
                "out.weight": TensorSpec((self.width, inner), MATRIX, ("normal", self.out_init_std))}

    def bind(self, tensors):
        super().bind(tensors)
        for name in ("t_conv_weight", "t_dt_weight", "t_A_log"):
            setattr(self, name, getattr(self, name).contiguous())
        self.no_state = torch.empty((1, 0, self.inner), dtype=torch.float32, device=self.t_in_weight.device)

    def cache_need(self):
        states = (StateSpec("scan", (self.inner, self.n_state), torch.float32),)
        if self.taps > 1:
            states += (StateSpec("x_taps", (self.taps - 1, self.inner), torch.float32),)
        return CacheNeed(states=states)

    def forward(self, ctx, x, residual, entry, owns_cache=True):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("a selective scan has no phase in the fused step")
        if not owns_cache:
            raise ShapeError("selective scan: a recurrent state cannot be another layer's")
        mark = ctx.ws.mark()
        n, dtype, inner = ctx.n_tokens, ctx.dtype, self.inner
        xz = ctx.ws.take((n, 2 * inner), dtype)
        linear(ctx, x, self.t_in_weight, None, xz, m=n, w_is_nk=True)
        xc = ctx.ws.take((n, inner), dtype)
        taps_state = ctx.cache.state(entry, "x_taps") if self.taps > 1 else self.no_state
        kernels.short_conv(xz[:, :inner], self.t_conv_weight, self.t_conv_bias, taps_state, ctx.slots, ctx.seq_start,
                           ctx.token_seq, xc, n_tokens=n, n_seqs=ctx.n_seqs, activation="swish")
        low = ctx.ws.take((n, self.low_width), dtype)
        linear(ctx, xc, self.t_x_weight, None, low, m=n, w_is_nk=True)
        dt = ctx.ws.take((n, inner), torch.float32)
        kernels.selective_scan_dt(low, self.t_dt_weight, self.t_dt_bias, dt, n_tokens=n)
        y = ctx.ws.take((n, inner), dtype)
        scratch = None
        need = kernels.selective_scan_pieces(ctx.max_new, n, ctx.n_seqs, inner, self.n_state)[2]
        if need:
            scratch = ctx.ws.take((need,), torch.float32)
        kernels.selective_scan(xc, xz[:, inner:], dt, low, self.dt_rank, self.dt_rank + self.n_state, self.t_A_log,
                               self.t_D, ctx.cache.state(entry, "scan"), ctx.slots, ctx.seq_start, y, n_seqs=ctx.n_seqs,
                               out_scale=self.out_scale, max_new=ctx.max_new, scratch=scratch)
        linear(ctx, y, self.t_out_weight, None, residual, m=n, residual=residual, w_is_nk=True)
        ctx.ws.release(mark)
