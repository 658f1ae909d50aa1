"""Feed-forward parts."""
from __future__ import annotations

from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .. import kernels
from .base import FeedForward
from .linear import linear

ACTIVATIONS = ("gelu_new", "gelu")
# rules for the (gate, up) pair of a gated feed-forward: an activation on the gate, or the clamped rule
PAIR_RULES = ACTIVATIONS + ("swish_clamp",)


class DenseFeedForward(FeedForward):
    """down(act(up(x))), added to the residual stream (src/feed_forward.rs:111-114 of the reference).
    `gelu_new` is the tanh form, `gelu` the erf form; both are evaluated in 32-bit on the
    accumulator and rounded once."""

    accepts_lazy_norm = True
    linear_weights = ("up.weight", "down.weight")

    def __init__(self, width: int, inner: int, activation: str, *, bias: bool = True, init_std: float = 0.02,
                 down_init_std: float | None = None):
        if activation not in ACTIVATIONS:
            raise ValueError(f"activation must be one of {ACTIVATIONS}, found {activation!r}")
        self.width, self.inner, self.activation, self.has_bias = width, inner, activation, bias
        self.init_std = init_std
        self.down_init_std = init_std if down_init_std is None else down_init_std

    def specs(self):
        specs = {"up.weight": TensorSpec((self.width, self.inner), MATRIX, ("normal", self.init_std)),
                 "down.weight": TensorSpec((self.inner, self.width), MATRIX, ("normal", self.down_init_std))}
        if self.has_bias:
            specs["up.bias"] = TensorSpec((self.inner,), VECTOR, ("zeros",))
            specs["down.bias"] = TensorSpec((self.width,), VECTOR, ("zeros",))
        return specs

    def forward(self, ctx, x, residual):
        n = ctx.n_tokens
        hidden = ctx.ws.take((n, self.inner), ctx.dtype)
        linear(ctx, x, self.t_up_weight, self.t_up_bias if self.has_bias else None, hidden, m=n,
               activation=self.activation, w_is_nk=self.nk_up_weight)
        linear(ctx, hidden, self.t_down_weight, self.t_down_bias if self.has_bias else None, residual, m=n,
               residual=residual, w_is_nk=self.nk_down_weight)


class GatedFeedForward(FeedForward):
    """down(act(gate(x)) * up(x)), added to the residual stream; no biases.  The gate and up matrices are one product:
    `gate_up.weight` is [2 * inner, width] (stored [out, in]: the gate's rows, then up's), `down.weight` [width, inner].
    The activation and the product of the two halves are formed in 32-bit and rounded once.  With the rule
    `swish_clamp` the hidden row is g' sigmoid(1.702 g') (u' + 1), g' = min(gate x, limit), u' = up x clamped to
    [-limit, limit]."""

    accepts_lazy_norm = True

    def __init__(self, width: int, inner: int, activation: str = "gelu_new", *, limit: float = 0.0,
                 init_std: float = 0.02, down_init_std: float | None = None):
        if activation not in PAIR_RULES:
            raise ValueError(f"activation must be one of {PAIR_RULES}, found {activation!r}")
        self.width, self.inner, self.activation, self.limit = width, inner, activation, float(limit)
        self.init_std = init_std
        self.down_init_std = init_std if down_init_std is None else down_init_std

    def specs(self):
        return {"gate_up.weight": TensorSpec((2 * self.inner, self.width), MATRIX, ("normal", self.init_std)),
                "down.weight": TensorSpec((self.width, self.inner), MATRIX, ("normal", self.down_init_std))}

    def forward(self, ctx, x, residual):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("a gated feed-forward has no phase in the fused step")
        n = ctx.n_tokens
        mark = ctx.ws.mark()
        both = ctx.ws.take((n, 2 * self.inner), ctx.dtype)
        linear(ctx, x, self.t_gate_up_weight, None, both, m=n, w_is_nk=True)
        hidden = ctx.ws.take((n, self.inner), ctx.dtype)
        kernels.gated_activation(both, hidden, n_rows=n, activation=self.activation, limit=self.limit)
        linear(ctx, hidden, self.t_down_weight, None, residual, m=n, residual=residual, w_is_nk=True)
        ctx.ws.release(mark)


class PolyNormFeedForward(FeedForward):
    """down(act(up(x))) with a polynomial activation over the whole hidden row z:

        act(z) = a N(z) + b N(z^2) + c N(z^3) + e,     N(v) = v / sqrt(mean(v^2) + eps)

    powers element by element, (a, b, c, e) the four numbers of `act`; the activation is formed in 32-bit and rounded
    once (csrc/rowwise.cu).  No biases; `up.weight` [inner, width] and `down.weight` [width, inner] (stored [out, in])."""

    accepts_lazy_norm = True

    def __init__(self, width: int, inner: int, eps: float, *, init_std: float = 0.02, down_init_std: float | None = None):
        self.width, self.inner, self.eps = width, inner, float(eps)
        self.init_std = init_std
        self.down_init_std = init_std if down_init_std is None else down_init_std

    def specs(self):
        return {"up.weight": TensorSpec((self.inner, self.width), MATRIX, ("normal", self.init_std)),
                "act": TensorSpec((4,), VECTOR, ("normal", 0.5)),
                "down.weight": TensorSpec((self.width, self.inner), MATRIX, ("normal", self.down_init_std))}

    def forward(self, ctx, x, residual):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("a polynomial activation has no phase in the fused step")
        n = ctx.n_tokens
        mark = ctx.ws.mark()
        hidden = ctx.ws.take((n, self.inner), ctx.dtype)
        linear(ctx, x, self.t_up_weight, None, hidden, m=n, w_is_nk=True)
        shaped = ctx.ws.take((n, self.inner), ctx.dtype)
        kernels.polynorm(hidden, self.t_act, shaped, self.eps, n_rows=n)
        linear(ctx, shaped, self.t_down_weight, None, residual, m=n, residual=residual, w_is_nk=True)
        ctx.ws.release(mark)
