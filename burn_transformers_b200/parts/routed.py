"""A feed-forward of routed experts."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import ShapeError
from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .base import FeedForward


class RoutedFeedForward(FeedForward):
    """`n_experts` small feed-forwards of which every token uses `top`, and optionally one that every token uses.

        s = sigmoid(W_r h)                              router, summed in 32-bit
        experts lie in `n_groups` equal groups of neighbours; a group's score is the sum of its two largest s; only the
        experts of the `keep` best groups can be chosen; of those the `top` largest s are
        weight_e = s_e / (sum of the chosen s + 1e-20) * scale
        y = sum over the chosen e of weight_e * down_e(pair(gate_e h, up_e h))  (+ shared(h))

    `pair` is a rule of parts.feed_forward.PAIR_RULES (`swish_clamp` with `limit`: g' sigmoid(1.702 g') (u' + 1), g' =
    min(g, limit), u' = u clamped to +-limit).  The (token, expert) pairs are sorted by expert on the device, the
    experts' products run over the sorted rows (csrc/moe.cu), and the weighted results are summed per token in the order
    of its choices; nothing is read back by the host, so the step can be recorded as a CUDA graph.

    Other routers and experts, by argument:

        router="softmax"     s = softmax(W_r h) over all experts
        choice_bias=True     the experts are chosen by s + `router.correction`; the weights still come from s
        normalise=False      weight_e = s_e, the chosen scores as they are
        identity=k           the router has k more outputs, experts without tensors whose result is their input: a
                             token that chooses one gets weight_e * h (h in 32-bit: `forward(..., x32=)`)
        gated=False          an expert is down_e(act(up_e h)) with `activation` one of kernels.ACTIVATIONS

    Tensors: `router.weight` [experts + identity, width]; `router.correction` [experts + identity] (with `choice_bias`);
    `in.weight` [experts * 2 * inner, width] (per expert the gate's rows, then up's; without a gate [experts * inner,
    width]); `out.weight` [experts * width, inner].  `shared` is a feed-forward part of its own.
    """

    accepts_lazy_norm = False

    def __init__(self, width: int, n_experts: int, top: int, inner: int, *, activation: str = "swish_clamp",
                 limit: float = 0.0, n_groups: int = 1, keep: int = 1, scale: float = 1.0, shared: FeedForward | None = None,
                 init_std: float = 0.02, down_init_std: float | None = None, router: str = "sigmoid",
                 choice_bias: bool = False, normalise: bool = True, identity: int = 0, gated: bool = True):
        if min(width, n_experts, top, inner, n_groups, keep) <= 0:
            raise ShapeError("routed feed-forward: sizes must be positive")
        if identity < 0 or (identity and n_groups != 1) or router not in ("sigmoid", "softmax"):
            raise ShapeError("routed feed-forward: experts without tensors go with one group of experts; the router is "
                             "`sigmoid` or `softmax`")
        if (n_experts + identity) % n_groups or keep > n_groups or top > keep * ((n_experts + identity) // n_groups):
            raise ShapeError(f"routed feed-forward: {n_experts} experts in {n_groups} groups of which {keep} are kept "
                             f"cannot give {top} experts a token")
        if n_experts + identity > 1024 or top > 32:
            raise ShapeError("routed feed-forward: the router kernel takes up to 1024 experts and 32 a token")
        if activation not in (kernels.PAIR_RULES if gated else kernels.ACTIVATIONS):
            raise ShapeError(f"routed feed-forward: unknown rule {activation!r}")
        self.width, self.n_experts, self.top, self.inner = width, n_experts, top, inner
        self.activation, self.limit = activation, float(limit)
        self.n_groups, self.keep, self.scale, self.shared = n_groups, keep, float(scale), shared
        self.router, self.has_choice_bias, self.normalise = router, choice_bias, normalise
        self.identity, self.gated = int(identity), gated
        self.in_rows = (2 if gated else 1) * inner          # rows of an expert's first matrix
        self.init_std = init_std
        self.down_init_std = inner ** -0.5 if down_init_std is None else down_init_std

    def specs(self):
        e, routes = self.n_experts, self.n_experts + self.identity
        specs = {"router.weight": TensorSpec((routes, self.width), MATRIX, ("normal", self.init_std)),
                 "in.weight": TensorSpec((e * self.in_rows, self.width), MATRIX, ("normal", self.init_std)),
                 "out.weight": TensorSpec((e * self.width, self.inner), MATRIX, ("normal", self.down_init_std))}
        if self.has_choice_bias:
            specs["router.correction"] = TensorSpec((routes,), VECTOR, ("normal", 0.05))
        return specs

    def parts(self):
        return {} if self.shared is None else {"shared": self.shared}

    @property
    def graph_safe(self):
        return self.shared is None or self.shared.graph_safe

    def bind(self, tensors):
        super().bind(tensors)
        self.w_in = self.t_in_weight.view(self.n_experts, self.in_rows, self.width)
        self.w_out = self.t_out_weight.view(self.n_experts, self.width, self.inner)

    @property
    def wants_x32(self) -> bool:
        """Whether `forward` needs the 32-bit rows beside the rounded ones (experts that hand their input on)."""
        return self.identity > 0

    # `forward(..., store=True)` writes the result into `residual` instead of adding it (rows that hold nothing yet)
    can_store = True

    def forward(self, ctx, x, residual, x32=None, store=False):
        self.forward_routed(ctx, x, residual, x32, store)
        if self.shared is not None:
            self.shared.forward(ctx, x, residual)

    def forward_routed(self, ctx, x, residual, x32=None, store=False):
        """The routed experts alone (the shared one is a feed-forward of its own and may run beside them)."""
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("routed experts have no phase in the fused step")
        n, top, e = ctx.n_tokens, self.top, self.n_experts
        routes = e + self.identity
        if self.identity and x32 is None:
            if x.dtype != torch.float32:
                raise ShapeError("routed feed-forward: experts that hand their input on need the 32-bit rows (x32)")
            x32 = x
        pairs = n * top
        mark = ctx.ws.mark()
        ids = ctx.ws.take((n, top), torch.int32)
        weights = ctx.ws.take((n, top), torch.float32)
        kernels.moe_route(x, self.t_router_weight, ids, weights, n_tokens=n, top=top, n_groups=self.n_groups,
                          keep=self.keep, scale=self.scale, rule=self.router,
                          choice_bias=self.t_router_correction if self.has_choice_bias else None, normalise=self.normalise)
        # (the pairs of experts without tensors sort behind the others' rows, where no product looks)
        offsets = ctx.ws.take((routes + 1,), torch.int32)
        tile_first = ctx.ws.take((routes + 1,), torch.int32)
        order = ctx.ws.take((pairs,), torch.int32)
        place = ctx.ws.take((pairs,), torch.int32)
        kernels.moe_sort(ids, offsets, tile_first, order, place, pairs=pairs, n_experts=routes)
        hidden = ctx.ws.take((pairs, self.inner), ctx.dtype)
        kernels.moe_expert(True, x, self.w_in, hidden, offsets, tile_first, order, None, pairs=pairs, top=top,
                           activation=self.activation, limit=self.limit, gated=self.gated)
        part = ctx.ws.take((pairs, self.width), torch.float32)
        kernels.moe_expert(False, hidden, self.w_out, part, offsets, tile_first, order, weights, pairs=pairs, top=top)
        if self.identity:
            kernels.moe_combine(part, place, residual, n_tokens=n, top=top, ids=ids, weights=weights, identity_input=x32,
                                n_stored=e, store=store)
        else:
            kernels.moe_combine(part, place, residual, n_tokens=n, top=top, store=store)
        ctx.ws.release(mark)
