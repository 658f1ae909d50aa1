"""Arrangements of norms, a mixer and a feed-forward in one layer."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Block, FeedForward, Mixer, Norm


class PreNormBlock(Block):
    """x + mixer(norm1(x)), then y + feed_forward(norm2(y)); no post-norms
    (src/models/gpt2/model.rs:218-270 of the reference).  A layer without a feed-forward (`norm2` and `feed_forward`
    None) has the first sublayer only."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm | None = None, feed_forward: FeedForward | None = None):
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("a block has both a second norm and a feed-forward, or neither")
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        found = {"norm1": self.norm1, "mixer": self.mixer}
        if self.feed_forward is not None:
            found.update({"norm2": self.norm2, "feed_forward": self.feed_forward})
        return found

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts().values())

    def forward(self, ctx, residual, entry, owns_cache=True):
        x = self.norm1.forward(ctx, residual, ctx.dtype, lazy=self.mixer.accepts_lazy_norm)
        self.mixer.forward(ctx, x, residual, entry, owns_cache)
        if self.feed_forward is None:
            return
        x = self.norm2.forward(ctx, residual, ctx.dtype, lazy=self.feed_forward.accepts_lazy_norm)
        self.feed_forward.forward(ctx, x, residual)


class ParallelBlock(Block):
    """x + mixer(h) + feed_forward(h) with h = norm(x): one norm whose output both sublayers read, both results added
    to the stream.  A layer without a feed-forward has the mixer only."""

    def __init__(self, norm: Norm, mixer: Mixer, feed_forward: FeedForward | None = None):
        self.norm, self.mixer, self.feed_forward = norm, mixer, feed_forward

    def parts(self):
        found = {"norm": self.norm, "mixer": self.mixer}
        for name, part in getattr(self.mixer, "parts", dict)().items():
            found["mixer." + name] = part
        if self.feed_forward is not None:
            found["feed_forward"] = self.feed_forward
            for name, part in getattr(self.feed_forward, "parts", dict)().items():
                found["feed_forward." + name] = part
        return found

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts().values())

    # Steps of at most this many tokens run the layer's independent parts side by side: each part but the first on a
    # stream of its own, adding into a zeroed buffer of its own; when all are done, one kernel adds the buffers to the
    # stream in a fixed order.  A decode step is a chain of short kernels, and its time is the length of the longest
    # chain, not the number of kernels (Gokezen of 12 x 768 at 8 sequences: 0.96 to 0.70 ms); prompts of a few thousand
    # tokens still gain where a part's kernels leave multiprocessors idle (2 x 1,024 tokens: 3.84 to 3.36 ms; 8 x 512:
    # 5.86 to 5.68 ms).  Longer steps fill the GPU with every kernel and run in order; the scratch a layer holds while
    # its parts run grows with the step.
    side_by_side_up_to = 4096
    _streams: dict = {}

    def _branches(self, entry, owns_cache):
        """The parts of the layer that need nothing of one another, as calls (ctx, x, target)."""
        mixers = list(self.mixer.parts().values()) if hasattr(self.mixer, "left") else [self.mixer]
        found = [lambda ctx, x, target, m=m: m.forward(ctx, x, target, entry, owns_cache) for m in mixers]
        ff = self.feed_forward
        if ff is not None and hasattr(ff, "forward_routed") and ff.shared is not None:
            found += [ff.forward_routed, ff.shared.forward]
        elif ff is not None:
            found.append(ff.forward)
        return found

    @classmethod
    def _sides(cls, device, count):
        from ..engine.step import SideWork
        have = cls._streams.setdefault(torch.device(device), [])
        while len(have) < count:
            have.append(SideWork(device))
        return have[:count]

    def forward(self, ctx, residual, entry, owns_cache=True):
        # (both sublayers read the same rows, so the norm hands out real rows, never a handle for one product)
        n = ctx.n_tokens
        branches = self._branches(entry, owns_cache)
        if (n > self.side_by_side_up_to or len(branches) < 2 or len(branches) > 4 or residual.device.type != "cuda"
                or getattr(ctx, "program", None) is not None):
            x = self.norm.forward(ctx, residual, ctx.dtype, lazy=False)
            for branch in branches:
                branch(ctx, x, residual)
            return
        mark = ctx.ws.mark()
        x = self.norm.forward(ctx, residual, ctx.dtype, lazy=False)
        sides = self._sides(residual.device, len(branches) - 1)
        # no piece of scratch is handed out twice while the branches run, and nothing is left on the step's own second
        # stream that reads a branch's scratch after the layer has given it back
        held, ctx.ws.hold = ctx.ws.hold, True
        step_side, ctx.side = getattr(ctx, "side", None), None
        buffers = []
        try:
            for side, branch in zip(sides, branches[1:]):
                target = ctx.ws.take((n, residual.shape[1]), torch.float32)
                side.fork()
                with side.stream_context():
                    target.zero_()
                    branch(ctx, x, target)
                buffers.append(target)
            branches[0](ctx, x, residual)
        finally:
            for side in sides:
                side.join()
            ctx.ws.hold, ctx.side = held, step_side
        kernels.add_rows(residual, buffers, n_rows=n)
        ctx.ws.release(mark)


class SandwichBlock(Block):
    """A norm before and after each sublayer: x + norm1b(mixer(norm1(x))), then y + norm2b(feed_forward(norm2(y))).

    The sublayers add into a zeroed 32-bit buffer instead of the stream; one kernel then norms the buffer, adds it to
    the stream and, where another sublayer of the layer follows, norms the new row for it in the same pass
    (csrc/rowwise.cu: rmsnorm_add).  All four norms are RMS norms of one eps."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm1b: Norm, norm2: Norm | None = None,
                 feed_forward: FeedForward | None = None, norm2b: Norm | None = None):
        if len({norm2 is None, feed_forward is None, norm2b is None}) != 1:
            raise ValueError("a block has a feed-forward with both of its norms, or none of the three")
        norms = [n for n in (norm1, norm1b, norm2, norm2b) if n is not None]
        if any(getattr(n, "has_bias", True) or n.eps != norm1.eps or not hasattr(n, "offset") for n in norms):
            raise ValueError("the norms around a sublayer are RMS norms with one eps")
        self.norm1, self.mixer, self.norm1b = norm1, mixer, norm1b
        self.norm2, self.feed_forward, self.norm2b = norm2, feed_forward, norm2b

    def parts(self):
        found = {"norm1": self.norm1, "mixer": self.mixer, "norm1b": self.norm1b}
        for name, part in getattr(self.mixer, "parts", dict)().items():
            found["mixer." + name] = part
        if self.feed_forward is not None:
            found.update({"norm2": self.norm2, "feed_forward": self.feed_forward, "norm2b": self.norm2b})
        return found

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts().values())

    def _mixers_side_by_side(self, ctx, x, branch, entry, owns_cache):
        """The two mixers of the layer need nothing of one another: the right one runs on a stream of its own and adds
        into a zeroed buffer of its own, which one kernel then adds to the left one's (as ParallelBlock runs a layer's
        parts; the same streams)."""
        n = ctx.n_tokens
        side, = ParallelBlock._sides(branch.device, 1)
        held, ctx.ws.hold = ctx.ws.hold, True
        step_side, ctx.side = getattr(ctx, "side", None), None
        try:
            other = ctx.ws.take((n, branch.shape[1]), torch.float32)
            side.fork()
            with side.stream_context():
                other.zero_()
                self.mixer.right.forward(ctx, x, other, entry, owns_cache)
            self.mixer.left.forward(ctx, x, branch, entry, owns_cache)
        finally:
            side.join()
            ctx.ws.hold, ctx.side = held, step_side
        kernels.add_rows(branch, [other], n_rows=n)

    def forward(self, ctx, residual, entry, owns_cache=True):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("norms after a sublayer have no phase in the fused step")
        n, width = ctx.n_tokens, residual.shape[1]
        mark = ctx.ws.mark()
        branch = ctx.ws.take((n, width), torch.float32)
        x = self.norm1.forward(ctx, residual, ctx.dtype, lazy=False)
        inner = ctx.ws.mark()
        branch.zero_()
        if hasattr(self.mixer, "left") and n <= ParallelBlock.side_by_side_up_to and residual.device.type == "cuda":
            self._mixers_side_by_side(ctx, x, branch, entry, owns_cache)
        else:
            self.mixer.forward(ctx, x, branch, entry, owns_cache)
        ctx.ws.release(inner)
        if self.feed_forward is None:
            kernels.rmsnorm_add(branch, self.norm1b.t_weight, residual, self.norm1b.eps, n_rows=n)
        else:
            kernels.rmsnorm_add(branch, self.norm1b.t_weight, residual, self.norm1b.eps, n_rows=n,
                                next_weight=self.norm2.t_weight, next_out=x)
            branch.zero_()
            self.feed_forward.forward(ctx, x, branch)
            kernels.rmsnorm_add(branch, self.norm2b.t_weight, residual, self.norm2b.eps, n_rows=n)
        ctx.ws.release(mark)


class OutputNormBlock(Block):
    """The norm stands on a sublayer's OUTPUT only: x + m * norm1(mixer(x)), then y + m * norm2(feed_forward(y)), with m
    one number for the whole model.  The sublayers read the stream itself (rounded to the products' type); with a
    `shift` (parts.token_shift.TokenShift) the mixer reads every row blended with the row of the token before it.

    A sublayer leaves its result in a 32-bit buffer (zeroed first for parts that can only add); one kernel
    (csrc/rowwise.cu: rmsnorm_add) norms the buffer, adds m times the result to the stream and, where the feed-forward
    follows, writes the new row in the products' type for it in the same pass.  Both norms are RMS norms of one eps."""

    def __init__(self, mixer: Mixer, norm1: Norm, feed_forward: FeedForward | None = None, norm2: Norm | None = None,
                 *, scale: float = 1.0, shift=None):
        if (norm2 is None) != (feed_forward is None):
            raise ValueError("a block has both a feed-forward and the norm of its output, or neither")
        norms = [n for n in (norm1, norm2) if n is not None]
        if any(getattr(n, "has_bias", True) or n.eps != norm1.eps or not hasattr(n, "offset") for n in norms):
            raise ValueError("the norms of the sublayers' outputs are RMS norms with one eps")
        self.mixer, self.norm1, self.feed_forward, self.norm2 = mixer, norm1, feed_forward, norm2
        self.scale, self.shift = float(scale), shift

    def parts(self):
        found = {"mixer": self.mixer, "norm1": self.norm1}
        if self.shift is not None:
            found["shift"] = self.shift
        if self.feed_forward is not None:
            found.update({"feed_forward": self.feed_forward, "norm2": self.norm2})
        return found

    def cache_need(self):
        need = self.mixer.cache_need()
        if self.shift is None:
            return need
        import dataclasses
        return dataclasses.replace(need, states=tuple(need.states) + self.shift.states())

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts().values())

    def forward(self, ctx, residual, entry, owns_cache=True):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("a norm on a sublayer's output has no phase in the fused step")
        n, width = ctx.n_tokens, residual.shape[1]
        exact = ctx.dtype == torch.float32
        mark = ctx.ws.mark()
        branch = ctx.ws.take((n, width), torch.float32)
        rows = ctx.ws.take((n, width), ctx.dtype) if (self.shift is not None or not exact) else None
        if self.shift is not None:
            self.shift.forward(ctx, residual, rows, entry)
            x = rows
        elif exact:
            x = residual
        else:
            rows[:n].copy_(residual[:n])
            x = rows
        inner = ctx.ws.mark()
        # (a part that can store its result instead of adding it needs no zeroed buffer: one launch less a sublayer)
        if getattr(self.mixer, "can_store", False):
            self.mixer.forward(ctx, x, branch, entry, owns_cache, store=True)
        else:
            branch.zero_()
            self.mixer.forward(ctx, x, branch, entry, owns_cache)
        ctx.ws.release(inner)
        if self.feed_forward is None:
            kernels.rmsnorm_add(branch, self.norm1.t_weight, residual, self.norm1.eps, n_rows=n, factor=self.scale)
            ctx.ws.release(mark)
            return
        # the feed-forward reads the new rows of the stream: as they are in 32-bit, else rounded by the same kernel
        kernels.rmsnorm_add(branch, self.norm1.t_weight, residual, self.norm1.eps, n_rows=n, factor=self.scale,
                            next_out=None if exact else rows)
        x = residual if exact else rows
        more = {"x32": residual} if getattr(self.feed_forward, "wants_x32", False) else {}
        if getattr(self.feed_forward, "can_store", False) and getattr(self.feed_forward, "shared", None) is None:
            self.feed_forward.forward(ctx, x, branch, store=True, **more)
        else:
            branch.zero_()
            self.feed_forward.forward(ctx, x, branch, **more)
        kernels.rmsnorm_add(branch, self.norm2.t_weight, residual, self.norm2.eps, n_rows=n, factor=self.scale)
        ctx.ws.release(mark)
