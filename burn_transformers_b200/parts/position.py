"""Position encodings."""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..weights.spec import MATRIX, TensorSpec
from .base import PositionEncoding


class NoPositions(PositionEncoding):
    """No position signal outside the causal mask."""


class LearnedPositions(PositionEncoding):
    """A learned table added to the token embedding: x0[t] = wte[id] + wpe[position]
    (src/models/gpt2/model.rs:428-450).  The table bounds the longest sequence."""
    adds_to_embedding = True

    def __init__(self, n_positions: int, width: int, init_std: float = 0.02):
        self.n_positions, self.width, self.init_std = n_positions, width, init_std

    def specs(self):
        return {"weight": TensorSpec((self.n_positions, self.width), MATRIX, ("normal", self.init_std))}

    def max_positions(self):
        return self.n_positions


class InterleavedRotary(PositionEncoding):
    """Turns channel pairs of query and key vectors by an angle that grows with the position: the pair (2i, 2i+1),
    i < dims/2, of a vector at position p becomes (u cos a - v sin a, v cos a + u sin a) with a = p * base^(-2i/dims);
    channels from `dims` on pass unchanged.  The frequencies are formed in 64-bit on the host and rounded once; angle,
    sine and cosine are 32-bit on the device.  Owns no tensor.

    `stretch` = (factor, low, high, original) slows the long waves down: with the wavelength l = 2 pi / f of a
    frequency f, f stays where l < original / high, becomes f / factor where l > original / low, and in between is
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    rotates = True

    def __init__(self, dims: int, base: float, stretch: tuple[float, float, float, float] | None = None):
        if dims < 0 or dims % 2:
            raise ValueError(f"a rotation takes an even number of channels, not {dims}")
        self.dims, self.base = int(dims), float(base)
        self.stretch = None if stretch is None else tuple(float(v) for v in stretch)
        if self.stretch is not None and (len(self.stretch) != 4 or self.stretch[0] <= 0 or self.stretch[3] <= 0
                                         or self.stretch[2] <= self.stretch[1]):
            raise ValueError(f"a stretch is (factor > 0, low, high > low, original > 0), not {stretch}")
        self._freq: dict = {}

    def frequencies(self) -> list[float]:
        """The dims / 2 frequencies, in 64-bit."""
        values = [self.base ** (-2.0 * i / self.dims) for i in range(self.dims // 2)]
        if self.stretch is None:
            return values
        factor, low, high, original = self.stretch
        out = []
        for f in values:
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                out.append(f)
            elif wavelength > original / low:
                out.append(f / factor)
            else:
                s = (original / wavelength - low) / (high - low)
                out.append((1.0 - s) * f / factor + s * f)
        return out

    def inv_freq(self, device) -> torch.Tensor:
        """[dims / 2] 32-bit frequencies on `device` (made once per device; before any stream capture: a mixer that
        uses this part asks for them when it is bound)."""
        device = torch.device(device)
        hit = self._freq.get(device)
        if hit is None:
            values = self.frequencies() or [1.0]
            hit = torch.tensor(values, dtype=torch.float64).to(torch.float32).to(device)
            self._freq[device] = hit
        return hit

    def rotate_vectors(self, ctx, src, dst) -> None:
        """dst[t, v, :] = src[t, v, :] turned by the position of token t (views [tokens, vectors, length])."""
        kernels.rotary_interleaved(src, dst, ctx.positions, self.inv_freq(src.device), n_tokens=ctx.n_tokens,
                                   dims=self.dims)

    def rotate(self, ctx, proj, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        n = ctx.n_tokens
        heads = n_heads + n_kv_heads              # queries and keys lie side by side, values after them
        view = proj[:n, :heads * head_dim].view(n, heads, head_dim)
        self.rotate_vectors(ctx, view, view)


class HalfSplitRotary(InterleavedRotary):
    """The same turn with the other pairing: channel i < dims/2 of a vector goes with channel i + dims/2.  Its kernel
    writes 32-bit vectors (a recurrence reads them), can scale the vectors from one index on afterwards (keys), and
    copies the channels that follow the vectors in a row."""

    def rotate_rows(self, ctx, src, dst, *, n_vecs: int, length: int, scaled_from=None, scale: float = 1.0,
                    tail: int = 0) -> None:
        kernels.rotary_half(src, dst, ctx.positions, self.inv_freq(src.device), n_tokens=ctx.n_tokens, n_vecs=n_vecs,
                            length=length, dims=self.dims, scaled_from=scaled_from, scale=scale, tail=tail)

    def rotate_vectors(self, ctx, src, dst) -> None:
        raise NotImplementedError("the half-split rotation writes 32-bit rows: use rotate_rows")

    def rotate(self, ctx, proj, n_heads, n_kv_heads, head_dim) -> None:
        raise NotImplementedError("the half-split rotation writes 32-bit rows: use rotate_rows")
