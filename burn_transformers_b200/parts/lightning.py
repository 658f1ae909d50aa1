"""Linear attention with a per-head decay: a recurrent state instead of cached keys."""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import CacheNeed, StateSpec
from ..errors import ShapeError
from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .base import Mixer
from .linear import linear


class LightningAttention(Mixer):
    """Per head a state S (dim x vdim, 32-bit, zero for a new sequence) that every token updates and reads:

        q = act(W_q h), k = act(W_k h), v = act(W_v h)       act(x) = x * sigmoid(x)
        S_t = decay_i * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t

    with one decay per head and no other scale.  The heads' o_t side by side are RMS-normed together (plain weight, eps
    inside the root), multiplied by sigmoid(W_g h) and projected by W_o into the residual stream.  The recurrence,
    the norm and the gate run in 32-bit (csrc/lightning.cu, csrc/rowwise.cu).  The state is the layer's only cache:
    `StateSpec("s", (heads, dim, vdim))`, one row per live sequence.

    Tensors (stored [out, in]): `in.weight` = rows of W_q, W_k, W_v, W_g; `norm.weight` [heads * vdim];
    `out.weight` [width, heads * vdim].
    """

    accepts_lazy_norm = True

    def __init__(self, width: int, n_heads: int, dim: int, vdim: int, decay, eps: float, *, init_std: float = 0.02,
                 out_init_std: float | None = None):
        decay = [float(d) for d in decay]
        if min(width, n_heads, dim, vdim) <= 0 or len(decay) != n_heads:
            raise ShapeError(f"lightning attention: {n_heads} heads need as many decays, found {len(decay)}")
        if dim > 256:
            raise ShapeError(f"lightning attention: {dim} key channels per head exceed the 256 the recurrence kernel takes")
        self.width, self.n_heads, self.dim, self.vdim, self.decay, self.eps = width, n_heads, dim, vdim, decay, float(eps)
        self.qk_width, self.v_width = n_heads * dim, n_heads * vdim
        self.in_width = 2 * self.qk_width + 2 * self.v_width
        self.init_std = init_std
        self.out_init_std = init_std if out_init_std is None else out_init_std

    def specs(self):
        return {"in.weight": TensorSpec((self.in_width, self.width), MATRIX, ("normal", self.init_std)),
                "norm.weight": TensorSpec((self.v_width,), VECTOR, ("ones",)),
                "out.weight": TensorSpec((self.width, self.v_width), MATRIX, ("normal", self.out_init_std))}

    def bind(self, tensors):
        super().bind(tensors)
        self.decay_device = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(self.t_in_weight.device)

    def cache_need(self):
        return CacheNeed(states=(StateSpec("s", (self.n_heads, self.dim, self.vdim), torch.float32),))

    def forward(self, ctx, x, residual, entry, owns_cache=True):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("lightning attention has no phase in the fused step")
        if not owns_cache:
            raise ShapeError("lightning attention: a recurrent state cannot be another layer's")
        mark = ctx.ws.mark()      # (this layer's scratch is handed out again to the next one)
        n = ctx.n_tokens
        proj = ctx.ws.take((n, self.in_width), ctx.dtype)
        linear(ctx, x, self.t_in_weight, None, proj, m=n, w_is_nk=True)
        read = ctx.ws.take((n, self.v_width), torch.float32)
        scratch = None
        if ctx.max_new > kernels.LIGHTNING_CHUNK:
            # long runs of new tokens: the chunks of a run are worked side by side (csrc/lightning.cu)
            scratch = ctx.ws.take((kernels.lightning_chunked_scratch_floats(ctx.n_seqs, ctx.max_new, self.n_heads, self.dim,
                                                                            self.vdim),), torch.float32)
        kernels.lightning_scan(proj, 0, self.qk_width, 2 * self.qk_width, ctx.cache.state(entry, "s"), ctx.slots,
                               ctx.seq_start, self.decay_device, read, n_seqs=ctx.n_seqs, n_heads=self.n_heads,
                               dim=self.dim, vdim=self.vdim, max_new=ctx.max_new, scratch=scratch)
        mixed = ctx.ws.take((n, self.v_width), ctx.dtype)
        kernels.rmsnorm(read, self.t_norm_weight, mixed, self.eps, n_rows=n, gate=proj[:, 2 * self.qk_width + self.v_width:])
        linear(ctx, mixed, self.t_out_weight, None, residual, m=n, residual=residual, w_is_nk=True)
        ctx.ws.release(mark)


class Retention(Mixer):
    """Linear attention with one fixed decay per head, rotated queries and keys, and neither softmax nor denominator:

        q = rot(W_q h),  k = rot(W_k h) * dim^-1/2,  v = W_v h          (`positions`: a rotation of the first channels)
        S_t = decay_i * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t

    Each head's o_t is divided by its own root mean square (eps inside the root, no weight); the heads side by side are
    multiplied by g * sigmoid(g), g = W_g h, and projected by W_o into the residual stream.  Rotation, the scale, the
    recurrence, the norm and the gate run in 32-bit (csrc/rowwise.cu, csrc/lightning.cu): the rotated vectors are
    written as 32-bit rows, which the recurrence reads as they are.  The state is the layer's only cache:
    `StateSpec("s", (heads, dim, vdim))`, one row per live sequence.

    Tensors (stored [out, in]): `in.weight` = rows of W_q, W_k, W_v, W_g; `out.weight` [width, heads * vdim].
    """

    accepts_lazy_norm = True

    def __init__(self, width: int, n_heads: int, dim: int, vdim: int, decay, eps: float, positions, *,
                 key_scale: float | None = None, init_std: float = 0.02, out_init_std: float | None = None):
        decay = [float(d) for d in decay]
        if min(width, n_heads, dim, vdim) <= 0 or len(decay) != n_heads:
            raise ShapeError(f"retention: {n_heads} heads need as many decays, found {len(decay)}")
        if dim > 256:
            raise ShapeError(f"retention: {dim} key channels per head exceed the 256 the recurrence kernel takes")
        if positions.dims > dim:
            raise ShapeError(f"retention: {positions.dims} rotated channels of {dim}")
        self.width, self.n_heads, self.dim, self.vdim, self.decay, self.eps = width, n_heads, dim, vdim, decay, float(eps)
        self.positions = positions
        self.key_scale = dim ** -0.5 if key_scale is None else float(key_scale)
        self.qk_width, self.v_width = n_heads * dim, n_heads * vdim
        self.in_width = 2 * self.qk_width + 2 * self.v_width
        self.g_off = 2 * self.qk_width + self.v_width
        self.init_std = init_std
        self.out_init_std = init_std if out_init_std is None else out_init_std

    def specs(self):
        return {"in.weight": TensorSpec((self.in_width, self.width), MATRIX, ("normal", self.init_std)),
                "out.weight": TensorSpec((self.width, self.v_width), MATRIX, ("normal", self.out_init_std))}

    def bind(self, tensors):
        super().bind(tensors)
        device = self.t_in_weight.device
        self.decay_device = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(device)
        self.unit_weight = torch.ones(self.v_width, dtype=torch.float32, device=device)
        self.positions.inv_freq(device)       # (made now: not inside a stream capture)

    def cache_need(self):
        return CacheNeed(states=(StateSpec("s", (self.n_heads, self.dim, self.vdim), torch.float32),))

    def forward(self, ctx, x, residual, entry, owns_cache=True):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("retention has no phase in the fused step")
        if not owns_cache:
            raise ShapeError("retention: a recurrent state cannot be another layer's")
        mark = ctx.ws.mark()
        n = ctx.n_tokens
        proj = ctx.ws.take((n, self.in_width), ctx.dtype)
        linear(ctx, x, self.t_in_weight, None, proj, m=n, w_is_nk=True)
        # q and k turned and k scaled, v beside them, all 32-bit
        turned = ctx.ws.take((n, self.g_off), torch.float32)
        self.positions.rotate_rows(ctx, proj, turned, n_vecs=2 * self.n_heads, length=self.dim, scaled_from=self.n_heads,
                                   scale=self.key_scale, tail=self.v_width)
        read = ctx.ws.take((n, self.v_width), torch.float32)
        scratch = None
        if ctx.max_new > kernels.LIGHTNING_CHUNK:
            scratch = ctx.ws.take((kernels.lightning_chunked_scratch_floats(ctx.n_seqs, ctx.max_new, self.n_heads, self.dim,
                                                                            self.vdim),), torch.float32)
        kernels.lightning_scan(turned, 0, self.qk_width, 2 * self.qk_width, ctx.cache.state(entry, "s"), ctx.slots,
                               ctx.seq_start, self.decay_device, read, n_seqs=ctx.n_seqs, n_heads=self.n_heads,
                               dim=self.dim, vdim=self.vdim, max_new=ctx.max_new, scratch=scratch, activation=None)
        mixed = ctx.ws.take((n, self.v_width), ctx.dtype)
        kernels.rmsnorm(read, self.unit_weight, mixed, self.eps, n_rows=n, gate=proj[:, self.g_off:], groups=self.n_heads,
                        gate_rule="swish")
        linear(ctx, mixed, self.t_out_weight, None, residual, m=n, residual=residual, w_is_nk=True)
        ctx.ws.release(mark)
