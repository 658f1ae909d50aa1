"""Attention with a low-rank latent for keys and values."""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import PAGE_SIZE, CacheNeed, KvSpec
from ..errors import ShapeError
from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .attention import _sm_count
from .base import Mixer
from .linear import linear


class LatentAttention(Mixer):
    """Multi-head causal attention whose keys and values come from one low-rank latent per position.

    With h the mixer's input, per position:

        q       = W_q h                     per head [dim plain | rot_dim rotated] channels
        [d | r] = W_dkv h                   d: kv_rank channels, r: rot_dim channels
        c       = d / rms(d) * norm         the latent (eps inside the root)
        r'      = rotate(r, position)       one rotated key part that all heads share

    Head i has keys [W_uk,i c | r'] and values W_uv,i c; its scores are (q_plain . W_uk,i c + q_rot' . r') * scale,
    causal, with a softmax whose denominator may also hold exp(sink_i): a learned per-head logit that competes for
    weight but contributes nothing to the output.  The heads side by side are multiplied by sigmoid(W_g h) and projected by W_o into the residual stream.

    Only [c | r'] is cached: one row of kv_rank + rot_dim per position for all heads, and it is both key and value
    (`KvSpec(1, kv_rank + rot_dim, has_values=False)`).  The up-projections act on the query side instead
    (csrc/latent_attention.cu): q~_i = W_uk,i^T q_plain,i meets c directly, and W_uv,i acts once on the weighted sum
    of latents.  A layer built with `owns_latent=False` has no W_dkv; the model's run order gives it another layer's
    cache entry, whose rows it reads with its own W_uk, W_uv, queries and everything else.

    By argument: `gate=False` leaves the output gate out; `window` = W lets position i see j with 0 <= i - j < W only;
    `q_rank` = r sends the queries through a latent of their own, c_q = (W_dq h) / rms(W_dq h) * q_norm, q = W_uq c_q
    (then `in.weight` opens with W_dq's r rows in W_q's place, and the part has `q_norm.weight` [r] and `uq.weight`
    [heads * (dim + rot_dim), r]).  A windowed layer keeps every position in its pages all the same: the kernels skip
    the tiles of keys before a block's first visible one.

    Tensors (stored [out, in]): `in.weight` = rows of W_q (or W_dq), then W_g, then (owner only) W_dkv; `uk.weight`
    [heads * dim, kv_rank]; `uv.weight` [heads * vdim, kv_rank]; `latent_norm.weight` [kv_rank] (owner only); `sink`
    [heads] (if `sink`); `out.weight` [width, heads * vdim].
    """

    accepts_lazy_norm = True
    # Prompts of sequences that start at position 0 and bring at least this many tokens take the plain form in bfloat16:
    # keys and values up-projected per head for the step's tokens, then multi-head attention (dim + rot_dim + vdim
    # multiply-adds a key and head instead of 2 kv_rank + rot_dim).  Everything else (decode steps, portions that continue a
    # sequence, 32-bit) reads the latent rows directly.
    plain_from = 48
    # Steps of at most this many tokens (decode steps) run the steps around the attention as two fused kernels
    # (csrc/latent_decode.cu) instead of five launches.
    fused_up_to = 64

    def __init__(self, width: int, n_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float, eps: float,
                 positions, *, owns_latent: bool = True, sink: bool = True, init_std: float = 0.02,
                 out_init_std: float | None = None, gate: bool = True, window: int | None = None,
                 q_rank: int | None = None):
        if min(width, n_heads, dim, vdim, kv_rank) <= 0 or rot_dim < 0:
            raise ShapeError("latent attention: sizes must be positive")
        if kv_rank > 512:
            raise ShapeError(f"latent attention: a latent of {kv_rank} channels exceeds the 512 the attention kernel takes")
        if positions is None or not positions.rotates or positions.dims > rot_dim:
            raise ShapeError("latent attention: needs a rotating position encoding over at most rot_dim channels")
        self.width, self.n_heads, self.dim, self.rot_dim, self.vdim, self.kv_rank = width, n_heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.eps, self.positions = float(scale), float(eps), positions
        if (window is not None and window <= 0) or (q_rank is not None and q_rank <= 0):
            raise ShapeError("latent attention: a window and a query latent are positive")
        self.owns_latent, self.has_sink, self.has_gate = owns_latent, sink, gate
        self.window, self.q_rank = window, q_rank
        self.q_width = n_heads * (dim + rot_dim)
        self.mixed_width = n_heads * vdim
        self.gate_width = self.mixed_width if gate else 0
        self.latent_width = kv_rank + rot_dim
        self.q_in_width = self.q_width if q_rank is None else q_rank      # what the first product gives of the queries
        self.in_width = self.q_in_width + self.gate_width + (self.latent_width if owns_latent else 0)
        self.init_std = init_std
        self.out_init_std = init_std if out_init_std is None else out_init_std

    def specs(self):
        up_std = self.kv_rank ** -0.5
        specs = {"in.weight": TensorSpec((self.in_width, self.width), MATRIX, ("normal", self.init_std)),
                 "uk.weight": TensorSpec((self.n_heads * self.dim, self.kv_rank), MATRIX, ("normal", up_std)),
                 "uv.weight": TensorSpec((self.n_heads * self.vdim, self.kv_rank), MATRIX, ("normal", up_std)),
                 "out.weight": TensorSpec((self.width, self.n_heads * self.vdim), MATRIX, ("normal", self.out_init_std))}
        if self.owns_latent:
            specs["latent_norm.weight"] = TensorSpec((self.kv_rank,), VECTOR, ("ones",))
        if self.has_sink:
            specs["sink"] = TensorSpec((self.n_heads,), VECTOR, ("normal", 1.0))
        if self.q_rank is not None:
            specs["q_norm.weight"] = TensorSpec((self.q_rank,), VECTOR, ("ones",))
            specs["uq.weight"] = TensorSpec((self.q_width, self.q_rank), MATRIX, ("normal", self.q_rank ** -0.5))
        return specs

    def bind(self, tensors):
        super().bind(tensors)
        # per head [K, N] operands of the per-head products: W_uk,i as stored ([dim, kv_rank]), W_uv,i turned
        # ([kv_rank, vdim])
        self.uk_heads = self.t_uk_weight.view(self.n_heads, self.dim, self.kv_rank)
        self.uv_heads = self.t_uv_weight.view(self.n_heads, self.vdim, self.kv_rank).transpose(1, 2).contiguous()
        self.uk_heads_t = self.uk_heads.transpose(1, 2).contiguous()       # [heads, kv_rank, dim]: latent -> plain key
        self.positions.inv_freq(self.t_uk_weight.device)

    def cache_need(self):
        if not self.owns_latent:
            return CacheNeed()
        return CacheNeed(kv=KvSpec(1, self.latent_width, None, has_values=False))

    def _splits(self, ctx, rows_per_block: int) -> int:
        """Runs the keys of a row tile are cut into: enough blocks to fill the GPU about twice, none when the step's
        rows do that by themselves; at most one per 32 keys."""
        hb = min(self.n_heads, rows_per_block)
        tiles = -(-self.n_heads // hb) * -(-ctx.max_new // max(1, rows_per_block // hb)) * ctx.n_seqs
        by_fill = -(-2 * _sm_count(ctx.ws.device) // max(1, tiles))
        span = ctx.ctx_bound if self.window is None else min(ctx.ctx_bound, self.window + 64)
        return int(max(1, min(by_fill, -(-span // 32), 64)))

    # `forward(..., store=True)` writes the result into `residual` instead of adding it (rows that hold nothing yet)
    can_store = True

    def forward(self, ctx, x, residual, entry, owns_cache=True, store=False):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("latent attention has no phase in the fused step")
        if owns_cache != self.owns_latent:
            raise ShapeError("latent attention: a layer with its own latent projection owns its cache entry, and a "
                             "layer without one reads another layer's")
        mark = ctx.ws.mark()      # (this layer's scratch is handed out again to the next one)
        n, dtype, heads = ctx.n_tokens, ctx.dtype, self.n_heads
        rank, rot, dk = self.kv_rank, self.rot_dim, self.latent_width
        proj = ctx.ws.take((n, self.in_width), dtype)
        linear(ctx, x, self.t_in_weight, None, proj, m=n, w_is_nk=True)
        window = self.window or 0
        gate_off, latent_off = self.q_in_width, self.q_in_width + self.gate_width
        if self.q_rank is None:
            queries = proj
        else:
            # the queries out of their own latent: norm of the first q_rank channels, then W_uq
            low = ctx.ws.take((n, self.q_rank), dtype)
            kernels.rmsnorm(proj[:, :self.q_rank], self.t_q_norm_weight, low, self.eps, n_rows=n)
            queries = ctx.ws.take((n, self.q_width), dtype)
            linear(ctx, low, self.t_uq_weight, None, queries, m=n, w_is_nk=True)
        k_pool, _, group, g = ctx.cache.layer_pools(entry)
        if group.spec.head_dim != dk or group.spec.n_kv_heads != 1:
            raise ShapeError(f"latent attention: the cache entry holds rows of {group.spec.n_kv_heads} x "
                             f"{group.spec.head_dim}, this layer reads rows of 1 x {dk}")
        pool = k_pool.view(-1, PAGE_SIZE, dk)
        table = ctx.tables[g]
        freq = self.positions.inv_freq(proj.device)
        if n <= self.fused_up_to:
            # few tokens: query into the latent space + rotation + filing in one launch, the attention, then
            # join of the splits + W_uv + gate in one launch
            q_latent = ctx.ws.take((n, heads * dk), dtype)
            kernels.latent_decode_prep(queries, 0, latent_off, self.uk_heads,
                                       self.t_latent_norm_weight if self.owns_latent else None, self.eps, ctx.positions,
                                       ctx.token_seq, freq, self.positions.dims, table, group.table_len, pool, q_latent,
                                       n_tokens=n, n_heads=heads, dim=self.dim, rank=rank, rot=rot, owns=self.owns_latent,
                                       latent_rows=proj[:, latent_off:] if self.owns_latent and queries is not proj
                                       else None)
            mixed_latent = ctx.ws.take((n, heads * rank), dtype)
            splits = self._splits(ctx, kernels.latent_attention_rows(rank, rot, dtype))
            scratch = None
            if splits > 1:
                scratch = ctx.ws.take((kernels.latent_attention_scratch_floats(n, heads, rank, splits),), torch.float32)
            kernels.latent_attention(q_latent, mixed_latent, pool, table, group.table_len, ctx.seq_start, ctx.past_len,
                                     n_tokens=n, n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=heads, rank=rank, rot=rot,
                                     scale=self.scale, sink=self.t_sink if self.has_sink else None, n_splits=splits,
                                     scratch=scratch, merge=False, window=window)
            mixed = ctx.ws.take((n, self.mixed_width), dtype)
            kernels.latent_decode_finish(self.uv_heads, mixed, n_tokens=n, n_splits=splits, scratch=scratch,
                                         mixed_latent=mixed_latent,
                                         gate=proj[:, gate_off:latent_off] if self.has_gate else None)
            linear(ctx, mixed, self.t_out_weight, None, residual, m=n, residual=None if store else residual, w_is_nk=True)
            ctx.ws.release(mark)
            return
        if self.owns_latent:
            kernels.latent_append(proj[:, latent_off:], self.t_latent_norm_weight, self.eps,
                                  ctx.positions, ctx.token_seq, freq, self.positions.dims, table, group.table_len, pool,
                                  n, rank, rot)
        q_heads = queries[:, :self.q_width].view(n, heads, self.dim + rot)
        gate = proj[:, gate_off:latent_off].view(n, heads, self.vdim) if self.has_gate else None
        if dtype == torch.bfloat16 and ctx.fresh and not ctx.is_decode and ctx.max_new >= self.plain_from:
            # fresh prompts: the step's own latent rows, keys and values per head, ordinary attention
            rows = ctx.ws.take((n, dk), dtype)
            keys = ctx.ws.take((n, heads, self.dim + rot), dtype)
            values = ctx.ws.take((n, heads, self.vdim), dtype)
            mixed = ctx.ws.take((n, self.mixed_width), dtype)
            mixed_heads = mixed.view(n, heads, self.vdim)
            if kernels.sink_attention_supports(q_heads, keys, values, gate, mixed_heads):
                kernels.latent_gather(pool, ctx.positions, ctx.token_seq, table, group.table_len, rows, n_tokens=n)
                latent = rows[:, :rank].unsqueeze(1).expand(n, heads, rank)
                kernels.head_linear(latent, self.uk_heads_t, keys[:, :, :self.dim], n_tokens=n)
                kernels.head_linear(latent, self.uv_heads, values, n_tokens=n)
                if rot:
                    shared = rows[:, rank:].unsqueeze(1).expand(n, heads, rot)
                    kernels.rotary_interleaved(shared, keys[:, :, self.dim:], ctx.positions, freq, n_tokens=n, dims=0)
                    self.positions.rotate_vectors(ctx, q_heads[:, :, self.dim:], q_heads[:, :, self.dim:])
                kernels.sink_attention(q_heads, keys, values, mixed_heads, ctx.seq_start, n_seqs=ctx.n_seqs,
                                       max_new=ctx.max_new, scale=self.scale,
                                       sink=self.t_sink if self.has_sink else None, gate=gate, window=window)
                linear(ctx, mixed, self.t_out_weight, None, residual, m=n, residual=None if store else residual, w_is_nk=True)
                ctx.ws.release(mark)
                return
        # the queries as the latent rows meet them: per head [W_uk^T q_plain | q_rot turned]
        q_latent = ctx.ws.take((n, heads * dk), dtype)
        q_latent_heads = q_latent.view(n, heads, dk)
        kernels.head_linear(q_heads[:, :, :self.dim], self.uk_heads, q_latent_heads[:, :, :rank], n_tokens=n)
        if rot:
            self.positions.rotate_vectors(ctx, q_heads[:, :, self.dim:], q_latent_heads[:, :, rank:])
        mixed_latent = ctx.ws.take((n, heads * rank), dtype)
        splits = self._splits(ctx, kernels.latent_attention_rows(rank, rot, dtype))
        scratch = None
        if splits > 1:
            scratch = ctx.ws.take((kernels.latent_attention_scratch_floats(n, heads, rank, splits),), torch.float32)
        kernels.latent_attention(q_latent, mixed_latent, pool, table, group.table_len, ctx.seq_start, ctx.past_len,
                                 n_tokens=n, n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=heads, rank=rank, rot=rot,
                                 scale=self.scale, sink=self.t_sink if self.has_sink else None, n_splits=splits,
                                 scratch=scratch, window=window)
        # values: W_uv on the weighted latents, times the output gate
        mixed = ctx.ws.take((n, self.mixed_width), dtype)
        kernels.head_linear(mixed_latent.view(n, heads, rank), self.uv_heads, mixed.view(n, heads, self.vdim), n_tokens=n,
                            gate=gate)
        linear(ctx, mixed, self.t_out_weight, None, residual, m=n, residual=None if store else residual, w_is_nk=True)
        ctx.ws.release(mark)
