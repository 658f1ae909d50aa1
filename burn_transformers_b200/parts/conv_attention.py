"""Windowed softmax attention behind a short convolution, whose heads talk before the softmax and whose values are
its keys."""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import PAGE_SIZE, CacheNeed, KvSpec, StateSpec
from ..errors import CacheError, ShapeError
from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .base import Mixer
from .linear import linear


class TalkingConvAttention(Mixer):
    """Grouped-head attention over the last `window` positions (all of them when `window` is None):

        u = [W_q h | W_k h]                            projections, no biases
        c_t = sum_j conv[:, j] * u_(t - taps + 1 + j)   per channel, causal, zeros before the sequence's start
        q, k = c divided by its root mean square per head (eps inside the root, no weight);  v = the key part of c
        raw_g(i, j) = cap tanh((q_g(i) . k_g(j)) scale temp_g / cap) - slope_g (i - j)
        s_h(i, j) = sum_g talk[h, g] raw_g(i, j)        the heads' scores mixed before the softmax
        o_h(i) = sum_j softmax_j(s_h(i, .)) v_h(j),  then * sigmoid(W_g h), W_o, times `out_scale`

    with slope_g = 2^(-8 (g + 1) / heads).  The convolution, the norms, the scores and the softmax run in 32-bit
    (csrc/short_conv.cu, csrc/talking_attention.cu).  The cache: pages with the normed keys as keys and the undivided
    ones as values, and the last taps - 1 projected rows of every sequence as the state "qk_taps".

    Tensors: `in.weight` [(heads + kv_heads) * dim + heads * dim, width] = rows of W_q, W_k, W_g; `conv.weight`
    [(heads + kv_heads) * dim, taps]; `temp` [heads]; `talk` [heads, heads]; `out.weight` [width, heads * dim].
    """

    accepts_lazy_norm = True
    MAX_HEADS = 32          # a warp a head in the attention kernel
    MAX_TAPS = 16

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, dim: int, taps: int, scale: float, softcap: float,
                 eps: float, *, window: int | None = None, out_scale: float = 1.0, init_std: float = 0.02,
                 out_init_std: float | None = None):
        if n_heads <= 0 or n_kv_heads <= 0 or n_heads % n_kv_heads:
            raise ShapeError(f"{n_heads} query heads cannot share {n_kv_heads} key heads")
        if n_heads > self.MAX_HEADS:
            raise ShapeError(f"talking attention: {n_heads} heads exceed the {self.MAX_HEADS} its kernel takes")
        if not 1 <= dim <= 256:
            raise ShapeError(f"talking attention: head size {dim} is outside 1..256")
        if not 1 <= taps <= self.MAX_TAPS:
            raise ShapeError(f"short convolution: {taps} taps are outside 1..{self.MAX_TAPS}")
        self.width, self.n_heads, self.n_kv_heads, self.dim, self.taps = width, n_heads, n_kv_heads, dim, taps
        self.scale, self.softcap, self.eps, self.window = float(scale), float(softcap), float(eps), window
        self.out_scale = float(out_scale)
        self.q_width, self.kv_width = n_heads * dim, n_kv_heads * dim
        self.conv_width = self.q_width + self.kv_width
        self.in_width = self.conv_width + self.q_width
        self.init_std = init_std
        self.out_init_std = init_std if out_init_std is None else out_init_std

    def specs(self):
        return {"in.weight": TensorSpec((self.in_width, self.width), MATRIX, ("normal", self.init_std)),
                "conv.weight": TensorSpec((self.conv_width, self.taps), VECTOR, ("normal", self.taps ** -0.5)),
                "temp": TensorSpec((self.n_heads,), VECTOR, ("ones",)),
                "talk": TensorSpec((self.n_heads, self.n_heads), VECTOR, ("normal", self.n_heads ** -0.5)),
                "out.weight": TensorSpec((self.width, self.q_width), MATRIX, ("normal", self.out_init_std))}

    def bind(self, tensors):
        if self.out_scale != 1.0:
            tensors = dict(tensors)
            t = tensors["out.weight"]
            tensors["out.weight"] = (t.to(torch.float32) * self.out_scale).to(t.dtype)
        super().bind(tensors)
        slopes = [2.0 ** (-8.0 * (h + 1) / self.n_heads) for h in range(self.n_heads)]
        self.slope = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(self.t_in_weight.device)
        self.t_conv_weight = self.t_conv_weight.contiguous()
        self.t_talk = self.t_talk.contiguous()
        # (a convolution of one tap keeps nothing: an empty state of the right shape)
        self.no_state = torch.empty((1, 0, self.conv_width), dtype=torch.float32, device=self.t_in_weight.device)

    def cache_need(self):
        states = (StateSpec("qk_taps", (self.taps - 1, self.conv_width), torch.float32),) if self.taps > 1 else ()
        return CacheNeed(kv=KvSpec(self.n_kv_heads, self.dim, self.window), states=states)

    def forward(self, ctx, x, residual, entry, owns_cache=True):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("talking attention has no phase in the fused step")
        if not owns_cache:
            raise ShapeError("talking attention: the convolution's state cannot be another layer's")
        mark = ctx.ws.mark()
        n, dtype = ctx.n_tokens, ctx.dtype
        proj = ctx.ws.take((n, self.in_width), dtype)
        linear(ctx, x, self.t_in_weight, None, proj, m=n, w_is_nk=True)
        # [normed q | normed k | k as it leaves the convolution]
        qkv = ctx.ws.take((n, self.conv_width + self.kv_width), dtype)
        state = ctx.cache.state(entry, "qk_taps") if self.taps > 1 else self.no_state
        kernels.short_conv(proj[:, :self.conv_width], self.t_conv_weight, None, state, ctx.slots, ctx.seq_start,
                           ctx.token_seq, qkv[:, :self.conv_width], n_tokens=n, n_seqs=ctx.n_seqs, norm_group=self.dim,
                           eps=self.eps, raw_out=qkv[:, self.conv_width:], raw_first_group=self.n_heads)
        k_pool, v_pool, group, g = ctx.cache.layer_pools(entry)
        table = ctx.tables[g]
        kernels.kv_append(qkv, self.q_width, self.conv_width, ctx.positions, ctx.token_seq, ctx.ctx_len, table,
                          group.table_len, k_pool, v_pool, n, self.n_kv_heads, self.dim)
        mixed = ctx.ws.take((n, self.q_width), dtype)
        common = dict(n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=self.n_heads, n_kv_heads=self.n_kv_heads,
                      head_dim=self.dim, scale=self.scale, window=self.window or 0, cap=self.softcap, temp=self.t_temp,
                      slope=self.slope, talk=self.t_talk, gate=proj[:, self.conv_width:])
        if dtype == torch.bfloat16:
            # few tokens a sequence: the keys of each are shared among blocks
            n_split, need = kernels.talking_attention_split(ctx.n_seqs, ctx.max_new, self.n_heads, self.dim,
                                                            self.window or 0, ctx.ctx_bound)
            if n_split > 1:
                common.update(n_split=n_split, parts=ctx.ws.take((need,), torch.float32))
        if ctx.fresh:
            # every sequence starts at position 0: keys and values are the step's own rows
            kernels.talking_attention(qkv[:, :self.q_width], mixed, ctx.seq_start, ctx.past_len,
                                      k=qkv[:, self.q_width:self.conv_width], v=qkv[:, self.conv_width:], **common)
        else:
            if group.is_ring and ctx.max_new > group.table_len * PAGE_SIZE - self.window + 1:
                raise CacheError("a step that brings this many tokens to sequences that already hold some would "
                                 "overwrite keys of a windowed layer's ring that its first tokens still see")
            kernels.talking_attention(qkv[:, :self.q_width], mixed, ctx.seq_start, ctx.past_len, k_pool=k_pool,
                                      v_pool=v_pool, table=table, table_len=group.table_len, **common)
        linear(ctx, mixed, self.t_out_weight, None, residual, m=n, residual=residual, w_is_nk=True)
        ctx.ws.release(mark)

