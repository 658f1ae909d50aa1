"""Attention whose weights are sigmoids of the scores."""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import PAGE_SIZE, CacheNeed, KvSpec
from ..errors import ShapeError
from ..weights.spec import MATRIX, VECTOR, TensorSpec
from .base import Mixer
from .linear import linear


class SigmoidAttention(Mixer):
    """Grouped-head attention without a softmax: the weight of a visible key is sigmoid(q . k * scale + bias_h), and
    the weights of a query are not normalised over its keys.

    With h the mixer's input, per position:

        [q | k | v] = W_in h + b_in          heads * dim, kv_heads * dim, kv_heads * vdim channels
        q, k        <- per head x / rms(x) * weight ([dim], one for all query heads, one for all key heads), then the
                       first `positions.dims` channels turned by the position, channel i with i + dims / 2
        v           <- per head x / rms(x) (no weight); then, with `values_from`, (1 - mix) v + mix v', v' the values
                       another layer published for the same token under that name in this step
        out[i, h]   = sum over visible j of sigmoid(q[i, h] . k[j, g] * scale + bias[h]) v[j, g],  g = h // (heads / kv_heads)
        y           = W_out out + b_out, added to the residual stream

    Position i sees j <= i with i - j < window or j < keep_first (`window` None: every j <= i).  Keys and values have
    sizes of their own, so the cache holds one row [k | v] per position and key head (`KvSpec(kv_heads, dim + vdim,
    has_values=False)`); every position is kept, since the first `keep_first` stay visible for ever and the kernel
    walks only the two runs of keys a query sees.  `values_as` publishes this layer's values (after their norm and
    mixing, 32-bit) for later layers of the step under that name (`ModelPlan.step_tensors` must list it).

    Tensors: `in.weight` [q + k + v rows, width] with `in.bias`; `q_norm.weight`, `k_norm.weight` [dim]; `bias` [heads];
    `mix` [] (only with `values_from`); `out.weight` [width, heads * vdim] with `out.bias`.
    """

    accepts_lazy_norm = False
    # Steps whose longest run of new tokens is at least this take a tensor-core kernel in bfloat16:
    # csrc/attention_prefill_tcgen05.cu for keys and values of 64 or 128 channels a head each (fresh prompts over the
    # step's own rows, portions that continue a sequence over its pages), csrc/sink_attention_mma.cu for fresh prompts
    # of other sizes; everything else (decode steps, short portions, 32-bit, other sizes) takes the multiply-add kernels
    # over the pages.
    prompt_from = 48

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float, eps: float, positions,
                 *, window: int | None = None, keep_first: int = 0, values_as: str | None = None,
                 values_from: str | None = None, init_std: float = 0.02, out_init_std: float | None = None):
        if min(width, n_heads, n_kv_heads, dim, vdim) <= 0 or n_heads % n_kv_heads:
            raise ShapeError(f"sigmoid attention: {n_heads} query heads cannot share {n_kv_heads} key heads")
        if vdim > 256:
            raise ShapeError(f"sigmoid attention: values of {vdim} channels exceed the 256 the kernel takes")
        if positions is None or not positions.rotates or positions.dims > dim:
            raise ShapeError("sigmoid attention: needs a rotating position encoding over at most dim channels")
        if window is not None and window <= 0 or keep_first < 0:
            raise ShapeError("sigmoid attention: a window is positive, the kept first positions are not negative")
        self.width, self.n_heads, self.n_kv_heads, self.dim, self.vdim = width, n_heads, n_kv_heads, dim, vdim
        self.scale, self.eps, self.positions = float(scale), float(eps), positions
        self.window, self.keep_first = window, int(keep_first)
        self.values_as, self.values_from = values_as, values_from
        self.q_width, self.k_width, self.v_width = n_heads * dim, n_kv_heads * dim, n_kv_heads * vdim
        self.proj_width = self.q_width + self.k_width + self.v_width
        self.init_std = init_std
        self.out_init_std = init_std if out_init_std is None else out_init_std

    linear_weights = ()      # (both matrices are stored [out, in] and used so)

    def specs(self):
        specs = {"in.weight": TensorSpec((self.proj_width, self.width), MATRIX, ("normal", self.init_std)),
                 "in.bias": TensorSpec((self.proj_width,), VECTOR, ("normal", 0.1)),
                 "q_norm.weight": TensorSpec((self.dim,), VECTOR, ("ones",)),
                 "k_norm.weight": TensorSpec((self.dim,), VECTOR, ("ones",)),
                 "bias": TensorSpec((self.n_heads,), VECTOR, ("normal", 1.0)),
                 "out.weight": TensorSpec((self.width, self.n_heads * self.vdim), MATRIX, ("normal", self.out_init_std)),
                 "out.bias": TensorSpec((self.width,), VECTOR, ("normal", 0.1))}
        if self.values_from is not None:
            specs["mix"] = TensorSpec((), VECTOR, ("normal", 0.3))
        return specs

    def bind(self, tensors):
        super().bind(tensors)
        self.positions.inv_freq(self.t_in_weight.device)
        if self.values_from is not None:
            self.t_mix = self.t_mix.reshape(1).contiguous()

    def cache_need(self):
        return CacheNeed(kv=KvSpec(self.n_kv_heads, self.dim + self.vdim, None, has_values=False))

    # `forward(..., store=True)` writes the result into `residual` instead of adding it (rows that hold nothing yet)
    can_store = True

    def forward(self, ctx, x, residual, entry, owns_cache=True, store=False):
        if getattr(ctx, "program", None) is not None:
            from ..engine.program import ProgramUnsupported
            raise ProgramUnsupported("sigmoid attention has no phase in the fused step")
        if not owns_cache:
            raise ShapeError("sigmoid attention: a layer files its own keys and values")
        mark = ctx.ws.mark()
        n, dtype = ctx.n_tokens, ctx.dtype
        proj = ctx.ws.take((n, self.proj_width), dtype)
        linear(ctx, x, self.t_in_weight, self.t_in_bias, proj, m=n, w_is_nk=True)
        k_pool, _, group, g = ctx.cache.layer_pools(entry)
        if group.spec.head_dim != self.dim + self.vdim or group.spec.n_kv_heads != self.n_kv_heads or group.is_ring:
            raise ShapeError("sigmoid attention: the cache entry does not hold this layer's rows")
        table = ctx.tables[g]
        shared = getattr(ctx, "shared", {})
        v_other = v_publish = None
        if self.values_from is not None:
            v_other = shared.get(self.values_from)
            if v_other is None:
                raise ShapeError(f"sigmoid attention: no layer has published `{self.values_from}` in this step")
        if self.values_as is not None:
            v_publish = shared.get(self.values_as)
            if v_publish is None:
                raise ShapeError(f"sigmoid attention: the step has no tensor `{self.values_as}` to publish into")
        kernels.sigmoid_attention_prep(proj, self.t_q_norm_weight, self.t_k_norm_weight, self.eps, ctx.positions,
                                       ctx.token_seq, self.positions.inv_freq(proj.device), self.positions.dims, table,
                                       group.table_len, k_pool, n_tokens=n, n_heads=self.n_heads,
                                       n_kv_heads=self.n_kv_heads, dim=self.dim, vdim=self.vdim,
                                       mix=self.t_mix if v_other is not None else None, v_other=v_other, v_publish=v_publish)
        mixed = ctx.ws.take((n, self.n_heads * self.vdim), dtype)
        if dtype == torch.bfloat16 and not ctx.is_decode and ctx.max_new >= self.prompt_from:
            # prompts and their portions on tensor cores: tcgen05 with the scores in tensor memory where keys and values
            # have sizes the kernel is built for (fresh prompts attend over the step's own rows, portions that continue
            # a sequence over its pages); else, for fresh prompts, `mma.sync`
            if kernels.sigmoid_attention_tcgen05_supports(self.dim, self.vdim, self.proj_width):
                paged = {} if ctx.fresh else {"pool": k_pool, "table": table, "table_len": group.table_len}
                kernels.sigmoid_attention_tcgen05(proj, mixed, ctx.seq_start, ctx.past_len, n_seqs=ctx.n_seqs,
                                                  max_new=ctx.max_new, n_heads=self.n_heads, n_kv_heads=self.n_kv_heads,
                                                  head_dim=self.dim, v_dim=self.vdim, scale=self.scale, bias=self.t_bias,
                                                  window=self.window or 0, keep_first=self.keep_first, **paged)
                linear(ctx, mixed, self.t_out_weight, self.t_out_bias, residual, m=n, residual=None if store else residual,
                       w_is_nk=True)
                ctx.ws.release(mark)
                return
            q = proj[:, :self.q_width].view(n, self.n_heads, self.dim)
            k = proj[:, self.q_width:self.q_width + self.k_width].view(n, self.n_kv_heads, self.dim)
            v = proj[:, self.q_width + self.k_width:].view(n, self.n_kv_heads, self.vdim)
            out = mixed.view(n, self.n_heads, self.vdim)
            if ctx.fresh and kernels.sigmoid_attention_prompt_supports(q, k, v, out):
                kernels.sigmoid_attention_prompt(q, k, v, out, ctx.seq_start, n_seqs=ctx.n_seqs, max_new=ctx.max_new,
                                                 scale=self.scale, bias=self.t_bias, window=self.window or 0,
                                                 keep_first=self.keep_first)
                linear(ctx, mixed, self.t_out_weight, self.t_out_bias, residual, m=n, residual=None if store else residual,
                       w_is_nk=True)
                ctx.ws.release(mark)
                return
        kernels.sigmoid_attention(proj, mixed, k_pool, table, group.table_len, ctx.seq_start, ctx.past_len,
                                  n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=self.n_heads,
                                  n_kv_heads=self.n_kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale,
                                  bias=self.t_bias, window=self.window or 0, keep_first=self.keep_first)
        linear(ctx, mixed, self.t_out_weight, self.t_out_bias, residual, m=n, residual=None if store else residual,
                       w_is_nk=True)
        ctx.ws.release(mark)
