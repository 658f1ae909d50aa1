"""Python face of the CUDA kernel library: loads it, checks arguments, launches on torch's stream.

There is no fallback: if the library cannot be built or loaded, or a tensor lies on the host,
the call raises.  Tensors are passed as raw device pointers; shapes and dtypes are checked here
so that a kernel never sees a size it was not written for.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .errors import KernelError, ShapeError

_LIB = None
DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
ACTIVATIONS = {None: 0, "none": 0, "gelu_new": 1, "gelu_tanh": 1, "gelu": 2, "gelu_erf": 2}
# rules for the (gate, up) pair of a gated feed-forward: the activations above on the gate, or the clamped rule
PAIR_RULES = dict(ACTIVATIONS, swish_clamp=3)
PAGE_SIZE = 64


def library() -> ctypes.CDLL:
    """The loaded kernel library; builds it on first use."""
    global _LIB
    if _LIB is None:
        from .csrc.build import build
        path = build()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise KernelError(f"cannot load the CUDA kernel library {path}: {error}") from None
        lib.bt_last_error.restype = ctypes.c_char_p
        lib.bt_attention_decode_scratch_floats.restype = c_longlong
        lib.bt_latent_attention_scratch_floats.restype = c_longlong
        lib.bt_lightning_chunked_scratch_floats.restype = c_longlong
        lib.bt_mlstm_chunked_scratch_floats.restype = c_longlong
        lib.bt_launch_count.restype = c_longlong
        if lib.bt_abi_version() != 1:
            raise KernelError(f"{path} has an unexpected interface version")
        _LIB = lib
    return _LIB if _PROFILE is None else _Bracketed(_LIB, _PROFILE)


class KernelProfile:
    """Times every launch of the library on the device while it is active (`with KernelProfile() as p: ...`).

    Each launch is bracketed by two CUDA events on the launching stream; `summary()` waits for them and returns, per
    kernel, the number of launches, the time, and what the wrappers said the launches had to do (floating-point
    operations and bytes that must move), from which achieved TFLOP/s and GB/s follow.  Launches recorded into a
    CUDA graph cannot be timed this way: profile steps that run their kernels directly."""

    SKIP = ("bt_last_error", "bt_launch_count", "bt_abi_version", "bt_tensor_map", "bt_decode_flow_plan",
            "bt_decode_flow_phase_bytes", "bt_attention_decode_scratch_floats", "bt_latent_attention_scratch_floats",
            "bt_latent_attention_rows", "bt_lightning_chunked_scratch_floats", "bt_sink_attention_supports",
            "bt_mlstm_chunked_scratch_floats", "bt_moe_tile_rows", "bt_mlstm_scan_fuses")

    def __init__(self, context_hint: int | None = None):
        self.records = []          # (name, start event, stop event, flops, bytes)
        self.pending = (0.0, 0.0)
        # the length of the profiled sequences, for kernels whose work depends on lengths that only the device knows
        self.context_hint = context_hint

    def __enter__(self):
        global _PROFILE
        _PROFILE = self
        return self

    def __exit__(self, *exc):
        global _PROFILE
        _PROFILE = None

    def summary(self) -> list[dict]:
        torch.cuda.synchronize()
        rows: dict[str, dict] = {}
        for name, start, stop, flops, nbytes in self.records:
            row = rows.setdefault(name, {"kernel": name, "launches": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
            row["launches"] += 1
            row["ms"] += start.elapsed_time(stop)
            row["flops"] += flops
            row["bytes"] += nbytes
        total = sum(r["ms"] for r in rows.values()) or 1.0
        out = []
        for row in sorted(rows.values(), key=lambda r: -r["ms"]):
            seconds = row["ms"] * 1e-3
            row["share"] = row["ms"] / total
            row["tflops"] = row["flops"] / seconds / 1e12 if seconds > 0 and row["flops"] else None
            row["gbs"] = row["bytes"] / seconds / 1e9 if seconds > 0 and row["bytes"] else None
            out.append(row)
        return out


class _Bracketed:
    """The library as the wrappers see it while a profile is active: every launch between two events and inside
    an NVTX range of the kernel's name."""

    def __init__(self, lib, profile):
        self._lib, self._profile = lib, profile

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if name.endswith("_supports") or name.startswith(KernelProfile.SKIP):
            return fn
        profile = self._profile

        def launch(*args):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.nvtx.range_push(name)      # (a timeline tool shows the same brackets by name)
            start.record()
            code = fn(*args)
            stop.record()
            torch.cuda.nvtx.range_pop()
            flops, nbytes = profile.pending
            profile.pending = (0.0, 0.0)
            profile.records.append((name[3:] if name.startswith("bt_") else name, start, stop, flops, nbytes))
            return code
        return launch


_PROFILE: KernelProfile | None = None


def _work(flops: float = 0.0, nbytes: float = 0.0) -> None:
    """What the next launch has to do (for a profile; costs nothing otherwise)."""
    if _PROFILE is not None:
        _PROFILE.pending = (float(flops), float(nbytes))


def _linear_work(m, n, k, a, w, out) -> None:
    if _PROFILE is not None:
        _work(2.0 * m * n * k, m * k * (a.element_size() if hasattr(a, "element_size") else 4) + n * k * w.element_size()
              + m * n * out.element_size())


def launch_count() -> int:
    """Kernel launches issued through the library so far (a launch recorded into a CUDA graph counts once)."""
    return int(library().bt_launch_count())


def _check(code: int) -> None:
    if code != 0:
        raise KernelError(library().bt_last_error().decode(errors="replace"))


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    """Device, layout, element type and extents of one argument (None in `shape` leaves an extent free)."""
    try:
        ok = t.is_cuda and t.is_contiguous()
    except AttributeError:
        raise ShapeError(f"{name}: expected a tensor, found {type(t).__name__}") from None
    if not ok:
        if not t.is_cuda:
            raise KernelError(f"{name}: lies on {t.device}; the kernels of this library run on a CUDA device only")
        raise ShapeError(f"{name}: must be contiguous")
    if dtype is not None and t.dtype is not dtype:
        if not isinstance(dtype, (tuple, list)) or t.dtype not in dtype:
            raise ShapeError(f"{name}: expected dtype {dtype}, found {t.dtype}")
    if shape is not None:
        got = t.shape
        if len(shape) != len(got):
            raise ShapeError(f"{name}: expected shape {list(shape)}, found {list(got)}")
        for want, have in zip(shape, got):
            if want is not None and want != have:
                raise ShapeError(f"{name}: expected shape {list(shape)}, found {list(got)}")


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise ShapeError(f"unsupported element type {dtype}") from None


# --------------------------------------------------------------------------------------------

def embed(tokens, positions, wte, wpe, out, status=None, scale: float = 1.0):
    """out[t] = (wte[tokens[t]] (+ wpe[positions[t]])) * scale into the 32-bit residual stream."""
    n = tokens.shape[0]
    vocab, width = wte.shape
    _need(tokens, "tokens", torch.int32, (n,))
    _need(wte, "wte", (torch.float32, torch.bfloat16))
    _need(out, "out", torch.float32, (None, width))
    n_pos = 0
    if wpe is not None:
        _need(positions, "positions", torch.int32, (n,))
        _need(wpe, "wpe", wte.dtype, (None, width))
        n_pos = wpe.shape[0]
    if out.shape[0] < n:
        raise ShapeError(f"out: {out.shape[0]} rows for {n} tokens")
    _work(0.0, n * width * (wte.element_size() * (2 if wpe is not None else 1) + 4))
    _check(library().bt_embed(_ptr(tokens), _ptr(positions if wpe is not None else None), _ptr(wte), _ptr(wpe), _ptr(out),
                              c_int(n), c_int(width), c_int(vocab), c_int(n_pos), c_float(scale),
                              c_int(_code(wte.dtype)), _ptr(status), _stream()))


def layernorm(x, gamma, beta, out, eps: float, rows=None, n_rows=None):
    """out[r] = LayerNorm(x[rows[r]] or x[r]); x is 32-bit, out is 32-bit or bfloat16."""
    width = x.shape[-1]
    _need(x, "x", torch.float32, (None, width))
    _need(gamma, "gamma", torch.float32, (width,))
    if beta is not None:
        _need(beta, "beta", torch.float32, (width,))
    n = n_rows if n_rows is not None else (rows.shape[0] if rows is not None else x.shape[0])
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _need(out, "out", (torch.float32, torch.bfloat16), (None, width))
    if out.shape[0] < n:
        raise ShapeError(f"out: {out.shape[0]} rows for {n} rows")
    _work(0.0, n * width * (4 + out.element_size()))
    _check(library().bt_layernorm(_ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out), c_int(n), c_int(width),
                                  c_float(eps), c_int(_code(out.dtype)), _stream()))


def linear_simt(a, w, bias, out, *, m=None, w_is_nk=False, activation=None, residual=None):
    """out = act(a @ w + bias) (+ residual) with 32-bit fused multiply-adds.

    a: [M, K]; w: [K, N] (or [N, K] when w_is_nk); bias: [N] float32 or None; residual: [M, N]
    float32 (may be `out` itself); out: [M, N] float32 or a's dtype.
    """
    k = a.shape[1]
    n = w.shape[0] if w_is_nk else w.shape[1]
    m = a.shape[0] if m is None else m
    _need(a, "a", (torch.float32, torch.bfloat16), (None, k))
    _need(w, "w", a.dtype, (n, k) if w_is_nk else (k, n))
    _need(out, "out", (torch.float32, a.dtype), (None, n))
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if a.shape[0] < m or out.shape[0] < m:
        raise ShapeError(f"linear: {m} rows asked of a[{a.shape[0]}] and out[{out.shape[0]}]")
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear: unknown activation {activation!r}")
    _linear_work(m, n, k, a, w, out)
    _check(library().bt_linear_simt(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), c_int(m), c_int(n), c_int(k),
                                    c_int(1 if w_is_nk else 0), c_int(ACTIVATIONS[activation]), c_int(_code(a.dtype)),
                                    c_int(_code(out.dtype)), _stream()))


def linear_skinny_supports(m, n, k, w_is_nk, fuse_ln) -> bool:
    return _supports("bt_linear_skinny_supports", m, n, k, 1 if w_is_nk else 0, 1 if fuse_ln else 0)


def linear_skinny(a, w, bias, out, *, m, w_is_nk=False, activation=None, residual=None, norm=None, split=0):
    """out[:m] = act(rows @ w + bias) (+ residual) for at most 64 bfloat16 rows.

    rows are `a` (bfloat16 [M, K]) or, when `norm` = (x32, gamma, beta, eps, row_index) is given and `a` is None,
    LayerNorm(x32[row_index]) formed inside the kernel."""
    n = w.shape[0] if w_is_nk else w.shape[1]
    k = w.shape[1] if w_is_nk else w.shape[0]
    _need(w, "w", torch.bfloat16, (n, k) if w_is_nk else (k, n))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, n))
    if out.shape[0] < m:
        raise ShapeError(f"linear_skinny: {m} rows asked of out[{out.shape[0]}]")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear_skinny: unknown activation {activation!r}")
    x32 = gamma = beta = rows = None
    eps = 0.0
    if norm is not None:
        x32, gamma, beta, eps, rows = norm
        _need(x32, "x32", torch.float32, (None, k))
        _need(gamma, "gamma", torch.float32, (k,))
        if beta is not None:
            _need(beta, "beta", torch.float32, (k,))
        if rows is not None:
            _need(rows, "rows", torch.int32)
        elif x32.shape[0] < m:
            raise ShapeError(f"linear_skinny: {m} rows asked of x32[{x32.shape[0]}]")
    else:
        _need(a, "a", torch.bfloat16, (None, k))
        if a.shape[0] < m:
            raise ShapeError(f"linear_skinny: {m} rows asked of a[{a.shape[0]}]")
    _linear_work(m, n, k, w, w, out)
    _check(library().bt_linear_skinny(_ptr(a if norm is None else None), _ptr(x32), _ptr(rows), _ptr(gamma), _ptr(beta),
                                      c_float(eps), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), c_int(m), c_int(n),
                                      c_int(k), c_int(1 if w_is_nk else 0), c_int(ACTIVATIONS[activation]),
                                      c_int(1 if out.dtype == torch.float32 else 0), c_int(split), _stream()))


def linear_mid(a, w, bias, out, *, m, activation=None, residual=None, split=0):
    """out[:m] = act(a[:m] @ w^T + bias) (+ residual) for at most 64 bfloat16 rows and weights stored [N, K]: the
    product made for 17 to 64 rows (a block per 16 columns over the whole of K, operands through a ring of
    tensor-map copies)."""
    n, k = w.shape
    _need(w, "w", torch.bfloat16, (n, k))
    _need(a, "a", torch.bfloat16, (None, k))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, n))
    if a.shape[0] < m or out.shape[0] < m:
        raise ShapeError(f"linear_mid: {m} rows asked of a[{a.shape[0]}], out[{out.shape[0]}]")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear_mid: unknown activation {activation!r}")
    _linear_work(m, n, k, a, w, out)
    _check(library().bt_linear_mid(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), _ptr(kernel_status(a.device)),
                                   c_int(m), c_int(n), c_int(k), c_int(ACTIVATIONS[activation]),
                                   c_int(1 if out.dtype == torch.float32 else 0), c_int(split), _stream()))


def linear_mid_supports(m, n, k) -> bool:
    return _supports("bt_linear_mid_supports", m, n, k)


_SUPPORTS: dict = {}


def _supports(name: str, *args) -> bool:
    """Answers of the library's pure `..._supports` questions, remembered."""
    key = (name, args)
    hit = _SUPPORTS.get(key)
    if hit is None:
        hit = bool(getattr(library(), name)(*[c_int(int(a)) for a in args]))
        _SUPPORTS[key] = hit
    return hit


def linear_tcgen05_supports(m, n, k) -> bool:
    return _supports("bt_linear_tcgen05_supports", m, n, k)


def linear_tcgen05(a, w, bias, out, *, m, activation=None, residual=None):
    """out[:m] = act(a[:m] @ w^T + bias) (+ residual) on the tcgen05 tensor cores; a [M, K] and w [N, K] bfloat16."""
    n, k = w.shape
    _need(a, "a", torch.bfloat16, (None, k))
    _need(w, "w", torch.bfloat16, (n, k))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, n))
    if a.shape[0] < m or out.shape[0] < m:
        raise ShapeError(f"linear_tcgen05: {m} rows asked of a[{a.shape[0]}] and out[{out.shape[0]}]")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear_tcgen05: unknown activation {activation!r}")
    _linear_work(m, n, k, a, w, out)
    _check(library().bt_linear_tcgen05(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                       _ptr(kernel_status(a.device)), c_int(m), c_int(n), c_int(k),
                                       c_int(ACTIVATIONS[activation]), c_int(1 if out.dtype == torch.float32 else 0),
                                       _stream()))


def linear_few_tcgen05_supports(m, n, k) -> bool:
    return _supports("bt_linear_few_tcgen05_supports", m, n, k)


def linear_few_tcgen05(a, w, bias, out, *, m, activation=None, residual=None, split=0):
    """out[:m] = act(a[:m] @ w^T + bias) (+ residual) for at most 128 bfloat16 rows and weights stored [N, K], on the
    tcgen05 tensor cores with the weights on their M side: the product for few rows over large weights (a block per
    128 columns and slice of K, the slices of a cluster summed through distributed shared memory)."""
    n, k = w.shape
    _need(a, "a", torch.bfloat16, (None, k))
    _need(w, "w", torch.bfloat16, (n, k))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, n))
    if a.shape[0] < m or out.shape[0] < m:
        raise ShapeError(f"linear_few_tcgen05: {m} rows asked of a[{a.shape[0]}] and out[{out.shape[0]}]")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear_few_tcgen05: unknown activation {activation!r}")
    _linear_work(m, n, k, a, w, out)
    _check(library().bt_linear_few_tcgen05(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                           _ptr(kernel_status(a.device)), c_int(m), c_int(n), c_int(k),
                                           c_int(ACTIVATIONS[activation]), c_int(1 if out.dtype == torch.float32 else 0),
                                           c_int(split), _stream()))


def linear_stream_supports(m, n, k, fuse_ln) -> bool:
    return _supports("bt_linear_stream_supports", m, n, k, 1 if fuse_ln else 0)


def linear_stream(a, w, bias, out, *, m, activation=None, residual=None, norm=None, warps_k=0):
    """out[:m] = act(rows @ w^T + bias) (+ residual) for at most 64 bfloat16 rows; w is [N, K].

    rows are `a` (bfloat16 [M, K]) or, when `norm` = (x32, gamma, beta, eps, row_index) is given and `a` is None,
    LayerNorm(x32[row_index]) formed inside the kernel (at most 16 rows)."""
    n, k = w.shape
    _need(w, "w", torch.bfloat16, (n, k))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, n))
    if out.shape[0] < m:
        raise ShapeError(f"linear_stream: {m} rows asked of out[{out.shape[0]}]")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n,))
    if residual is not None:
        _need(residual, "residual", torch.float32, (None, n))
    if activation not in ACTIVATIONS:
        raise ShapeError(f"linear_stream: unknown activation {activation!r}")
    x32 = gamma = beta = rows = None
    eps = 0.0
    if norm is not None:
        x32, gamma, beta, eps, rows = norm
        _need(x32, "x32", torch.float32, (None, k))
        _need(gamma, "gamma", torch.float32, (k,))
        if beta is not None:
            _need(beta, "beta", torch.float32, (k,))
        if rows is not None:
            _need(rows, "rows", torch.int32)
        elif x32.shape[0] < m:
            raise ShapeError(f"linear_stream: {m} rows asked of x32[{x32.shape[0]}]")
    else:
        _need(a, "a", torch.bfloat16, (None, k))
        if a.shape[0] < m:
            raise ShapeError(f"linear_stream: {m} rows asked of a[{a.shape[0]}]")
    _linear_work(m, n, k, w, w, out)
    _check(library().bt_linear_stream(_ptr(a if norm is None else None), _ptr(x32), _ptr(rows), _ptr(gamma), _ptr(beta),
                                      c_float(eps), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), c_int(m), c_int(n),
                                      c_int(k), c_int(ACTIVATIONS[activation]),
                                      c_int(1 if out.dtype == torch.float32 else 0), c_int(warps_k), _stream()))


def kv_append(proj, k_offset, v_offset, positions, token_seq, ctx_len, table, table_len, k_pool, v_pool,
              n_tokens, n_kv_heads, head_dim):
    """Copies the new tokens' key and value channels of `proj` rows into the layer's pages."""
    _need(proj, "proj", (torch.float32, torch.bfloat16))
    _need(k_pool, "k_pool", proj.dtype)
    _need(v_pool, "v_pool", proj.dtype)
    _need(table, "table", torch.int32)
    _work(0.0, 4.0 * n_tokens * n_kv_heads * head_dim * proj.element_size())
    _check(library().bt_kv_append(_ptr(proj), c_longlong(proj.shape[1]), c_int(k_offset), c_int(v_offset),
                                  _ptr(positions), _ptr(token_seq), _ptr(ctx_len), _ptr(table), c_int(table.shape[1]),
                                  c_int(table_len), c_int(PAGE_SIZE), _ptr(k_pool), _ptr(v_pool), c_int(n_tokens),
                                  c_int(n_kv_heads), c_int(head_dim), c_int(_code(proj.dtype)), _stream()))


def attention_prefill_simt(q_proj, out, seq_start, past_len, n_seqs, max_new, n_heads, n_kv_heads, head_dim, scale,
                           *, causal=True, window=0, k_pool=None, v_pool=None, table=None, table_len=0,
                           k_offset=None, v_offset=None):
    """Attention of several new tokens per sequence.

    Queries are the first n_heads*head_dim channels of `q_proj` rows.  Keys and values come either
    from the pages (`k_pool`, `v_pool`, `table`) or, when `table` is None, from the channels
    `k_offset`, `v_offset` of the same rows (sequences that start at position 0).
    """
    _need(q_proj, "q_proj", (torch.float32, torch.bfloat16))
    _need(out, "out", q_proj.dtype, (None, n_heads * head_dim))
    stride = q_proj.shape[1]
    es = q_proj.element_size()
    if table is None:
        k_ptr = c_void_p(q_proj.data_ptr() + k_offset * es)
        v_ptr = c_void_p(q_proj.data_ptr() + v_offset * es)
        t_ptr, t_stride = c_void_p(0), 0
    else:
        _need(k_pool, "k_pool", q_proj.dtype)
        _need(v_pool, "v_pool", q_proj.dtype)
        _need(table, "table", torch.int32)
        k_ptr, v_ptr, t_ptr, t_stride = _ptr(k_pool), _ptr(v_pool), _ptr(table), table.shape[1]
    _check(library().bt_attention_prefill_simt(
        _ptr(q_proj), c_longlong(stride), k_ptr, v_ptr, t_ptr, c_int(t_stride), c_int(table_len), c_int(PAGE_SIZE),
        c_longlong(stride), _ptr(out), _ptr(seq_start), _ptr(past_len), c_int(n_seqs), c_int(max_new), c_int(n_heads),
        c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_int(1 if causal else 0), c_int(window),
        c_int(_code(q_proj.dtype)), _stream()))


def attention_prefill(q_proj, out, seq_start, past_len, n_seqs, max_new, n_heads, n_kv_heads, head_dim, scale, *,
                      impl=None, **kw):
    """Attention of several new tokens per sequence.  bfloat16 with a head size the kernels are built for runs on
    tensor cores (tcgen05 with the scores in tensor memory), everything else with the plain 32-bit kernel.
    `impl` ("tcgen05", "simt") asks for one kernel by name.  Arguments as attention_prefill_simt."""
    bf16 = q_proj.dtype == torch.bfloat16
    if impl is None:
        if bf16 and _supports("bt_attention_prefill_tcgen05_supports", head_dim, PAGE_SIZE):
            impl = "tcgen05"
        else:
            impl = "simt"
    if impl == "tcgen05":
        return _attention_prefill_tcgen05(q_proj, out, seq_start, past_len, n_seqs, max_new, n_heads, n_kv_heads,
                                          head_dim, scale, **kw)
    return attention_prefill_simt(q_proj, out, seq_start, past_len, n_seqs, max_new, n_heads, n_kv_heads, head_dim,
                                  scale, **kw)


def _attention_prefill_tcgen05(q_proj, out, seq_start, past_len, n_seqs, max_new, n_heads, n_kv_heads, head_dim, scale,
                               *, causal=True, window=0, k_pool=None, v_pool=None, table=None, table_len=0,
                               k_offset=None, v_offset=None):
    _need(q_proj, "q_proj", torch.bfloat16)
    _need(out, "out", torch.bfloat16, (None, n_heads * head_dim))
    stride = q_proj.shape[1]
    if table is None:
        k_ptr = c_void_p(q_proj.data_ptr() + k_offset * 2)
        v_ptr = c_void_p(q_proj.data_ptr() + v_offset * 2)
        t_ptr, t_stride, pages = c_void_p(0), 0, 0
    else:
        _need(k_pool, "k_pool", torch.bfloat16)
        _need(v_pool, "v_pool", torch.bfloat16)
        _need(table, "table", torch.int32)
        k_ptr, v_ptr, t_ptr, t_stride, pages = _ptr(k_pool), _ptr(v_pool), _ptr(table), table.shape[1], k_pool.shape[0]
    _check(library().bt_attention_prefill_tcgen05(
        _ptr(q_proj), c_longlong(q_proj.shape[0]), c_longlong(stride), k_ptr, v_ptr, c_longlong(pages), t_ptr,
        c_int(t_stride), c_int(table_len), c_int(PAGE_SIZE), _ptr(out), _ptr(kernel_status(q_proj.device)),
        _ptr(seq_start), _ptr(past_len), c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n_kv_heads),
        c_int(head_dim), c_float(scale), c_int(1 if causal else 0), c_int(window), _stream()))


def attention_decode_supports(head_dim: int, row_stride: int, dtype) -> bool:
    """Whether the decode-attention kernels take this head size: they move rows as 16-byte pieces, so a head and a
    projection row must be whole pieces (8 bfloat16 or, as the kernel is built, 8 floats), at most 256 wide."""
    return head_dim % 8 == 0 and row_stride % 8 == 0 and 0 < head_dim <= 256


def attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits) -> int:
    return int(library().bt_attention_decode_scratch_floats(c_int(n_seqs), c_int(n_heads), c_int(head_dim), c_int(n_splits)))


_TICKETS: dict = {}


def _tickets(device, count: int) -> torch.Tensor:
    """Zeroed counters for the decode attention's merge; the kernel leaves them zero, so they are made once."""
    t = _TICKETS.get(device)
    if t is None or t.numel() < count:
        t = torch.zeros(max(count, 1 << 14), dtype=torch.int32, device=device)
        _TICKETS[device] = t
    return t


_STATUS: dict = {}


def kernel_status(device) -> torch.Tensor:
    """One int per device that a kernel sets when a bounded wait of its own ran out (see attention_decode)."""
    t = _STATUS.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[device] = t
    return t


_STATUS_TEXT = {1: "decode attention gave up waiting for a copy of cache pages",
                2: "the tcgen05 matrix product gave up waiting for a stage of its pipeline",
                3: "the fused decode step gave up at a grid barrier or waiting for cache pages",
                4: "the fused decode step met a token id or position outside its table",
                5: "the matrix product for 17 to 64 rows gave up waiting for a stage of its pipeline",
                6: "the tcgen05 prefill attention gave up waiting for a stage of its pipeline (or found its shared memory "
                   "misaligned)",
                7: "the tcgen05 matrix product for few rows gave up waiting for a stage of its pipeline"}


def check_status(device) -> None:
    """Raises if a kernel on `device` reported that one of its bounded waits ran out (its results are then not to be
    trusted), and clears the report.  Reads one int from the device: call it where the host waits anyway."""
    t = _STATUS.get(device)
    if t is None:
        return
    code = int(t.item())
    if code:
        t.zero_()
        raise KernelError(_STATUS_TEXT.get(code, f"a kernel reported status {code}"))


def attention_decode(q_proj, out, k_pool, v_pool, table, table_len, ctx_len, n_seqs, n_heads, n_kv_heads, head_dim,
                     scale, *, max_ctx, window=0, n_splits=1, scratch=None, new_kv_offsets=None, merge_in_scratch=False,
                     tensor_cores=True):
    """Attention of one new token per sequence over that sequence's pages.

    bfloat16 with a head size of 16..128 in steps of 16 runs on tensor cores (`tensor_cores=False` keeps it on
    the 32-bit multiply-add kernel that every other case takes).

    `max_ctx`: no sequence of the call is longer than this.  `new_kv_offsets` = (k_offset, v_offset): the new
    token's key and value are channels of the same `q_proj` rows; the kernel reads them from there and files
    them in the pages itself.  None: the pages already hold them.  Up to 8 splits merge inside a thread-block
    cluster; more (or `merge_in_scratch`) need `scratch`."""
    _need(q_proj, "q_proj", (torch.float32, torch.bfloat16))
    _need(out, "out", q_proj.dtype, (None, n_heads * head_dim))
    _need(k_pool, "k_pool", q_proj.dtype)
    _need(v_pool, "v_pool", q_proj.dtype)
    _need(table, "table", torch.int32)
    tickets = None
    use_mma = (tensor_cores and q_proj.dtype == torch.bfloat16
               and bool(library().bt_attention_decode_mma_supports(c_int(head_dim))))
    if n_splits > 1 and (n_splits > 8 or merge_in_scratch):
        need = attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise ShapeError(f"attention_decode: {n_splits} splits need {need} floats of scratch")
        tickets = _tickets(q_proj.device, n_seqs * n_heads)
    es = q_proj.element_size()
    new_k = new_v = c_void_p(0)
    if new_kv_offsets is not None:
        new_k = c_void_p(q_proj.data_ptr() + new_kv_offsets[0] * es)
        new_v = c_void_p(q_proj.data_ptr() + new_kv_offsets[1] * es)
    if use_mma:
        _check(library().bt_attention_decode_mma(
            _ptr(q_proj), c_longlong(q_proj.shape[1]), new_k, new_v, _ptr(k_pool), _ptr(v_pool),
            c_longlong(k_pool.numel() // (n_kv_heads * PAGE_SIZE * head_dim)), _ptr(table), c_int(table.shape[1]),
            c_int(table_len), _ptr(out), _ptr(scratch), _ptr(tickets), _ptr(kernel_status(q_proj.device)), _ptr(ctx_len),
            c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_int(window),
            c_int(n_splits), c_int(max_ctx), c_int(1 if merge_in_scratch else 0), _stream()))
        return
    _check(library().bt_attention_decode(
        _ptr(q_proj), c_longlong(q_proj.shape[1]), new_k, new_v, _ptr(k_pool), _ptr(v_pool), _ptr(table),
        c_int(table.shape[1]), c_int(table_len), c_int(PAGE_SIZE), _ptr(out), _ptr(scratch), _ptr(tickets),
        _ptr(kernel_status(q_proj.device)), _ptr(ctx_len), c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads),
        c_int(head_dim), c_float(scale), c_int(window), c_int(n_splits), c_int(max_ctx),
        c_int(1 if merge_in_scratch else 0), c_int(_code(q_proj.dtype)), _stream()))


def sample(logits, n_rows, *, do_sample, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, uniforms=None,
           stream_seeds=None, counters=None, out_ids=None, out_logp=None):
    """Selects one token per row of 32-bit logits; writes ids (int32) and log-probabilities (float32).

    Sampling takes one uniform per row from `uniforms`, or draws it on the device as draw `counters[r]` of the
    SplitMix64 stream `stream_seeds[r]` (int64 tensor holding the unsigned seeds' bits)."""
    _need(logits, "logits", torch.float32)
    vocab = logits.shape[1]
    _need(out_ids, "out_ids", torch.int32)
    _need(out_logp, "out_logp", torch.float32)
    if do_sample and stream_seeds is not None:
        _need(stream_seeds, "stream_seeds", torch.int64)
        _need(counters, "counters", torch.int32)
    elif do_sample:
        _need(uniforms, "uniforms", torch.float32)
    _check(library().bt_sample(_ptr(logits), c_longlong(logits.stride(0)), c_int(n_rows), c_int(vocab),
                               c_int(1 if do_sample else 0), c_float(temperature), c_int(top_k or 0),
                               c_float(1.0 if top_p is None else top_p), c_float(0.0 if min_p is None else min_p),
                               _ptr(uniforms), _ptr(stream_seeds), _ptr(counters), _ptr(out_ids), _ptr(out_logp),
                               _stream()))


def advance(ids, tokens, positions, past_len, ctx_len, counters, n):
    """tokens <- ids; positions, past_len, ctx_len and counters += 1 (all int32 device tensors of n entries)."""
    for name, t in (("ids", ids), ("tokens", tokens), ("positions", positions), ("past_len", past_len),
                    ("ctx_len", ctx_len), ("counters", counters)):
        _need(t, name, torch.int32)
    _check(library().bt_advance(_ptr(ids), _ptr(tokens), _ptr(positions), _ptr(past_len), _ptr(ctx_len), _ptr(counters),
                                c_int(n), _stream()))


def logit_edits(logits, rows, tokens, vals, n_edits):
    """Applies sparse edits (row, token, [add, repetition, subtract, ban]) to 32-bit logits in place."""
    _need(logits, "logits", torch.float32)
    _check(library().bt_logit_edits(_ptr(logits), c_longlong(logits.stride(0)), _ptr(rows), _ptr(tokens), _ptr(vals),
                                    c_int(n_edits), c_int(logits.shape[1]), _stream()))


# ---- attention over a latent cache, the decayed linear recurrence, row-wise kernels ---------------------------

def latent_append(src, norm_weight, eps, positions, token_seq, inv_freq, rot_dims, table, table_len, pool, n_tokens,
                  rank, rot):
    """Files the new tokens' latent rows: `src` [tokens, rank + rot] (a view whose rows may lie `stride(0)` apart, the
    channels contiguous) is RMS-normed over its first `rank` channels (times `norm_weight`), its last `rot` channels are
    turned pairwise by the token's position (the first `rot_dims` of them), and both go to `pool`
    [pages, PAGE_SIZE, rank + rot]."""
    if src.dim() != 2 or src.shape[1] != rank + rot or src.stride(1) != 1 or not src.is_cuda:
        raise ShapeError(f"latent_append: src must be a device view [tokens, {rank + rot}] with contiguous channels")
    _need(pool, "pool", src.dtype, (None, PAGE_SIZE, rank + rot))
    _need(norm_weight, "norm_weight", torch.float32, (rank,))
    _need(inv_freq, "inv_freq", torch.float32)
    if inv_freq.numel() < rot_dims // 2:
        raise ShapeError(f"latent_append: {inv_freq.numel()} frequencies for {rot_dims} rotated channels")
    _need(table, "table", torch.int32)
    _work(0.0, 2.0 * n_tokens * (rank + rot) * src.element_size())
    _check(library().bt_latent_append(_ptr(src), c_longlong(src.stride(0)), _ptr(norm_weight), c_float(eps),
                                      _ptr(positions), _ptr(token_seq), _ptr(inv_freq), c_int(rot_dims), _ptr(table),
                                      c_int(table.shape[1]), c_int(table_len), c_int(PAGE_SIZE), _ptr(pool),
                                      c_int(n_tokens), c_int(rank), c_int(rot), c_int(_code(src.dtype)), _stream()))


def _head_view(t, name, n_heads, width):
    """(row stride, head stride) of a view [tokens, heads, width] whose channels are contiguous."""
    if t.dim() != 3 or t.shape[1] != n_heads or t.shape[2] != width or t.stride(2) != 1 or not t.is_cuda:
        raise ShapeError(f"{name}: expected a device view [tokens, {n_heads}, {width}] with contiguous channels, found "
                         f"{list(t.shape)} with strides {list(t.stride())}")
    return t.stride(0), t.stride(1)


def head_linear(a, w, out, *, n_tokens, gate=None, tensor_cores=True):
    """out[t, h, :] = a[t, h, :] @ w[h]  (times sigmoid(gate[t, h, :]) if `gate`), sums in 32-bit.

    a: view [tokens, heads, K]; w: [heads, K, N] contiguous; out and gate: views [tokens, heads, N].  bfloat16 operands
    that lie on 16-byte boundaries with K and N multiples of 8 run on tensor cores (`tensor_cores=False`: never)."""
    n_heads, k, n = w.shape
    _need(w, "w", (torch.float32, torch.bfloat16), (n_heads, k, n))
    a_rs, a_hs = _head_view(a, "a", n_heads, k)
    o_rs, o_hs = _head_view(out, "out", n_heads, n)
    g_rs = g_hs = 0
    if gate is not None:
        g_rs, g_hs = _head_view(gate, "gate", n_heads, n)
    for name, t in (("a", a), ("out", out)) + ((("gate", gate),) if gate is not None else ()):
        if t.dtype is not w.dtype:
            raise ShapeError(f"head_linear: {name} is {t.dtype}, the weights are {w.dtype}")
        if t.shape[0] < n_tokens:
            raise ShapeError(f"head_linear: {n_tokens} tokens asked of {name}[{t.shape[0]}]")
    _work(2.0 * n_tokens * n_heads * k * n, (n_tokens * n_heads * (k + n) + n_heads * k * n) * w.element_size())
    _check(library().bt_head_linear(_ptr(a), c_longlong(a_rs), c_int(a_hs), _ptr(w), _ptr(out), c_longlong(o_rs),
                                    c_int(o_hs), _ptr(gate), c_longlong(g_rs), c_int(g_hs), c_int(n_tokens),
                                    c_int(n_heads), c_int(k), c_int(n), c_int(1 if tensor_cores else 0),
                                    c_int(_code(w.dtype)), _stream()))


def latent_attention_scratch_floats(n_tokens, n_heads, rank, n_splits) -> int:
    return int(library().bt_latent_attention_scratch_floats(c_int(n_tokens), c_int(n_heads), c_int(rank), c_int(n_splits)))


def latent_attention_rows(rank, rot, dtype, tensor_cores=True) -> int:
    """Rows, (token, head) pairs, one block of the attention kernel holds for this shape."""
    return \
        int(library().bt_latent_attention_rows(c_int(rank), c_int(rot), c_int(_code(dtype)), c_int(1 if tensor_cores else 0)))


def latent_attention(q, out, pool, table, table_len, seq_start, past_len, *, n_tokens, n_seqs, max_new, n_heads, rank,
                     rot, scale, sink=None, n_splits=1, scratch=None, tensor_cores=True, merge=True, window=0):
    """Causal attention of the step's tokens over their sequences' latent pages.

    q: [tokens, heads * (rank + rot)] (per head: the query carried into the latent space, then its rotated part);
    pool: [pages, PAGE_SIZE, rank + rot]; out: [tokens, heads * rank] = softmax-weighted sums of the latent rows.
    `sink` [heads] (32-bit) adds exp(sink_h) to head h's denominator.  With `n_splits` > 1 the keys of a row tile are
    cut into that many runs whose partial results meet in `scratch` (32-bit, latent_attention_scratch_floats).
    bfloat16 runs on tensor cores where the shape allows it (rank + rot a multiple of 8, rank a multiple of 8, 16 or 32
    up to 128, 256, 512); `tensor_cores=False` keeps it on the 32-bit multiply-add kernel that every other case takes.
    `merge=False` (with splits) leaves the partial results in `scratch` for latent_decode_finish to join.  `window` > 0:
    a token sees the last `window` positions up to its own (the splits cut the tiles from its first visible key on)."""
    dk = rank + rot
    _need(q, "q", (torch.float32, torch.bfloat16), (None, n_heads * dk))
    _need(out, "out", q.dtype, (None, n_heads * rank))
    _need(pool, "pool", q.dtype, (None, PAGE_SIZE, dk))
    _need(table, "table", torch.int32)
    if sink is not None:
        _need(sink, "sink", torch.float32, (n_heads,))
    if q.shape[0] < n_tokens or out.shape[0] < n_tokens:
        raise ShapeError(f"latent_attention: {n_tokens} tokens asked of q[{q.shape[0]}] and out[{out.shape[0]}]")
    if n_splits > 1:
        need = latent_attention_scratch_floats(n_tokens, n_heads, rank, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise ShapeError(f"latent_attention: {n_splits} splits need {need} floats of scratch")
    if _PROFILE is not None:
        # (a rough count for a profile: every row sees half of `ctx` keys in a prompt, all of them in a decode step; the
        # cache rows of a sequence move once per row tile)
        ctx = float(_PROFILE.context_hint or 0)
        seen = ctx if max_new == 1 else ctx / 2
        _work(2.0 * n_tokens * n_heads * seen * (dk + rank), n_seqs * ctx * dk * q.element_size()
              + n_tokens * n_heads * (dk + rank) * q.element_size())
    _check(library().bt_latent_attention(
        _ptr(q), c_longlong(q.shape[1]), _ptr(pool), _ptr(table), c_int(table.shape[1]), c_int(table_len),
        c_int(PAGE_SIZE), _ptr(seq_start), _ptr(past_len), _ptr(sink), _ptr(out), c_longlong(out.shape[1]),
        _ptr(scratch if n_splits > 1 else None), c_int(n_tokens), c_int(n_seqs), c_int(max_new), c_int(n_heads),
        c_int(rank), c_int(rot), c_float(scale), c_int(n_splits), c_int(window), c_int(1 if tensor_cores else 0),
        c_int(1 if merge else 0), c_int(_code(q.dtype)), _stream()))


LIGHTNING_CHUNK = 64      # runs of more new tokens than this take the chunked form of the recurrence


def lightning_chunked_scratch_floats(n_seqs, max_new, n_heads, dim, vdim) -> int:
    return int(library().bt_lightning_chunked_scratch_floats(c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(dim),
                                                             c_int(vdim)))


def lightning_scan(proj, q_off, k_off, v_off, state, slots, seq_start, decay, out, *, n_seqs, n_heads, dim, vdim,
                   max_new=None, scratch=None, activation="swish"):
    """Runs S <- decay_h S + k v^T, o = S^T q over the step's tokens of every sequence, with q, k, v = x * sigmoid(x) of
    the channels at `q_off`, `k_off`, `v_off` of the rows of `proj` (`activation` None: the channels as they are).  state: [slots, heads, dim, vdim] 32-bit, read and
    written at the rows `slots[seq]`; out: [tokens, heads * vdim] 32-bit.

    With `max_new` (no sequence brings more tokens) above LIGHTNING_CHUNK and `scratch` (32-bit,
    lightning_chunked_scratch_floats) the chunks of a long run are worked side by side; else token by token."""
    _need(proj, "proj", (torch.float32, torch.bfloat16))
    _need(state, "state", torch.float32, (None, n_heads, dim, vdim))
    _need(decay, "decay", torch.float32, (n_heads,))
    _need(out, "out", torch.float32, (None, n_heads * vdim))
    if max(q_off, k_off) + n_heads * dim > proj.shape[1] or v_off + n_heads * vdim > proj.shape[1]:
        raise ShapeError("lightning_scan: the channel offsets leave the rows of proj")
    if activation not in ("swish", None):
        raise ShapeError(f"lightning_scan: unknown activation {activation!r}")
    act = c_int(0 if activation == "swish" else 1)
    n_rows = out.shape[0]
    _work(4.0 * n_rows * n_heads * dim * vdim, n_rows * n_heads * ((2 * dim + vdim) * proj.element_size() + 4 * vdim)
          + 8.0 * n_seqs * n_heads * dim * vdim)
    if max_new is not None and max_new > LIGHTNING_CHUNK and scratch is not None:
        need = lightning_chunked_scratch_floats(n_seqs, max_new, n_heads, dim, vdim)
        if scratch.dtype != torch.float32 or scratch.numel() < need or not scratch.is_cuda:
            raise ShapeError(f"lightning_scan: runs of {max_new} tokens need {need} floats of scratch")
        _check(library().bt_lightning_chunked(_ptr(proj), c_longlong(proj.shape[1]), c_int(q_off), c_int(k_off),
                                              c_int(v_off), _ptr(state), _ptr(slots), _ptr(seq_start), _ptr(decay),
                                              _ptr(out), c_longlong(out.shape[1]), _ptr(scratch), c_int(max_new),
                                              c_int(n_seqs), c_int(n_heads), c_int(dim), c_int(vdim), act,
                                              c_int(_code(proj.dtype)), _stream()))
        return
    _check(library().bt_lightning_scan(_ptr(proj), c_longlong(proj.shape[1]), c_int(q_off), c_int(k_off), c_int(v_off),
                                       _ptr(state), _ptr(slots), _ptr(seq_start), _ptr(decay), _ptr(out),
                                       c_longlong(out.shape[1]), c_int(n_seqs), c_int(n_heads), c_int(dim), c_int(vdim),
                                       act, c_int(_code(proj.dtype)), _stream()))


GATE_RULES = {"sigmoid": 0, "swish": 1}


def rmsnorm(x, weight, out, eps: float, *, n_rows, gate=None, groups: int = 1, gate_rule: str = "sigmoid"):
    """out[r] = x[r] / sqrt(mean(x[r]^2) + eps) * weight  (* sigmoid(gate[r]) if `gate`), in 32-bit.  x, gate and out are
    2-D views with contiguous channels (rows may lie further apart); 32-bit or bfloat16 each.  With `groups` > 1 a row
    is that many equal runs of channels (heads side by side), each divided by its own root mean square.  `gate_rule`
    "swish" multiplies by gate * sigmoid(gate) instead."""
    if gate_rule not in GATE_RULES:
        raise ShapeError(f"rmsnorm: unknown gate rule {gate_rule!r}")
    width = weight.shape[0]
    if groups <= 0 or width % groups:
        raise ShapeError(f"rmsnorm: {width} channels are no {groups} equal groups")
    _need(weight, "weight", torch.float32, (width,))
    for name, t in (("x", x), ("out", out)) + ((("gate", gate),) if gate is not None else ()):
        if t.dim() != 2 or t.shape[1] != width or t.stride(1) != 1 or not t.is_cuda or t.shape[0] < n_rows:
            raise ShapeError(f"rmsnorm: {name} must be a device view [>= {n_rows}, {width}] with contiguous channels")
    _work(0.0, n_rows * width * (x.element_size() + out.element_size()))
    _check(library().bt_rmsnorm(_ptr(x), c_int(_code(x.dtype)), c_longlong(x.stride(0)), _ptr(weight), _ptr(gate),
                                c_int(_code(gate.dtype)) if gate is not None else c_int(0),
                                c_longlong(gate.stride(0) if gate is not None else 0), _ptr(out), c_int(_code(out.dtype)),
                                c_longlong(out.stride(0)), c_int(n_rows), c_int(width), c_int(groups), c_float(eps),
                                c_int(GATE_RULES[gate_rule]), _stream()))


def rotary_interleaved(src, dst, positions, inv_freq, *, n_tokens, dims):
    """dst[t, v] = src[t, v] with the channel pairs (2i, 2i+1), i < dims/2, turned by positions[t] * inv_freq[i]
    (angles, sines and cosines in 32-bit); channels from `dims` on are copied.  src, dst: views
    [tokens, vectors, len] with contiguous channels; they may be the same memory."""
    n_vecs, length = src.shape[1], src.shape[2]
    s_rs, s_vs = _head_view(src, "src", n_vecs, length)
    d_rs, d_vs = _head_view(dst, "dst", n_vecs, length)
    if src.dtype is not dst.dtype:
        raise ShapeError(f"rotary_interleaved: src is {src.dtype}, dst {dst.dtype}")
    _need(inv_freq, "inv_freq", torch.float32)
    if inv_freq.numel() < dims // 2:
        raise ShapeError(f"rotary_interleaved: {inv_freq.numel()} frequencies for {dims} rotated channels")
    _check(library().bt_rotary_interleaved(_ptr(src), c_longlong(s_rs), c_int(s_vs), _ptr(dst), c_longlong(d_rs),
                                           c_int(d_vs), _ptr(positions), _ptr(inv_freq), c_int(n_tokens), c_int(n_vecs),
                                           c_int(length), c_int(dims), c_int(_code(src.dtype)), _stream()))


def gated_activation(x, out, *, n_rows, activation, limit: float = 0.0):
    """out[r, j] = act(x[r, j]) * x[r, inner + j] for x [rows, 2 * inner], in 32-bit, rounded once.  `swish_clamp`:
    g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit), u' = u clamped to [-limit, limit]."""
    inner = out.shape[1]
    _need(x, "x", (torch.float32, torch.bfloat16), (None, 2 * inner))
    _need(out, "out", x.dtype, (None, inner))
    if activation not in PAIR_RULES:
        raise ShapeError(f"gated_activation: unknown activation {activation!r}")
    if x.shape[0] < n_rows or out.shape[0] < n_rows:
        raise ShapeError(f"gated_activation: {n_rows} rows asked of x[{x.shape[0]}] and out[{out.shape[0]}]")
    _work(0.0, 3.0 * n_rows * inner * x.element_size())
    _check(library().bt_gated_activation(_ptr(x), _ptr(out), c_longlong(n_rows), c_int(inner),
                                         c_int(PAIR_RULES[activation]), c_float(limit), c_int(_code(x.dtype)), _stream()))


def add_vector(x, vec, *, n_rows):
    """x[r] += vec for the first `n_rows` rows of a contiguous 32-bit [rows, width] tensor; vec: 32-bit [width]."""
    _need(x, "x", torch.float32, (None, vec.shape[0]))
    _need(vec, "vec", torch.float32)
    if x.shape[0] < n_rows:
        raise ShapeError(f"add_vector: {n_rows} rows asked of x[{x.shape[0]}]")
    _check(library().bt_add_vector(_ptr(x), _ptr(vec), c_longlong(n_rows), c_int(vec.shape[0]), _stream()))


def add_rows(x, addends, *, n_rows):
    """x[:n_rows] += addends[0] (+ addends[1]) (+ addends[2]), in this order; contiguous 32-bit [rows, width] tensors."""
    if not 1 <= len(addends) <= 3:
        raise ShapeError(f"add_rows: one to three addends, not {len(addends)}")
    _need(x, "x", torch.float32)
    for t in addends:
        _need(t, "addend", torch.float32, (None, x.shape[1]))
        if t.shape[0] < n_rows:
            raise ShapeError(f"add_rows: {n_rows} rows asked of an addend of {t.shape[0]}")
    if x.shape[0] < n_rows:
        raise ShapeError(f"add_rows: {n_rows} rows asked of x[{x.shape[0]}]")
    a, b, c = (list(addends) + [None, None])[:3]
    _check(library().bt_add_rows(_ptr(x), _ptr(a), _ptr(b), _ptr(c), c_longlong(n_rows * x.shape[1]), _stream()))


MLSTM_CHUNK = 64      # runs of more new tokens than this take the chunked form of the matrix memory's recurrence


def mlstm_chunked_scratch_floats(n_rows, n_seqs, max_new, n_heads, dim, vdim) -> int:
    return int(library().bt_mlstm_chunked_scratch_floats(c_longlong(n_rows), c_int(n_seqs), c_int(max_new), c_int(n_heads),
                                                         c_int(dim), c_int(vdim)))


def mlstm_scan(proj, offsets, i_bias, f_bias, cap: float, q_scale: float, s, n, m, slots, seq_start, out, *, n_seqs,
               n_heads, dim, vdim, max_new=None, scratch=None, norm=None) -> bool:
    """The matrix memory's recurrence over the step's tokens of every sequence (csrc/mlstm.cu).  `offsets` = channels
    of q, k, v (heads side by side) and of the input and forget gates (one channel a head) in the rows of `proj`.
    s [slots, heads, dim, vdim], n [slots, heads, dim], m [slots, heads]: 32-bit state, read and written at
    `slots[seq]`.  out [tokens, heads * vdim] 32-bit: S^T q / (max(|n . q|, exp(-m)) + 1e-6).

    With `max_new` (no sequence brings more tokens) above MLSTM_CHUNK and `scratch` (32-bit,
    mlstm_chunked_scratch_floats for out's rows) the chunks of a long run are worked side by side; else token by token.

    `norm` = (weight [heads * vdim] 32-bit, eps, channel of the output gate in proj's rows, mixed [tokens, heads * vdim]
    of proj's type): where the token-by-token kernel can hold a whole head in one block (mlstm_scan_fuses) it leaves
    out / rms(out per head) * weight * sigmoid(gate) in `mixed`, writes no `out`, and the call returns True; otherwise
    `out` is written and the caller norms."""
    q_off, k_off, v_off, i_off, f_off = (int(o) for o in offsets)
    _need(proj, "proj", (torch.float32, torch.bfloat16))
    _need(s, "s", torch.float32, (None, n_heads, dim, vdim))
    _need(n, "n", torch.float32, (s.shape[0], n_heads, dim))
    _need(m, "m", torch.float32, (s.shape[0], n_heads))
    _need(i_bias, "i_bias", torch.float32, (n_heads,))
    _need(f_bias, "f_bias", torch.float32, (n_heads,))
    _need(out, "out", torch.float32, (None, n_heads * vdim))
    width = proj.shape[1]
    if (max(q_off, k_off) + n_heads * dim > width or v_off + n_heads * vdim > width or max(i_off, f_off) + n_heads > width
            or min(q_off, k_off, v_off, i_off, f_off) < 0):
        raise ShapeError("mlstm_scan: the channel offsets leave the rows of proj")
    n_rows = out.shape[0]
    _work(4.0 * n_rows * n_heads * dim * vdim, n_rows * n_heads * ((2 * dim + vdim) * proj.element_size() + 4 * vdim)
          + 8.0 * n_seqs * n_heads * dim * vdim)
    if max_new is not None and max_new > MLSTM_CHUNK and scratch is not None:
        need = mlstm_chunked_scratch_floats(n_rows, n_seqs, max_new, n_heads, dim, vdim)
        if scratch.dtype != torch.float32 or scratch.numel() < need or not scratch.is_cuda:
            raise ShapeError(f"mlstm_scan: runs of {max_new} tokens need {need} floats of scratch")
        _check(library().bt_mlstm_chunked(_ptr(proj), c_longlong(width), c_int(q_off), c_int(k_off), c_int(v_off),
                                          c_int(i_off), c_int(f_off), _ptr(i_bias), _ptr(f_bias), c_float(cap),
                                          c_float(q_scale), _ptr(s), _ptr(n), _ptr(m), _ptr(slots), _ptr(seq_start),
                                          _ptr(out), c_longlong(out.shape[1]), _ptr(scratch), c_longlong(n_rows),
                                          c_int(max_new), c_int(n_seqs), c_int(n_heads), c_int(dim), c_int(vdim),
                                          c_int(_code(proj.dtype)), _stream()))
        return False
    fuse = norm is not None and mlstm_scan_fuses(dim, vdim)
    weight, eps, g_off, mixed = norm if fuse else (None, 0.0, 0, None)
    if fuse:
        _need(weight, "norm weight", torch.float32, (n_heads * vdim,))
        _need(mixed, "mixed", proj.dtype, (None, n_heads * vdim))
        if mixed.shape[0] < n_rows or g_off < 0 or g_off + n_heads * vdim > width:
            raise ShapeError("mlstm_scan: the gate's channels leave the rows of proj, or mixed is too short")
    _check(library().bt_mlstm_scan(_ptr(proj), c_longlong(width), c_int(q_off), c_int(k_off), c_int(v_off), c_int(i_off),
                                   c_int(f_off), _ptr(i_bias), _ptr(f_bias), c_float(cap), c_float(q_scale), _ptr(s),
                                   _ptr(n), _ptr(m), _ptr(slots), _ptr(seq_start), _ptr(out), c_longlong(out.shape[1]),
                                   _ptr(weight), c_float(eps), c_int(g_off), _ptr(mixed),
                                   c_longlong(mixed.shape[1] if fuse else 0), c_int(n_seqs), c_int(n_heads), c_int(dim),
                                   c_int(vdim), c_int(_code(proj.dtype)), _stream()))
    return fuse


def mlstm_scan_fuses(dim: int, vdim: int) -> bool:
    """Whether the token-by-token kernel holds a whole head of this size in one block (and can norm and gate it)."""
    return bool(library().bt_mlstm_scan_fuses(c_int(dim), c_int(vdim)))


def moe_route(x, router, ids, weights, *, n_tokens, top, n_groups=1, keep=1, scale=1.0, rule="sigmoid", choice_bias=None,
              normalise=True):
    """Per token the `top` experts with the largest sigmoid(router x) among the experts of the `keep` best of `n_groups`
    groups of neighbours (a group's score: the sum of its two largest), and their weights score / (sum + 1e-20) * scale.
    x [tokens, K] and router [experts, K] in the compute type, the products summed in 32-bit; ids int32 and weights
    32-bit, [tokens, top].  `rule` "softmax": the scores are softmax(router x) over all experts.  `choice_bias` [experts]
    (32-bit) is added to the scores for the choice only; without `normalise` a weight is the chosen score as it is."""
    e, k = router.shape
    if rule not in ("sigmoid", "softmax"):
        raise ShapeError(f"moe_route: unknown rule {rule!r}")
    if choice_bias is not None:
        _need(choice_bias, "choice_bias", torch.float32, (e,))
    _need(x, "x", (torch.float32, torch.bfloat16), (None, k))
    _need(router, "router", x.dtype)
    _need(ids, "ids", torch.int32, (None, top))
    _need(weights, "weights", torch.float32, (None, top))
    if min(x.shape[0], ids.shape[0], weights.shape[0]) < n_tokens:
        raise ShapeError(f"moe_route: {n_tokens} tokens asked of shorter tensors")
    _work(2.0 * n_tokens * e * k, n_tokens * k * x.element_size())
    _check(library().bt_moe_route(_ptr(x), c_longlong(x.stride(0)), _ptr(router), c_int(n_tokens), c_int(k), c_int(e),
                                  c_int(top), c_int(n_groups), c_int(keep), c_float(scale),
                                  c_int(1 if rule == "softmax" else 0), _ptr(choice_bias), c_int(1 if normalise else 0),
                                  _ptr(ids), _ptr(weights), c_int(_code(x.dtype)), _stream()))


def moe_sort(ids, offsets, tile_first, order, place, *, pairs, n_experts):
    """Sorts the (token, choice) pairs by expert: offsets [experts + 1] first row of each expert, tile_first
    [experts + 1] first row tile, order [pairs] the pair in each sorted row, place [pairs] the row of each pair."""
    for name, t, count in (("ids", ids, pairs), ("offsets", offsets, n_experts + 1), ("tile_first", tile_first, n_experts + 1),
                           ("order", order, pairs), ("place", place, pairs)):
        _need(t, name, torch.int32)
        if t.numel() < count:
            raise ShapeError(f"moe_sort: {name} holds {t.numel()} integers, {count} are needed")
    _check(library().bt_moe_sort(_ptr(ids), c_int(pairs), c_int(n_experts), _ptr(offsets), _ptr(tile_first), _ptr(order),
                                 _ptr(place), _stream()))


def moe_expert(first: bool, a, w, out, offsets, tile_first, order, pair_weight, *, pairs, top, activation=None,
               limit: float = 0.0, tensor_cores: bool = True, gated: bool = True):
    """One of the experts' two products over the sorted rows (csrc/moe.cu).  first: a [tokens, K] (gathered by the
    pair's token), w [experts, 2 N, K] (gate rows, then up rows), out [pairs, N] = pair rule(gate, up).  second: a
    [pairs, K], w [experts, N, K], out [pairs, N] 32-bit = the pair's weight times the product.  first without `gated`:
    w [experts, N, K], out [pairs, N] = activation(product).  `w` holds the experts with tensors; pairs whose expert has a
    higher number (sorted behind them) are left alone."""
    e, rows_w, k = w.shape
    n = rows_w // 2 if first and gated else rows_w
    _need(a, "a", (torch.float32, torch.bfloat16), (None, k))
    _need(w, "w", a.dtype)
    _need(out, "out", a.dtype if first else torch.float32, (None, n))
    if out.shape[0] < pairs or (not first and a.shape[0] < pairs):
        raise ShapeError(f"moe_expert: {pairs} rows asked of shorter tensors")
    if activation not in (PAIR_RULES if gated else ACTIVATIONS):
        raise ShapeError(f"moe_expert: unknown activation {activation!r}")
    _work(2.0 * pairs * rows_w * k, w.numel() * w.element_size() + pairs * (k * a.element_size() + n * out.element_size()))
    _check(library().bt_moe_expert(c_int((1 if gated else 2) if first else 0), _ptr(a), c_longlong(a.stride(0)), _ptr(w), _ptr(out),
                                   _ptr(offsets), _ptr(tile_first), _ptr(order), _ptr(pair_weight), c_int(pairs), c_int(e),
                                   c_int(top), c_int(k), c_int(n), c_int(PAIR_RULES[activation]), c_float(limit),
                                   c_int(1 if tensor_cores else 0), c_int(_code(a.dtype)), _stream()))


def moe_combine(part, place, stream_rows, *, n_tokens, top, ids=None, weights=None, identity_input=None, n_stored=0,
                store=False):
    """stream_rows[t] += sum over the token's `top` pairs of part[place[t * top + j]], in that order (32-bit).  With `ids`
    ([tokens, top], the pairs' experts), a pair whose expert is `n_stored` or more adds weights[t, j] * identity_input[t]
    instead (an expert without tensors that hands its input on; identity_input: contiguous 32-bit [tokens, width]).
    `store`: the sums are written into stream_rows instead of added (rows that hold nothing yet)."""
    width = stream_rows.shape[1]
    if ids is not None:
        _need(ids, "ids", torch.int32, (None, top))
        _need(weights, "weights", torch.float32, (None, top))
        _need(identity_input, "identity_input", torch.float32, (None, width))
        if min(ids.shape[0], weights.shape[0], identity_input.shape[0]) < n_tokens:
            raise ShapeError(f"moe_combine: {n_tokens} tokens asked of shorter tensors")
    _need(part, "part", torch.float32, (None, width))
    _need(place, "place", torch.int32)
    _need(stream_rows, "stream_rows", torch.float32)
    if stream_rows.shape[0] < n_tokens or place.numel() < n_tokens * top:
        raise ShapeError(f"moe_combine: {n_tokens} tokens asked of shorter tensors")
    _work(0.0, 4.0 * n_tokens * width * (top + 2))
    _check(library().bt_moe_combine(_ptr(part), _ptr(place), _ptr(stream_rows), c_longlong(n_tokens), c_int(top),
                                    c_int(width), _ptr(ids), _ptr(weights), _ptr(identity_input), c_int(n_stored),
                                    c_int(1 if store else 0), _stream()))


def scale_(x, factor: float):
    """x *= factor for a contiguous 32-bit tensor."""
    _need(x, "x", torch.float32)
    _check(library().bt_scale(_ptr(x), c_longlong(x.numel()), c_float(factor), _stream()))


def latent_gather(pool, positions, token_seq, table, table_len, rows, *, n_tokens):
    """rows[t] = the cached row at token t's own position: the step's latent rows side by side."""
    dk = pool.shape[2]
    _need(pool, "pool", (torch.float32, torch.bfloat16), (None, PAGE_SIZE, dk))
    _need(rows, "rows", pool.dtype, (None, dk))
    _need(table, "table", torch.int32)
    if rows.shape[0] < n_tokens:
        raise ShapeError(f"latent_gather: {n_tokens} tokens asked of rows[{rows.shape[0]}]")
    _work(0.0, 2.0 * n_tokens * dk * pool.element_size())
    _check(library().bt_latent_gather(_ptr(pool), _ptr(positions), _ptr(token_seq), _ptr(table), c_int(table.shape[1]),
                                      c_int(table_len), c_int(PAGE_SIZE), _ptr(rows), c_int(n_tokens), c_int(dk),
                                      c_int(_code(pool.dtype)), _stream()))


def _sink_attention_strides(q, k, v, gate, out):
    heads = q.shape[1]
    strides = []
    for name, t, width in (("q", q, q.shape[2]), ("k", k, q.shape[2]), ("v", v, v.shape[2]),
                           ("gate", gate, v.shape[2]), ("out", out, v.shape[2])):
        strides.append((0, 0) if t is None else _head_view(t, name, heads, width))
    return strides


def sink_attention_supports(q, k, v, gate, out) -> bool:
    """Whether sink_attention takes these views: bfloat16, whole 16-byte pieces per head and token, at most 128 value
    channels, operands on 16-byte boundaries."""
    if any(t is not None and t.dtype is not torch.bfloat16 for t in (q, k, v, gate, out)):
        return False
    (qr, qh), (kr, kh), (vr, vh), (gr, gh), (orow, oh) = _sink_attention_strides(q, k, v, gate, out)
    if any(t.data_ptr() % 16 for t in (q, k, v)) or out.data_ptr() % 4 or (gate is not None and gate.data_ptr() % 4):
        return False
    return bool(library().bt_sink_attention_supports(c_int(q.shape[2]), c_int(v.shape[2]), c_longlong(qr), c_int(qh),
                                                     c_longlong(kr), c_int(kh), c_longlong(vr), c_int(vh), c_longlong(gr),
                                                     c_int(gh), c_longlong(orow), c_int(oh)))


def sink_attention(q, k, v, out, seq_start, *, n_seqs, max_new, scale, sink=None, gate=None, window=0):
    """Causal multi-head attention of sequences that start at position 0, on tensor cores (bfloat16): token t of a
    sequence sees the sequence's tokens up to itself.  q, k: views [tokens, heads, dq]; v, out, gate: views
    [tokens, heads, dv].  `sink` [heads] adds exp(sink_h) to head h's softmax denominator; `gate` multiplies the result by
    sigmoid(gate).  Scores, softmax and sums are 32-bit."""
    heads, dq, dv = q.shape[1], q.shape[2], v.shape[2]
    if not sink_attention_supports(q, k, v, gate, out):
        raise ShapeError("sink_attention: the kernel does not take these views (see sink_attention_supports)")
    if sink is not None:
        _need(sink, "sink", torch.float32, (heads,))
    (qr, qh), (kr, kh), (vr, vh), (gr, gh), (orow, oh) = _sink_attention_strides(q, k, v, gate, out)
    if _PROFILE is not None:
        ctx = float(_PROFILE.context_hint or 0)
        _work(2.0 * q.shape[0] * heads * (ctx / 2) * (dq + dv), 2.0 * q.shape[0] * heads * (2 * dq + 2 * dv))
    _check(library().bt_sink_attention(_ptr(q), c_longlong(qr), c_int(qh), _ptr(k), c_longlong(kr), c_int(kh), _ptr(v),
                                       c_longlong(vr), c_int(vh), _ptr(gate), c_longlong(gr), c_int(gh), _ptr(out),
                                       c_longlong(orow), c_int(oh), _ptr(seq_start), _ptr(sink), c_int(n_seqs),
                                       c_int(max_new), c_int(heads), c_int(dq), c_int(dv), c_float(scale), c_int(window),
                                       c_int(0), c_int(1), c_int(0), c_void_p(0), _stream()))


def latent_decode_prep(proj, q_off, latent_off, uk_heads, norm_weight, eps, positions, token_seq, inv_freq, rot_dims, table,
                       table_len, pool, q_latent, *, n_tokens, n_heads, dim, rank, rot, owns, latent_rows=None):
    """For steps of few tokens, in one launch: q_latent[t, h] = [W_uk,h^T q_plain | q_rot turned by the position], and
    (if `owns`) the token's own latent row normed, turned and filed in its page.  proj: [tokens, width] rows with the
    queries at `q_off` (per head dim + rot channels) and the latent row at `latent_off`, or, with `latent_rows` (a view
    [tokens, rank + rot] with contiguous channels), the latent rows there; uk_heads: [heads, dim, rank]."""
    _need(proj, "proj", (torch.float32, torch.bfloat16))
    if latent_rows is not None:
        if (latent_rows.dim() != 2 or latent_rows.shape[1] != rank + rot or latent_rows.stride(1) != 1
                or latent_rows.dtype is not proj.dtype or not latent_rows.is_cuda or latent_rows.shape[0] < n_tokens):
            raise ShapeError(f"latent_decode_prep: latent_rows must be a device view [>= {n_tokens}, {rank + rot}] of the "
                             f"queries' type with contiguous channels")
        latent_off = 0
    _need(uk_heads, "uk_heads", proj.dtype, (n_heads, dim, rank))
    _need(pool, "pool", proj.dtype, (None, PAGE_SIZE, rank + rot))
    _need(q_latent, "q_latent", proj.dtype, (None, n_heads * (rank + rot)))
    _need(inv_freq, "inv_freq", torch.float32)
    if owns:
        _need(norm_weight, "norm_weight", torch.float32, (rank,))
    if q_off + n_heads * (dim + rot) > proj.shape[1] or (owns and latent_rows is None
                                                         and latent_off + rank + rot > proj.shape[1]):
        raise ShapeError("latent_decode_prep: the channel offsets leave the rows of proj")
    if proj.shape[0] < n_tokens or q_latent.shape[0] < n_tokens or inv_freq.numel() < rot_dims // 2:
        raise ShapeError("latent_decode_prep: too few rows or frequencies")
    _check(library().bt_latent_decode_prep(_ptr(proj), c_longlong(proj.shape[1]), c_int(q_off), c_int(latent_off),
                                           _ptr(latent_rows),
                                           c_longlong(latent_rows.stride(0) if latent_rows is not None else 0),
                                           _ptr(uk_heads), _ptr(norm_weight if owns else None), c_float(eps),
                                           _ptr(positions), _ptr(token_seq), _ptr(inv_freq), c_int(rot_dims), _ptr(table),
                                           c_int(table.shape[1]), c_int(table_len), c_int(PAGE_SIZE), _ptr(pool),
                                           _ptr(q_latent), c_int(n_tokens), c_int(n_heads), c_int(dim), c_int(rank),
                                           c_int(rot), c_int(1 if owns else 0), c_int(_code(proj.dtype)), _stream()))


def latent_decode_finish(uv_heads, out, *, n_tokens, n_splits, scratch=None, mixed_latent=None, gate=None):
    """For steps of few tokens, in one launch: joins the `n_splits` partial results of latent_attention(merge=False) in
    `scratch` (or reads `mixed_latent` [tokens, heads * rank] when there was one split), multiplies each head's weighted
    latent by uv_heads[h] ([heads, rank, vdim]) and by sigmoid(gate).  out: [tokens, heads * vdim]; gate: a view
    [tokens, heads * vdim] with contiguous channels."""
    n_heads, rank, vdim = uv_heads.shape
    _need(uv_heads, "uv_heads", (torch.float32, torch.bfloat16), (n_heads, rank, vdim))
    _need(out, "out", uv_heads.dtype, (None, n_heads * vdim))
    if n_splits > 1:
        need = latent_attention_scratch_floats(n_tokens, n_heads, rank, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise ShapeError(f"latent_decode_finish: {n_splits} splits leave {need} floats of partial results")
    else:
        _need(mixed_latent, "mixed_latent", uv_heads.dtype, (None, n_heads * rank))
    g_rs = 0
    if gate is not None:
        if gate.dim() != 2 or gate.shape[1] != n_heads * vdim or gate.stride(1) != 1 or gate.dtype is not uv_heads.dtype:
            raise ShapeError("latent_decode_finish: gate must be a view [tokens, heads * vdim] of the weights' type")
        g_rs = gate.stride(0)
    _check(library().bt_latent_decode_finish(_ptr(scratch if n_splits > 1 else None),
                                             _ptr(mixed_latent if n_splits == 1 else None), c_int(n_splits), _ptr(uv_heads),
                                             _ptr(gate), c_longlong(g_rs), _ptr(out), c_longlong(out.shape[1]),
                                             c_int(n_tokens), c_int(n_heads), c_int(rank), c_int(vdim),
                                             c_int(_code(uv_heads.dtype)), _stream()))


# ---- a sublayer's normed result into the stream; the polynomial activation; the half-split rotation -----------------

def rmsnorm_add(x, weight, stream_rows, eps: float, *, n_rows, next_weight=None, next_out=None, factor: float = 1.0):
    """stream_rows[r] += factor * x[r] / sqrt(mean(x[r]^2) + eps) * weight for contiguous 32-bit [rows, width] tensors.
    With `next_out` ([rows, width], 32-bit or bfloat16) the updated row is also written there: normed again with
    `next_weight`, or, without one, as it is (rounded to next_out's type)."""
    width = weight.shape[0]
    _need(x, "x", torch.float32, (None, width))
    _need(stream_rows, "stream_rows", torch.float32, (None, width))
    _need(weight, "weight", torch.float32, (width,))
    if min(x.shape[0], stream_rows.shape[0]) < n_rows:
        raise ShapeError(f"rmsnorm_add: {n_rows} rows asked of shorter tensors")
    if next_weight is not None and next_out is None:
        raise ShapeError("rmsnorm_add: the second norm needs a place for its rows")
    if next_out is not None:
        if next_weight is not None:
            _need(next_weight, "next_weight", torch.float32, (width,))
        _need(next_out, "next_out", (torch.float32, torch.bfloat16), (None, width))
        if next_out.shape[0] < n_rows:
            raise ShapeError(f"rmsnorm_add: {n_rows} rows asked of next_out[{next_out.shape[0]}]")
    _work(0.0, n_rows * width * (12.0 + (next_out.element_size() if next_out is not None else 0)))
    _check(library().bt_rmsnorm_add(_ptr(x), _ptr(weight), _ptr(stream_rows), _ptr(next_weight), _ptr(next_out),
                                    c_int(_code(next_out.dtype)) if next_out is not None else c_int(0),
                                    c_longlong(n_rows), c_int(width), c_float(eps), c_float(factor), _stream()))


def polynorm(x, coef, out, eps: float, *, n_rows):
    """out[r] = a N(z) + b N(z^2) + c N(z^3) + e for every row z of x, with the powers taken element by element,
    N(v) = v / sqrt(mean(v^2) + eps) over the row and coef = (a, b, c, e) 32-bit on the device; 32-bit arithmetic."""
    _need(x, "x", (torch.float32, torch.bfloat16))
    _need(out, "out", x.dtype, (None, x.shape[1]))
    _need(coef, "coef", torch.float32, (4,))
    if min(x.shape[0], out.shape[0]) < n_rows:
        raise ShapeError(f"polynorm: {n_rows} rows asked of shorter tensors")
    _work(0.0, 2.0 * n_rows * x.shape[1] * x.element_size())
    _check(library().bt_polynorm(_ptr(x), _ptr(coef), _ptr(out), c_longlong(n_rows), c_int(x.shape[1]), c_float(eps),
                                 c_int(_code(x.dtype)), _stream()))


def rotary_half(src, dst, positions, inv_freq, *, n_tokens, n_vecs, length, dims, scaled_from=None, scale=1.0, tail=0):
    """dst (32-bit) = the first n_vecs * length channels of src's rows as vectors of `length` channels, channel i <
    dims / 2 of each paired with channel i + dims / 2 and the pair turned by positions[t] * inv_freq[i] (32-bit angles);
    vectors from `scaled_from` on are then multiplied by `scale`; the `tail` channels after the vectors are copied."""
    need = n_vecs * length + tail
    for name, t in (("src", src), ("dst", dst)):
        if t.dim() != 2 or t.shape[1] < need or t.stride(1) != 1 or not t.is_cuda or t.shape[0] < n_tokens:
            raise ShapeError(f"rotary_half: {name} must be a device view [>= {n_tokens}, >= {need}] with contiguous channels")
    if dst.dtype != torch.float32 or src.dtype not in DTYPE_CODE:
        raise ShapeError("rotary_half: dst is 32-bit, src 32-bit or bfloat16")
    _need(inv_freq, "inv_freq", torch.float32)
    if inv_freq.numel() < dims // 2:
        raise ShapeError(f"rotary_half: {inv_freq.numel()} frequencies for {dims} rotated channels")
    _check(library().bt_rotary_half(_ptr(src), c_longlong(src.stride(0)), c_int(_code(src.dtype)), _ptr(dst),
                                    c_longlong(dst.stride(0)), _ptr(positions), _ptr(inv_freq), c_int(n_tokens),
                                    c_int(n_vecs), c_int(length), c_int(dims),
                                    c_int(n_vecs if scaled_from is None else scaled_from), c_float(scale), c_int(tail),
                                    _stream()))


# ---- short convolution, talking attention, selective scan -------------------------------------------------------------

def _channels_view(t, name, rows, width):
    if t.dim() != 2 or t.shape[1] != width or t.stride(1) != 1 or not t.is_cuda or t.shape[0] < rows:
        raise ShapeError(f"{name} must be a device view [>= {rows}, {width}] with contiguous channels, found "
                         f"{list(t.shape)} strides {list(t.stride())}")


def short_conv(src, weight, bias, state, slots, seq_start, token_seq, out, *, n_tokens, n_seqs, activation=None,
               norm_group=0, eps=0.0, raw_out=None, raw_first_group=0):
    """y[t, c] = act(bias[c] + sum_j weight[c, j] * u[t - taps + 1 + j, c]) over the step's rows `src` [tokens, channels],
    causal within each sequence; the inputs before the step come from `state` [slots, taps - 1, channels] (32-bit, zeros
    for a new sequence), which afterwards holds the sequences' newest inputs.  `activation` "swish": x * sigmoid(x).
    With `norm_group` every run of that many channels of y is divided by its root mean square (eps inside the root) and,
    with `raw_out`, the runs from `raw_first_group` on are also written undivided there."""
    channels, taps = weight.shape
    _need(weight, "weight", torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32, (channels,))
    _need(state, "state", torch.float32, (None, max(taps - 1, 0), channels))
    _channels_view(src, "short_conv: src", n_tokens, channels)
    _channels_view(out, "short_conv: out", n_tokens, channels)
    if src.dtype not in DTYPE_CODE or out.dtype not in DTYPE_CODE:
        raise ShapeError("short_conv: rows are 32-bit or bfloat16")
    if activation not in (None, "swish"):
        raise ShapeError(f"short_conv: unknown activation {activation!r}")
    raw_stride = 0
    if raw_out is not None:
        if not norm_group or raw_out.dtype != out.dtype:
            raise ShapeError("short_conv: undivided rows come with a norm only, in the type of out")
        _channels_view(raw_out, "short_conv: raw_out", n_tokens, channels - raw_first_group * norm_group)
        raw_stride = raw_out.stride(0)
    _work(2.0 * n_tokens * channels * taps, n_tokens * channels * (src.element_size() + out.element_size()))
    _check(library().bt_short_conv(_ptr(src), c_longlong(src.stride(0)), c_int(_code(src.dtype)), _ptr(weight), _ptr(bias),
                                   _ptr(state), _ptr(slots), _ptr(seq_start), _ptr(token_seq), _ptr(out),
                                   c_longlong(out.stride(0)), c_int(_code(out.dtype)), _ptr(raw_out), c_longlong(raw_stride),
                                   c_int(raw_first_group), c_longlong(n_tokens), c_int(n_seqs), c_int(channels), c_int(taps),
                                   c_int(1 if activation == "swish" else 0), c_int(norm_group), c_float(eps), _stream()))


TALK_SPLIT_ROWS = 16      # a step that brings at most this many tokens a sequence may share a sequence's keys among blocks
TALK_KEY_TILE = 32
N_SMS = 148               # of a B200


def talking_attention_split(n_seqs: int, max_new: int, n_heads: int, head_dim: int, window: int, ctx_bound: int):
    """Among how many blocks the tensor-core form shares the keys of every sequence in a step of `n_seqs` sequences that
    brings at most `max_new` tokens to each and leaves none longer than `ctx_bound`, and the 32-bit numbers of scratch
    they meet in: enough blocks to fill the GPU about twice, no more than a sequence has tiles of keys.  (1, 0): no
    sharing."""
    if max_new > TALK_SPLIT_ROWS or n_seqs <= 0:
        return 1, 0
    seen = min(ctx_bound, window + max_new - 1) if window else ctx_bound
    tiles = -(-seen // TALK_KEY_TILE) + 1
    n_split = max(1, min(tiles, -(-2 * N_SMS // n_seqs)))
    if n_split == 1:
        return 1, 0
    return n_split, n_seqs * n_split * n_heads * max_new * (head_dim + 2)


def talking_attention(q, out, seq_start, past_len, *, n_seqs, max_new, n_heads, n_kv_heads, head_dim, scale, window=0,
                      cap=0.0, temp=None, slope=None, talk=None, gate=None, out_scale=1.0, k=None, v=None, k_pool=None,
                      v_pool=None, table=None, table_len=0, plain=False, n_split=1, parts=None):
    """Causal (windowed) attention over all heads of a token at once (csrc/talking_attention.cu):
    raw_g = cap tanh((q_g . k_g) scale temp[g] / cap) - slope[g] (i - j), s_h = sum_g talk[h, g] raw_g, softmax over the
    visible keys, the value mix, times sigmoid(gate) and out_scale.  q, gate, out: views [tokens, heads * head_dim];
    keys and values either views [tokens, kv_heads * head_dim] of the step's own rows (`k`, `v`: sequences that start in
    this step) or the pages of the cache.  bfloat16 rows whose heads have a multiple of 8 channels (up to 128) run on
    tensor cores (csrc/talking_attention_mma.cu) unless `plain` is set; 32-bit rows and the rest in plain arithmetic.
    With `n_split` > 1 and `parts` (32-bit, as talking_attention_split says) that form shares every sequence's keys among
    n_split blocks."""
    width = n_heads * head_dim
    if n_split > 1:
        if max_new > TALK_SPLIT_ROWS or parts is None or parts.dtype != torch.float32 or not parts.is_contiguous() \
                or parts.numel() < n_seqs * n_split * n_heads * max_new * (head_dim + 2):
            raise ShapeError("talking_attention: sharing the keys among blocks needs a step of few tokens and scratch")
    for name, t in (("q", q), ("out", out)) + ((("gate", gate),) if gate is not None else ()):
        _channels_view(t, "talking_attention: " + name, 0, width)
        if t.dtype != q.dtype:
            raise ShapeError("talking_attention: q, gate and out have one type")
    if q.dtype not in DTYPE_CODE:
        raise ShapeError("talking_attention: rows are 32-bit or bfloat16")
    for name, t, shape in (("temp", temp, (n_heads,)), ("slope", slope, (n_heads,)), ("talk", talk, (n_heads, n_heads))):
        if t is not None:
            _need(t, name, torch.float32, shape)
    if table is None:
        for name, t in (("k", k), ("v", v)):
            _channels_view(t, "talking_attention: " + name, 0, n_kv_heads * head_dim)
            if t.dtype != q.dtype or t.stride(0) != k.stride(0):
                raise ShapeError("talking_attention: k and v are rows of one tensor of q's type")
        k_ptr, v_ptr, t_ptr, t_stride, kv_stride = _ptr(k), _ptr(v), c_void_p(0), 0, k.stride(0)
    else:
        _need(k_pool, "k_pool", q.dtype)
        _need(v_pool, "v_pool", q.dtype)
        _need(table, "table", torch.int32)
        k_ptr, v_ptr, t_ptr, t_stride, kv_stride = _ptr(k_pool), _ptr(v_pool), _ptr(table), table.shape[1], 0
    if _PROFILE is not None:
        seen = float(min(window or 1 << 30, _PROFILE.context_hint or max_new))
        rows = float(out.shape[0] if max_new > 1 else n_seqs)
        _work(4.0 * rows * n_heads * seen * head_dim, rows * (2 * width + 2 * n_kv_heads * head_dim) * q.element_size())
    _check(library().bt_talking_attention(
        _ptr(q), c_longlong(q.stride(0)), k_ptr, v_ptr, t_ptr, c_int(t_stride), c_int(table_len), c_int(PAGE_SIZE),
        c_longlong(kv_stride), _ptr(gate), c_longlong(gate.stride(0) if gate is not None else 0), _ptr(out),
        c_longlong(out.stride(0)), _ptr(seq_start), _ptr(past_len), _ptr(temp), _ptr(slope), _ptr(talk), c_int(n_seqs),
        c_int(max_new), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_float(cap), c_int(window),
        c_float(out_scale), c_int(1 if plain else 0), c_int(n_split if n_split > 1 else 1),
        _ptr(parts) if n_split > 1 else c_void_p(0), c_int(_code(q.dtype)), _stream()))


def selective_scan_dt(low, w_dt, b_dt, dt, *, n_tokens):
    """dt[t, c] = softplus(sum_r w_dt[c, r] * low[t, r] + b_dt[c]), 32-bit; low: a view whose first `rank` channels are
    read; w_dt [channels, rank], b_dt [channels] 32-bit."""
    channels, rank = w_dt.shape
    _need(w_dt, "w_dt", torch.float32)
    _need(b_dt, "b_dt", torch.float32, (channels,))
    _need(dt, "dt", torch.float32, (None, channels))
    if low.dim() != 2 or low.shape[1] < rank or low.stride(1) != 1 or low.dtype not in DTYPE_CODE or low.shape[0] < n_tokens \
            or dt.shape[0] < n_tokens:
        raise ShapeError("selective_scan_dt: low must hold the step's rows with at least `rank` contiguous channels")
    _work(2.0 * n_tokens * channels * rank, 4.0 * n_tokens * channels)
    _check(library().bt_selective_scan_dt(_ptr(low), c_longlong(low.stride(0)), _ptr(w_dt), _ptr(b_dt), _ptr(dt),
                                          c_longlong(n_tokens), c_int(channels), c_int(rank), c_int(_code(low.dtype)),
                                          _stream()))


SCAN_PIECE = 64          # tokens of a run that one block of the selective scan walks, while a run has at most ...
SCAN_MAX_PIECES = 64     # ... this many pieces


def selective_scan_pieces(max_new: int, n_tokens: int, n_seqs: int, channels: int, n_state: int):
    """How the selective scan cuts the runs of a step whose longest has `max_new` tokens: (tokens a piece, the most
    pieces of a run, 32-bit numbers of scratch).  (0, 1, 0): every run is one piece and needs no scratch."""
    if max_new <= SCAN_PIECE:
        return 0, 1, 0
    piece = max(SCAN_PIECE, -(-max_new // SCAN_MAX_PIECES))
    piece = (piece + 15) // 16 * 16
    return piece, -(-max_new // piece), (n_tokens // piece + n_seqs + 1) * channels * (n_state + 1)


def selective_scan(x, z, dt, low, b_off, c_off, a_log, d_skip, state, slots, seq_start, out, *, n_seqs, out_scale=1.0,
                   max_new=0, scratch=None):
    """The scan S[c, n] <- exp(dt A) S + dt x B_n, y = (S . C + D x) * z sigmoid(z) * out_scale over the step's tokens of
    every sequence (csrc/selective_scan.cu).  x, z, out: views [tokens, channels]; dt [tokens, channels] 32-bit; B and C
    are the channels b_off.. and c_off.. of the rows of `low`; a_log [channels, n_state], d_skip [channels] 32-bit;
    state [slots, channels, n_state] 32-bit, read and written at `slots[seq]`.  With `max_new` (the longest run of the
    step) and `scratch` (32-bit, as many numbers as selective_scan_pieces says) long runs are cut into pieces that run
    side by side; without them a block walks a whole run."""
    channels, n_state = a_log.shape
    _need(a_log, "a_log", torch.float32)
    _need(d_skip, "d_skip", torch.float32, (channels,))
    _need(state, "state", torch.float32, (None, channels, n_state))
    _need(dt, "dt", torch.float32, (None, channels))
    rows = dt.shape[0]
    for name, t in (("x", x), ("z", z), ("out", out)):
        _channels_view(t, "selective_scan: " + name, 0, channels)
        if t.dtype != x.dtype:
            raise ShapeError("selective_scan: x, z and out have one type")
    if low.dim() != 2 or low.stride(1) != 1 or low.dtype != x.dtype or max(b_off, c_off) + n_state > low.shape[1] \
            or min(b_off, c_off) < 0:
        raise ShapeError("selective_scan: B and C must be channels of the rows of low, of x's type")
    piece, max_pieces, need = selective_scan_pieces(max_new, rows, n_seqs, channels, n_state) if scratch is not None \
        else (0, 1, 0)
    if piece:
        if scratch.dtype != torch.float32 or not scratch.is_contiguous() or scratch.numel() < need:
            raise ShapeError(f"selective_scan: runs of up to {max_new} tokens in pieces need {need} floats of scratch")
    _work(6.0 * rows * channels * n_state, rows * channels * (3 * x.element_size() + 4) + 8.0 * n_seqs * channels * n_state)
    _check(library().bt_selective_scan(_ptr(x), c_longlong(x.stride(0)), _ptr(z), c_longlong(z.stride(0)), _ptr(dt), _ptr(low),
                                       c_longlong(low.stride(0)), c_int(b_off), c_int(c_off), _ptr(a_log), _ptr(d_skip),
                                       _ptr(state), _ptr(slots), _ptr(seq_start), _ptr(out), c_longlong(out.stride(0)),
                                       c_int(n_seqs), c_int(channels), c_int(n_state), c_float(out_scale), c_int(piece),
                                       c_int(max_pieces), _ptr(scratch) if piece else c_void_p(0),
                                       c_int(_code(x.dtype)), _stream()))


# ---- token shift, sigmoid attention -----------------------------------------------------------------------------------

def token_shift(x, shift, state, slots, seq_start, token_seq, out, *, n_rows):
    """out[t] = x[t] + (x[t - 1] - x[t]) * shift over the step's rows (32-bit arithmetic, rounded to out's type); the row
    before a sequence's first row of the step is state[slot], which afterwards holds the sequence's last row of x.
    x: contiguous 32-bit [rows, width]; shift: 32-bit [width]; state: 32-bit [slots, width]; out: [rows, width]."""
    width = shift.shape[0]
    _need(x, "x", torch.float32, (None, width))
    _need(shift, "shift", torch.float32, (width,))
    _need(state, "state", torch.float32, (None, width))
    _need(out, "out", (torch.float32, torch.bfloat16), (None, width))
    if min(x.shape[0], out.shape[0]) < n_rows:
        raise ShapeError(f"token_shift: {n_rows} rows asked of shorter tensors")
    _work(0.0, n_rows * width * (8.0 + out.element_size()))
    _check(library().bt_token_shift(_ptr(x), _ptr(shift), _ptr(state), _ptr(slots), _ptr(seq_start), _ptr(token_seq),
                                    _ptr(out), c_int(_code(out.dtype)), c_longlong(n_rows), c_int(width), _stream()))


def sigmoid_attention_prep(proj, q_weight, k_weight, eps, positions, token_seq, inv_freq, rot_dims, table, table_len, pool,
                           *, n_tokens, n_heads, n_kv_heads, dim, vdim, mix=None, v_other=None, v_publish=None):
    """Prepares a step's projections `proj` [tokens, (heads + kv_heads) * dim + kv_heads * vdim] (queries, keys, values)
    for sigmoid_attention: query and key heads divided by their root mean square times `q_weight` / `k_weight` [dim] and
    their first `rot_dims` channels turned by the position (channel i with channel i + rot_dims / 2, angle position *
    inv_freq[i]); value heads divided by their root mean square and, with `v_other` (32-bit [tokens, kv_heads * vdim]) and
    `mix` (a 32-bit number on the device), replaced by (1 - mix) v + mix v_other; `v_publish` receives the values as
    they end up.  Queries, keys and values are rewritten in place, and keys and values also go to the token's rows of
    `pool` [pages, kv_heads, PAGE_SIZE, dim + vdim]."""
    width = (n_heads + n_kv_heads) * dim + n_kv_heads * vdim
    _need(proj, "proj", (torch.float32, torch.bfloat16), (None, width))
    _need(pool, "pool", proj.dtype, (None, n_kv_heads, PAGE_SIZE, dim + vdim))
    _need(q_weight, "q_weight", torch.float32, (dim,))
    _need(k_weight, "k_weight", torch.float32, (dim,))
    _need(inv_freq, "inv_freq", torch.float32)
    _need(table, "table", torch.int32)
    if inv_freq.numel() < rot_dims // 2 or proj.shape[0] < n_tokens:
        raise ShapeError("sigmoid_attention_prep: too few rows or frequencies")
    if (v_other is None) != (mix is None):
        raise ShapeError("sigmoid_attention_prep: mixing needs both the other values and the mixing number")
    for name, t in (("v_other", v_other), ("v_publish", v_publish)):
        if t is not None:
            _need(t, name, torch.float32, (None, n_kv_heads * vdim))
            if t.shape[0] < n_tokens:
                raise ShapeError(f"sigmoid_attention_prep: {n_tokens} tokens asked of {name}[{t.shape[0]}]")
    if mix is not None:
        _need(mix, "mix", torch.float32)
    _work(0.0, 2.0 * n_tokens * width * proj.element_size())
    _check(library().bt_sigmoid_attention_prep(
        _ptr(proj), c_longlong(proj.shape[1]), _ptr(q_weight), _ptr(k_weight), c_float(eps), _ptr(positions),
        _ptr(token_seq), _ptr(inv_freq), c_int(rot_dims), _ptr(mix), _ptr(v_other), _ptr(v_publish), _ptr(table),
        c_int(table.shape[1]), c_int(table_len), c_int(PAGE_SIZE), _ptr(pool), c_int(n_tokens), c_int(n_heads),
        c_int(n_kv_heads), c_int(dim), c_int(vdim), c_int(_code(proj.dtype)), _stream()))


def sigmoid_attention_tcgen05_supports(dim: int, vdim: int, row_stride: int) -> bool:
    """Whether sigmoid_attention_tcgen05 takes these sizes: keys and values of 64 or 128 channels a head each, rows of
    whole 16-byte pieces."""
    return (row_stride % 8 == 0 and _supports("bt_attention_prefill_tcgen05_supports", dim, PAGE_SIZE)
            and _supports("bt_attention_prefill_tcgen05_supports", vdim, PAGE_SIZE))


def sigmoid_attention_tcgen05(proj, out, seq_start, past_len, *, n_seqs, max_new, n_heads, n_kv_heads, head_dim, scale,
                              v_dim=None, bias=None, window=0, keep_first=0, pool=None, table=None, table_len=0):
    """sigmoid_attention on the tcgen05 tensor cores (bfloat16; scores in tensor memory): `proj` rows hold the prepared
    queries, keys (heads of `head_dim` channels) and values (heads of `v_dim` channels, `head_dim` if not given) one
    after another; out: [tokens, heads * v_dim].  Keys and values are the step's own rows (sequences that start at
    position 0), or, with `pool` [pages, kv_heads, PAGE_SIZE, head_dim + v_dim] and `table`, the sequences' pages.
    Scores and sigmoids in 32-bit; a weight enters the value product rounded to bfloat16, the sums are 32-bit."""
    v_dim = head_dim if v_dim is None else v_dim
    _need(proj, "proj", torch.bfloat16, (None, (n_heads + n_kv_heads) * head_dim + n_kv_heads * v_dim))
    _need(out, "out", torch.bfloat16, (None, n_heads * v_dim))
    if bias is not None:
        _need(bias, "bias", torch.float32, (n_heads,))
    if not sigmoid_attention_tcgen05_supports(head_dim, v_dim, proj.shape[1]):
        raise ShapeError(f"sigmoid_attention_tcgen05: heads of {head_dim} and {v_dim} channels in rows of {proj.shape[1]}")
    if _PROFILE is not None:
        ctx = float(_PROFILE.context_hint or 0)
        seen = min(ctx / 2, float(window + keep_first)) if window else ctx / 2
        _work(2.0 * proj.shape[0] * n_heads * seen * (head_dim + v_dim),
              2.0 * proj.shape[0] * ((n_heads + n_kv_heads) * head_dim + (n_heads + n_kv_heads) * v_dim))
    q_width, k_width = n_heads * head_dim, n_kv_heads * head_dim
    if table is None:
        k_ptr = c_void_p(proj.data_ptr() + q_width * 2)
        v_ptr = c_void_p(proj.data_ptr() + (q_width + k_width) * 2)
        t_ptr, t_stride, pages, row = c_void_p(0), 0, 0, 0
    else:
        _need(pool, "pool", torch.bfloat16, (None, n_kv_heads, PAGE_SIZE, head_dim + v_dim))
        _need(table, "table", torch.int32)
        k_ptr, v_ptr = _ptr(pool), c_void_p(pool.data_ptr() + head_dim * 2)
        t_ptr, t_stride, pages, row = _ptr(table), table.shape[1], pool.shape[0], head_dim + v_dim
    _check(library().bt_sigmoid_attention_tcgen05(
        _ptr(proj), c_longlong(proj.shape[0]), c_longlong(proj.shape[1]), k_ptr, v_ptr, c_longlong(pages), t_ptr,
        c_int(t_stride), c_int(table_len), c_int(PAGE_SIZE), _ptr(out), _ptr(kernel_status(proj.device)), _ptr(seq_start),
        _ptr(past_len), c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(v_dim),
        c_float(scale), _ptr(bias), c_int(window), c_int(keep_first), c_longlong(row), _stream()))


def _grouped_views(q, k, v, out):
    """Strides of q [tokens, heads, dq], k [tokens, kv_heads, dq], v [tokens, kv_heads, dv], out [tokens, heads, dv]."""
    heads, groups, dq, dv = q.shape[1], k.shape[1], q.shape[2], v.shape[2]
    return (_head_view(q, "q", heads, dq), _head_view(k, "k", groups, dq), _head_view(v, "v", groups, dv),
            _head_view(out, "out", heads, dv))


def sigmoid_attention_prompt_supports(q, k, v, out) -> bool:
    """Whether sigmoid_attention_prompt takes these views: bfloat16, whole 16-byte pieces per head and token, at most 128
    value channels, operands on 16-byte boundaries, the query heads a multiple of the key heads."""
    if any(t.dtype is not torch.bfloat16 for t in (q, k, v, out)) or q.shape[1] % k.shape[1] or v.shape[1] != k.shape[1]:
        return False
    (qr, qh), (kr, kh), (vr, vh), (orow, oh) = _grouped_views(q, k, v, out)
    if any(t.data_ptr() % 16 for t in (q, k, v)) or out.data_ptr() % 4:
        return False
    return bool(library().bt_sink_attention_supports(c_int(q.shape[2]), c_int(v.shape[2]), c_longlong(qr), c_int(qh),
                                                     c_longlong(kr), c_int(kh), c_longlong(vr), c_int(vh), c_longlong(0),
                                                     c_int(0), c_longlong(orow), c_int(oh)))


def sigmoid_attention_prompt(q, k, v, out, seq_start, *, n_seqs, max_new, scale, bias=None, window=0, keep_first=0):
    """sigmoid_attention for sequences that start at position 0, on tensor cores (bfloat16), with keys and values read
    from the step's own rows: q [tokens, heads, dq], k [tokens, kv_heads, dq], v [tokens, kv_heads, dv], out [tokens,
    heads, dv] (views with contiguous channels).  Scores and sigmoids in 32-bit; a weight enters the value product
    rounded to bfloat16, the sums are 32-bit."""
    if not sigmoid_attention_prompt_supports(q, k, v, out):
        raise ShapeError("sigmoid_attention_prompt: views the kernel does not take")
    heads, groups = q.shape[1], k.shape[1]
    (qr, qh), (kr, kh), (vr, vh), (orow, oh) = _grouped_views(q, k, v, out)
    if bias is not None:
        _need(bias, "bias", torch.float32, (heads,))
    if _PROFILE is not None:
        ctx = float(_PROFILE.context_hint or 0)
        seen = min(ctx / 2, float(window + keep_first)) if window else ctx / 2
        _work(2.0 * q.shape[0] * heads * seen * (q.shape[2] + v.shape[2]),
              2.0 * q.shape[0] * (heads * (q.shape[2] + v.shape[2]) + groups * (q.shape[2] + v.shape[2])))
    _check(library().bt_sink_attention(_ptr(q), c_longlong(qr), c_int(qh), _ptr(k), c_longlong(kr), c_int(kh), _ptr(v),
                                       c_longlong(vr), c_int(vh), c_void_p(0), c_longlong(0), c_int(0), _ptr(out),
                                       c_longlong(orow), c_int(oh), _ptr(seq_start), c_void_p(0), c_int(n_seqs),
                                       c_int(max_new), c_int(heads), c_int(q.shape[2]), c_int(v.shape[2]), c_float(scale),
                                       c_int(window), c_int(keep_first), c_int(heads // groups), c_int(1), _ptr(bias),
                                       _stream()))


def sigmoid_attention(q, out, pool, table, table_len, seq_start, past_len, *, n_seqs, max_new, n_heads, n_kv_heads, dim,
                      vdim, scale, bias=None, window=0, keep_first=0):
    """out[t, h] = sum over the positions j that t sees of sigmoid(q[t, h] . k[j, g] * scale + bias[h]) v[j, g], with
    g = h // (heads / kv_heads): nothing is normalised over the keys.  A token at position i sees j <= i with
    i - j < window or j < keep_first (`window` 0: every j <= i).  q: rows whose first heads * dim channels are the
    queries; keys and values: `pool` [pages, kv_heads, PAGE_SIZE, dim + vdim] through `table`; out: [tokens, heads * vdim];
    scores, sigmoids and sums in 32-bit."""
    _need(q, "q", (torch.float32, torch.bfloat16))
    _need(out, "out", q.dtype, (None, n_heads * vdim))
    _need(pool, "pool", q.dtype, (None, n_kv_heads, PAGE_SIZE, dim + vdim))
    _need(table, "table", torch.int32)
    if q.shape[1] < n_heads * dim:
        raise ShapeError(f"sigmoid_attention: rows of {q.shape[1]} channels hold no {n_heads} queries of {dim}")
    if bias is not None:
        _need(bias, "bias", torch.float32, (n_heads,))
    if _PROFILE is not None:
        ctx = float(_PROFILE.context_hint or 0)
        seen = min(ctx if max_new == 1 else ctx / 2, float(window + keep_first) if window else ctx)
        rows = n_seqs * max_new
        _work(2.0 * rows * n_heads * seen * (dim + vdim),
              (rows * n_heads * (dim + vdim) + n_seqs * min(ctx, seen + max_new) * n_kv_heads * (dim + vdim)) * q.element_size())
    _check(library().bt_sigmoid_attention(
        _ptr(q), c_longlong(q.shape[1]), _ptr(pool), _ptr(table), c_int(table.shape[1]), c_int(table_len),
        c_int(PAGE_SIZE), _ptr(seq_start), _ptr(past_len), _ptr(bias), _ptr(out), c_longlong(out.shape[1]), c_int(n_seqs),
        c_int(max_new), c_int(n_heads), c_int(n_kv_heads), c_int(dim), c_int(vdim), c_float(scale), c_int(window),
        c_int(keep_first), c_int(_code(q.dtype)), _stream()))
