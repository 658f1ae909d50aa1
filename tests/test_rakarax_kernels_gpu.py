"""The kernels Rakarax added, each alone against float64: the short convolution with its taps carried from call to
call (both forms), the attention whose heads talk (the step's own rows and scattered pages, windows' edges, one loud
key), the selective scan with its step sizes, the half-split rotation, the recurrence fed with prepared vectors, the
polynomial activation, and the norm that adds a sublayer's result to the stream."""
import numpy as np
import pytest
import torch

import plain_rakarax as plain
from burn_transformers_b200 import kernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).to(DEV)


def rounded(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DT[dtype]).double().numpy()


def ints(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def close(got, want, tol, note=""):
    err = np.abs(got - want).max() / max(1.0, np.abs(want).max())
    assert err < tol, f"{note}{err:.3e}"


def step_tables(lengths):
    starts = np.concatenate([[0], np.cumsum(lengths)])
    token_seq = np.concatenate([np.full(n, i) for i, n in enumerate(lengths)])
    return starts, token_seq


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("channels, taps, with_bias, act", [(40, 4, True, "swish"), (7, 1, False, None), (130, 5, True, None),
                                                              (64, 2, False, "swish"), (33, 16, True, "swish")])
def test_short_convolution_carries_its_taps(dtype, channels, taps, with_bias, act):
    """Three calls on the same slots: runs of many tokens, of fewer tokens than taps, of one token."""
    rng = np.random.default_rng(channels + taps)
    slots = [4, 1, 2]
    w = rng.standard_normal((channels, taps))
    bias = rng.standard_normal(channels) if with_bias else None
    state = torch.zeros((6, taps - 1, channels), device=DEV)
    history = [np.zeros((0, channels)) for _ in slots]
    pad = 3
    for lengths in ([20, 2, 1], [1, 1, 1], [3, 9, 2]):
        starts, token_seq = step_tables(lengths)
        total = starts[-1]
        rows = rounded(rng.standard_normal((total, channels + 2 * pad)), dtype)
        src = dev(rows, DT[dtype])
        out = torch.full((total + 1, channels + pad), 7.0, dtype=DT[dtype], device=DEV)
        kernels.short_conv(src[:, pad:pad + channels], dev(w), None if bias is None else dev(bias), state, ints(slots),
                           ints(starts), ints(token_seq), out[:, :channels], n_tokens=total, n_seqs=len(lengths),
                           activation=act)
        got = out.double().cpu().numpy()
        assert np.all(got[total:] == 7.0) and np.all(got[:, channels:] == 7.0)
        w32 = w.astype(np.float32).astype(np.float64)
        b32 = None if bias is None else bias.astype(np.float32).astype(np.float64)
        for r, (lo, hi) in enumerate(zip(starts[:-1], starts[1:])):
            history[r] = np.concatenate([history[r], rows[lo:hi, pad:pad + channels]])
            want = plain.causal_conv(history[r], w32, b32)[-(hi - lo):]
            if act:
                want = plain.silu(want)
            close(got[lo:hi, :channels], want, TOL[dtype], f"sequence {r}: ")
    for r, slot in enumerate(slots):
        kept = np.concatenate([np.zeros((taps, channels)), history[r]])[len(history[r]) + 1:]
        np.testing.assert_allclose(state[slot].cpu().numpy(), kept, rtol=1e-6)
    assert float(state[0].abs().sum()) == 0 and float(state[5].abs().sum()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("groups, group, first_raw, taps", [(5, 12, 3, 3), (3, 64, 2, 4), (2, 100, 0, 2), (4, 130, 4, 1)])
def test_short_convolution_with_a_norm_per_head(dtype, groups, group, first_raw, taps):
    rng = np.random.default_rng(groups * group)
    channels = groups * group
    lengths, slots = [11, 1, 5], [0, 2, 1]
    w = rng.standard_normal((channels, taps))
    state = torch.zeros((3, taps - 1, channels), device=DEV)
    history = [np.zeros((0, channels)) for _ in slots]
    eps = 1e-3
    for _ in range(2):
        starts, token_seq = step_tables(lengths)
        total = starts[-1]
        rows = rounded(rng.standard_normal((total, channels)), dtype)
        both = torch.zeros((total, channels + (groups - first_raw) * group), dtype=DT[dtype], device=DEV)
        raw = both[:, channels:] if first_raw < groups else None
        kernels.short_conv(dev(rows, DT[dtype]), dev(w), None, state, ints(slots), ints(starts), ints(token_seq),
                           both[:, :channels], n_tokens=total, n_seqs=3, norm_group=group, eps=eps, raw_out=raw,
                           raw_first_group=first_raw)
        got = both.double().cpu().numpy()
        for r, (lo, hi) in enumerate(zip(starts[:-1], starts[1:])):
            history[r] = np.concatenate([history[r], rows[lo:hi]])
            conv = plain.causal_conv(history[r], w.astype(np.float32).astype(np.float64))[-(hi - lo):]
            want = plain.rms_unit(conv.reshape(hi - lo, groups, group), eps).reshape(hi - lo, channels)
            close(got[lo:hi, :channels], want, TOL[dtype])
            if raw is not None:
                close(got[lo:hi, channels:], conv[:, first_raw * group:], TOL[dtype])


def plain_talking(q, k, v, gate, temp, talk, scale, cap, window, out_scale, past=0):
    """q [n, H, D] at positions past .. past + n - 1; k, v [past + n, G, D].  float64."""
    n, H, D = q.shape
    G = k.shape[1]
    i, j = (past + np.arange(n))[:, None], np.arange(past + n)[None, :]
    raw = np.zeros((H, n, past + n))
    for a in range(H):
        s = (q[:, a] @ k[:, a // (H // G)].T) * scale * (1.0 if temp is None else temp[a])
        if cap > 0:
            s = cap * np.tanh(s / cap)
        raw[a] = s - 2.0 ** (-8.0 * (a + 1) / H) * (i - j)
    mixed = raw if talk is None else np.einsum("hg,gij->hij", talk, raw)
    seen = (j <= i) & ((i - j < window) if window else True)
    mixed = np.where(seen[None], mixed, -np.inf)
    p = np.exp(mixed - mixed.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    out = np.stack([p[a] @ v[:, a // (H // G)] for a in range(H)], axis=1)
    if gate is not None:
        out = out * plain.sigmoid(gate.reshape(n, H, D))
    return out.reshape(n, H * D) * out_scale


def slopes(H):
    return dev(np.array([2.0 ** (-8.0 * (a + 1) / H) for a in range(H)]))


KINDS = [("float32", False), ("bfloat16", False), ("bfloat16", True)]      # (type of the rows, the plain kernel only)


@pytest.mark.parametrize("dtype, plain_kernel", KINDS)
@pytest.mark.parametrize("H, G, D, window", [(6, 2, 24, 40), (4, 4, 32, 0), (1, 1, 14, 5), (5, 1, 12, 33), (2, 1, 128, 70),
                                             (3, 3, 72, 1), (8, 2, 64, 72), (2, 2, 200, 64), (12, 4, 48, 31), (20, 5, 16, 97)])
def test_talking_attention_over_the_steps_own_rows(dtype, plain_kernel, H, G, D, window):
    rng = np.random.default_rng(H * D + window)
    lengths = [75, 1, 130, 6]
    starts, _ = step_tables(lengths)
    total = starts[-1]
    width = (H + 2 * G) * D
    rows = rounded(rng.standard_normal((total, width)), dtype)
    gate = rounded(rng.standard_normal((total, H * D)), dtype)
    temp, talk = rng.standard_normal(H) + 1.5, rng.standard_normal((H, H)) * 0.5 + np.eye(H)
    t_rows = dev(rows, DT[dtype])
    out = torch.zeros((total, H * D), dtype=DT[dtype], device=DEV)
    scale, cap = 0.3 * D ** -0.5 * 4, 6.0
    kernels.talking_attention(t_rows[:, :H * D], out, ints(starts), ints([0] * 4), n_seqs=4, max_new=max(lengths), n_heads=H,
                              n_kv_heads=G, head_dim=D, scale=scale, window=window, cap=cap, temp=dev(temp), slope=slopes(H),
                              talk=dev(talk), gate=dev(gate, DT[dtype]), out_scale=0.7, k=t_rows[:, H * D:(H + G) * D],
                              v=t_rows[:, (H + G) * D:], plain=plain_kernel)
    got = out.double().cpu().numpy()
    t32 = lambda a: a.astype(np.float32).astype(np.float64)
    for lo, hi in zip(starts[:-1], starts[1:]):
        q = rows[lo:hi, :H * D].reshape(-1, H, D)
        k = rows[lo:hi, H * D:(H + G) * D].reshape(-1, G, D)
        v = rows[lo:hi, (H + G) * D:].reshape(-1, G, D)
        want = plain_talking(q, k, v, gate[lo:hi], t32(temp), t32(talk), scale, cap, window, 0.7)
        close(got[lo:hi], want, TOL[dtype])


@pytest.mark.parametrize("dtype, plain_kernel", KINDS)
@pytest.mark.parametrize("new", [1, 9, 40])
@pytest.mark.parametrize("H, G, D, window", [(6, 2, 24, 40), (4, 4, 32, 0), (3, 1, 16, 100), (2, 2, 72, 64), (8, 2, 64, 72),
                                             (10, 5, 40, 130)])
def test_talking_attention_over_scattered_pages(dtype, plain_kernel, new, H, G, D, window):
    """Sequences that already hold tokens: keys and values lie in pages in no order; a window's pages are a ring that
    has come round."""
    rng = np.random.default_rng(H + D + window + new)
    pasts = [0, 63, 64, 200, 131]
    n_seqs = len(pasts)
    ring = -(-window // 64) + (1 if window and new > 1 else 0) if window else 0
    table_len = ring if window else 5
    if window and new > table_len * 64 - window + 1:
        pytest.skip("a ring keeps one window and one run of new tokens")
    n_pages = n_seqs * table_len + 3
    k_pool = torch.zeros((n_pages, G, 64, D), dtype=DT[dtype], device=DEV)
    v_pool = torch.zeros_like(k_pool)
    pages = rng.permutation(n_pages)[:n_seqs * table_len].reshape(n_seqs, table_len)
    lengths = [new] * n_seqs
    starts, _ = step_tables(lengths)
    total = starts[-1]
    keys = [rounded(rng.standard_normal((p + new, G, D)), dtype) for p in pasts]
    values = [rounded(rng.standard_normal((p + new, G, D)), dtype) for p in pasts]
    kp, vp = k_pool.cpu(), v_pool.cpu()
    for s in range(n_seqs):
        for pos in range(pasts[s] + new):      # in order: a ring keeps the newest
            page = pages[s, (pos // 64) % table_len]
            kp[page, :, pos % 64] = torch.from_numpy(keys[s][pos]).to(DT[dtype])
            vp[page, :, pos % 64] = torch.from_numpy(values[s][pos]).to(DT[dtype])
    k_pool.copy_(kp)
    v_pool.copy_(vp)
    q = rounded(rng.standard_normal((total, H * D)), dtype)
    temp, talk = rng.standard_normal(H) + 1.5, rng.standard_normal((H, H)) * 0.5 + np.eye(H)
    out = torch.zeros((total, H * D), dtype=DT[dtype], device=DEV)
    scale, cap = 1.2 * D ** -0.5, 9.0
    t32 = lambda a: a.astype(np.float32).astype(np.float64)
    wants = [plain_talking(q[lo:hi].reshape(-1, H, D), keys[s], values[s], None, t32(temp), t32(talk), scale, cap, window, 1.0,
                           past=pasts[s]) for s, (lo, hi) in enumerate(zip(starts[:-1], starts[1:]))]
    # alone, and with every sequence's keys shared among 2, 3 or more blocks than the shortest has tiles
    for n_split in (1, 2, 3, 7) if dtype == "bfloat16" and not plain_kernel and new <= kernels.TALK_SPLIT_ROWS else (1,):
        shared = {}
        if n_split > 1:
            shared = dict(n_split=n_split,
                          parts=torch.full((n_seqs * n_split * H * new * (D + 2),), float("nan"), device=DEV))
        out.zero_()
        kernels.talking_attention(dev(q, DT[dtype]), out, ints(starts), ints(pasts), n_seqs=n_seqs, max_new=new, n_heads=H,
                                  n_kv_heads=G, head_dim=D, scale=scale, window=window, cap=cap, temp=dev(temp),
                                  slope=slopes(H), talk=dev(talk), k_pool=k_pool, v_pool=v_pool, table=ints(pages),
                                  table_len=table_len, plain=plain_kernel, **shared)
        got = out.double().cpu().numpy()
        for s, (lo, hi) in enumerate(zip(starts[:-1], starts[1:])):
            close(got[lo:hi], wants[s], TOL[dtype], f"{n_split} blocks, sequence {s}: ")


def test_how_a_steps_keys_are_shared_among_blocks():
    assert kernels.talking_attention_split(8, 17, 4, 32, 0, 4000) == (1, 0)
    assert kernels.talking_attention_split(1000, 1, 4, 32, 0, 4000) == (1, 0)
    n_split, need = kernels.talking_attention_split(8, 1, 4, 32, 100, 4000)
    assert n_split == 5 and need == 8 * 5 * 4 * 1 * 34          # a window of 100 keys: 4 tiles, or 5 where it straddles
    n_split, need = kernels.talking_attention_split(3, 2, 6, 24, 0, 100000)
    assert n_split == 99 and need == 3 * 99 * 6 * 2 * 26


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("distance, seen", [(0, True), (1, True), (63, True), (64, True), (70, True), (71, False), (300, False)])
def test_one_loud_key_at_and_past_the_windows_edge(dtype, distance, seen):
    """A window of 71: one key that every head's query prefers by far carries the row if it is at most 70 positions
    back, and is gone at 71; the values tell."""
    H, G, D, window, n = 4, 2, 16, 71, 400
    rng = np.random.default_rng(distance)
    q = rng.standard_normal((n, H, D)) * 0.1
    k = rng.standard_normal((n, G, D)) * 0.1
    v = rng.standard_normal((n, G, D))
    at = n - 1 - distance
    q[-1] = 1.0
    k[at] = 3.0
    v[at] = 50.0
    q, k, v = rounded(q, dtype), rounded(k, dtype), rounded(v, dtype)
    rows = np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], axis=1)
    t_rows = dev(rows, DT[dtype])
    out = torch.zeros((n, H * D), dtype=DT[dtype], device=DEV)
    kernels.talking_attention(t_rows[:, :H * D], out, ints([0, n]), ints([0]), n_seqs=1, max_new=n, n_heads=H, n_kv_heads=G,
                              head_dim=D, scale=1.0, window=window, cap=200.0, slope=slopes(H), k=t_rows[:, H * D:(H + G) * D],
                              v=t_rows[:, (H + G) * D:])
    last = out[-1].double().cpu().numpy()
    assert (np.abs(last - 50.0).max() < (1e-2 if dtype == "float32" else 0.3)) if seen else (np.abs(last).max() < 10.0)
    want = plain_talking(q, k, v, None, None, None, 1.0, 200.0, window, 1.0)
    close(out.double().cpu().numpy(), want, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inner, n_state, rank", [(80, 12, 5), (36, 5, 3), (30, 1, 2), (24, 70, 4), (16, 130, 6), (256, 32, 16),
                                                  (20, 300, 160), (6, 512, 3), (64, 16, 4), (40, 64, 8)])
def test_selective_scan_carries_its_state(dtype, inner, n_state, rank):
    rng = np.random.default_rng(inner + n_state)
    slots = [3, 0, 4]
    state = torch.zeros((5, inner, n_state), device=DEV)
    w_dt, b_dt = rng.standard_normal((inner, rank)) * rank ** -0.5, rng.standard_normal(inner) - 1.0
    a_log, d_skip = rng.standard_normal((inner, n_state)) * 0.5, rng.standard_normal(inner)
    t32 = lambda a: a.astype(np.float32).astype(np.float64)
    S = [np.zeros((inner, n_state)) for _ in slots]
    pad = 2
    for lengths in ([40, 1, 17], [1, 1, 1], [2, 33, 16]):
        starts, _ = step_tables(lengths)
        total = starts[-1]
        xz = rounded(rng.standard_normal((total, 2 * inner)), dtype)
        low = rounded(rng.standard_normal((total, pad + rank + 2 * n_state)), dtype)
        t_xz, t_low = dev(xz, DT[dtype]), dev(low, DT[dtype])
        dt = torch.zeros((total, inner), device=DEV)
        kernels.selective_scan_dt(t_low[:, pad:], dev(w_dt), dev(b_dt), dt, n_tokens=total)
        want_dt = plain.softplus(low[:, pad:pad + rank] @ t32(w_dt).T + t32(b_dt))
        close(dt.double().cpu().numpy(), want_dt, 2e-5)
        out = torch.zeros((total, inner), dtype=DT[dtype], device=DEV)
        kernels.selective_scan(t_xz[:, :inner], t_xz[:, inner:], dt, t_low, pad + rank, pad + rank + n_state, dev(a_log),
                               dev(d_skip), state, ints(slots), ints(starts), out, n_seqs=3, out_scale=1.3)
        got = out.double().cpu().numpy()
        dt64 = dt.double().cpu().numpy()
        A = -np.exp(t32(a_log))
        for r, (lo, hi) in enumerate(zip(starts[:-1], starts[1:])):
            for t in range(lo, hi):
                x, z = xz[t, :inner], xz[t, inner:]
                B, C = low[t, pad + rank:pad + rank + n_state], low[t, pad + rank + n_state:]
                S[r] = np.exp(dt64[t][:, None] * A) * S[r] + (dt64[t] * x)[:, None] * B[None, :]
                want = (S[r] @ C + t32(d_skip) * x) * plain.silu(z) * 1.3
                close(got[t], want, TOL[dtype], f"sequence {r}, token {t - lo}: ")
    for r, slot in enumerate(slots):
        close(state[slot].double().cpu().numpy(), S[r], 2e-5)
    assert float(state[1].abs().sum()) == 0 and float(state[2].abs().sum()) == 0


@pytest.mark.parametrize("inner, n_state, rank", [(40, 12, 5), (24, 70, 4), (130, 16, 8)])
@pytest.mark.parametrize("lengths", [[200, 1, 70, 65], [64, 129, 2, 1000], [4200, 3, 128, 127]])
def test_selective_scan_in_pieces_side_by_side(inner, n_state, rank, lengths):
    """Long runs are cut into pieces that run side by side and are joined through each piece's end state; the result
    and the stored state equal those of one walk over the run, from a state that is not zero."""
    rng = np.random.default_rng(inner + n_state + lengths[0])
    n_seqs = len(lengths)
    slots = [int(v) for v in rng.permutation(n_seqs + 2)[:n_seqs]]
    first = rng.standard_normal((n_seqs + 2, inner, n_state))
    w_dt, b_dt = rng.standard_normal((inner, rank)) * rank ** -0.5, rng.standard_normal(inner) - 3.0
    a_log, d_skip = rng.standard_normal((inner, n_state)) * 0.5 - 1.0, rng.standard_normal(inner)
    starts, _ = step_tables(lengths)
    total = starts[-1]
    xz = rng.standard_normal((total, 2 * inner))
    low = rng.standard_normal((total, rank + 2 * n_state))
    t_xz, t_low = dev(xz), dev(low)
    dt = torch.zeros((total, inner), device=DEV)
    kernels.selective_scan_dt(t_low, dev(w_dt), dev(b_dt), dt, n_tokens=total)
    results = []
    for pieces in (False, True):
        state = dev(first)
        out = torch.zeros((total, inner), device=DEV)
        extra = {}
        if pieces:
            piece, most, need = kernels.selective_scan_pieces(max(lengths), total, n_seqs, inner, n_state)
            assert piece > 0 and need > 0 and most * piece >= max(lengths)
            extra = dict(max_new=max(lengths), scratch=torch.full((need,), float("nan"), device=DEV))
        kernels.selective_scan(t_xz[:, :inner], t_xz[:, inner:], dt, t_low, rank, rank + n_state, dev(a_log), dev(d_skip),
                               state, ints(slots), ints(starts), out, n_seqs=n_seqs, **extra)
        results.append((out.double().cpu().numpy(), state.double().cpu().numpy()))
    close(results[1][0], results[0][0], 2e-5)
    close(results[1][1], results[0][1], 2e-5)
    # the pieces against the plain recurrence, on the second longest run
    r = int(np.argsort(lengths)[-2])
    lo, hi = starts[r], starts[r + 1]
    t32 = lambda a: a.astype(np.float32).astype(np.float64)
    S, A, dt64 = t32(first[slots[r]]), -np.exp(t32(a_log)), dt.double().cpu().numpy()
    for t in range(lo, hi):
        x, z = t32(xz[t, :inner]), t32(xz[t, inner:])
        B, C = t32(low[t, rank:rank + n_state]), t32(low[t, rank + n_state:])
        S = np.exp(dt64[t][:, None] * A) * S + (dt64[t] * x)[:, None] * B[None, :]
        close(results[1][0][t], (S @ C + t32(d_skip) * x) * plain.silu(z), 5e-5, f"token {t - lo}: ")
    close(results[1][1][slots[r]], S, 5e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("vecs, length, dims, tail", [(6, 16, 8, 20), (2, 40, 40, 0), (3, 6, 2, 5), (1, 10, 0, 3), (2, 130, 64, 7)])
def test_half_split_rotation(dtype, vecs, length, dims, tail):
    rng = np.random.default_rng(vecs * length + dims)
    n, base = 50, 777.0
    positions = rng.integers(0, 1500, n)
    rows = rounded(rng.standard_normal((n, vecs * length + tail + 3)), dtype)
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(max(1, dims // 2))] if dims else [1.0],
                        dtype=torch.float64).to(torch.float32).to(DEV)
    out = torch.full((n + 1, vecs * length + tail + 1), 7.0, device=DEV)
    first_scaled = vecs // 2
    kernels.rotary_half(dev(rows, DT[dtype]), out, ints(positions), freq, n_tokens=n, n_vecs=vecs, length=length, dims=dims,
                        scaled_from=first_scaled, scale=0.25, tail=tail)
    got = out.double().cpu().numpy()
    assert np.all(got[n:] == 7.0) and np.all(got[:, vecs * length + tail:] == 7.0)
    want = plain.rotate_half(rows[:, :vecs * length].reshape(n, vecs, length), positions, dims, base) if dims else \
        rows[:, :vecs * length].reshape(n, vecs, length).copy()
    want[:, first_scaled:] *= 0.25
    close(got[:n, :vecs * length], want.reshape(n, -1), 2e-4)        # (32-bit angles of up to 1500 radians)
    np.testing.assert_array_equal(got[:n, vecs * length:vecs * length + tail], rows[:, vecs * length:vecs * length + tail])


@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("heads, dim, vdim", [(3, 16, 24), (2, 40, 20), (1, 130, 20)])
def test_recurrence_over_prepared_vectors(heads, dim, vdim, chunked):
    """The decayed state fed with 32-bit vectors as they are (no activation): what the retention asks of it."""
    rng = np.random.default_rng(dim)
    lengths, slots = ([150, 70, 65] if chunked else [30, 1, 17]), [2, 0, 1]
    starts, _ = step_tables(lengths)
    total = starts[-1]
    decay = np.array([0.9, 0.995, 1.0][:heads])
    rows = rng.standard_normal((total, 2 * heads * dim + heads * vdim)).astype(np.float32).astype(np.float64)
    state = torch.zeros((3, heads, dim, vdim), device=DEV)
    state[0] = 0.5
    out = torch.zeros((total, heads * vdim), device=DEV)
    scratch = None
    if chunked:
        scratch = torch.zeros((kernels.lightning_chunked_scratch_floats(3, max(lengths), heads, dim, vdim),), device=DEV)
    kernels.lightning_scan(dev(rows), 0, heads * dim, 2 * heads * dim, state, ints(slots), ints(starts), dev(decay), out,
                           n_seqs=3, n_heads=heads, dim=dim, vdim=vdim, max_new=max(lengths), scratch=scratch, activation=None)
    got = out.double().cpu().numpy()
    for r, (lo, hi) in enumerate(zip(starts[:-1], starts[1:])):
        for a in range(heads):
            S = np.full((dim, vdim), 0.5 if slots[r] == 0 else 0.0)
            for t in range(lo, hi):
                q = rows[t, a * dim:(a + 1) * dim]
                k = rows[t, (heads + a) * dim:(heads + a + 1) * dim]
                v = rows[t, 2 * heads * dim + a * vdim:2 * heads * dim + (a + 1) * vdim]
                S = decay[a] * S + np.outer(k, v)
                close(got[t, a * vdim:(a + 1) * vdim], S.T @ q, 1e-4)
            close(state[slots[r], a].double().cpu().numpy(), S, 1e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [30, 88, 320, 1000, 2500])
def test_polynomial_activation(dtype, width):
    rng = np.random.default_rng(width)
    z = rounded(rng.standard_normal((13, width)) * 1.5, dtype)
    coef = np.array([0.7, -0.4, 0.25, 0.1])
    out = torch.zeros((14, width), dtype=DT[dtype], device=DEV)
    kernels.polynorm(dev(z, DT[dtype]), dev(coef), out, 1e-5, n_rows=13)
    c = coef.astype(np.float32).astype(np.float64)
    want = c[0] * plain.rms_unit(z, 1e-5) + c[1] * plain.rms_unit(z ** 2, 1e-5) + c[2] * plain.rms_unit(z ** 3, 1e-5) + c[3]
    close(out[:13].double().cpu().numpy(), want, TOL[dtype])
    assert float(out[13].abs().sum()) == 0


@pytest.mark.parametrize("next_dtype", [None, "float32", "bfloat16"])
@pytest.mark.parametrize("width", [52, 96, 768, 2000])
def test_norm_that_adds_a_sublayers_result_to_the_stream(width, next_dtype):
    rng = np.random.default_rng(width)
    x, stream = rng.standard_normal((9, width)) * 3, rng.standard_normal((10, width))
    w, w2 = rng.standard_normal(width) * 0.2 + 1.0, rng.standard_normal(width) * 0.2 + 1.0
    t_stream = dev(stream)
    nxt = None if next_dtype is None else torch.zeros((9, width), dtype=DT[next_dtype], device=DEV)
    kernels.rmsnorm_add(dev(x), dev(w), t_stream, 1e-5, n_rows=9, next_weight=None if nxt is None else dev(w2), next_out=nxt)
    t32 = lambda a: a.astype(np.float32).astype(np.float64)
    want = t32(stream[:9]) + plain.rms_unit(t32(x), 1e-5) * t32(w)
    close(t_stream[:9].double().cpu().numpy(), want, 2e-6)
    np.testing.assert_array_equal(t_stream[9].cpu().numpy(), stream[9].astype(np.float32))
    if nxt is not None:
        close(nxt.double().cpu().numpy(), plain.rms_unit(want, 1e-5) * t32(w2), TOL[next_dtype] if next_dtype == "bfloat16" else 2e-6)
