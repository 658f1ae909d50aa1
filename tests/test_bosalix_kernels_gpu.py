"""The kernels Bosalix brought, each alone against the plain implementation's function for the same mechanism (float64),
at sizes the models of the other tests do not have: the token shift with its kept row, the preparation and the sum of the
sigmoid attention with windows and kept positions at page borders, the latent attention's window in both of its
kernels and in the kernel for fresh prompts, the softmax router with its correction, experts without a gate and experts
without tensors, and the norm that is added with a factor."""
import math

import numpy as np
import pytest
import torch

import plain_bosalix as plain
from burn_transformers_b200 import kernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)]
PAGE = 64


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=torch.float64).to(dtype).to(DEV)


def ints(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def host(t):
    return t.detach().double().cpu()


def rel(got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return float(np.abs(got - want).max() / max(1e-30, np.abs(want).max()))


def step_layout(pasts, news, table_width):
    """The integers of a step of several sequences whose pages are handed out in a scrambled order."""
    n_seqs = len(news)
    seq_start = np.concatenate([[0], np.cumsum(news)])
    positions = np.concatenate([np.arange(p, p + n) for p, n in zip(pasts, news)])
    token_seq = np.concatenate([np.full(n, s) for s, n in enumerate(news)])
    pages = np.random.default_rng(7).permutation(n_seqs * table_width).reshape(n_seqs, table_width)
    return (ints(seq_start), ints(positions), ints(token_seq), ints(pasts), ints(pages), int(pages.max()) + 1)


@pytest.mark.parametrize("out_dtype, tol", DTYPES)
def test_token_shift_keeps_the_last_row_of_every_sequence(out_dtype, tol):
    rng = np.random.default_rng(0)
    width, news, slots = 70, [5, 1, 2, 9], [3, 0, 6, 1]
    n = sum(news)
    x = dev(rng.standard_normal((n, width)))
    shift = dev(rng.standard_normal(width))
    state = dev(rng.standard_normal((8, width)))
    before = host(state).clone()
    seq_start, _, token_seq, _, _, _ = step_layout([0] * 4, news, 1)
    out = torch.full((n + 2, width), 9.0, dtype=out_dtype, device=DEV)
    kernels.token_shift(x, shift, state, ints(slots), seq_start, token_seq, out, n_rows=n)
    at = 0
    for s, count in enumerate(news):
        want, last = plain.token_shift(host(x[at:at + count]), host(shift), before=before[slots[s]])
        assert rel(host(out[at:at + count]), want) < tol
        assert torch.equal(host(state[slots[s]]), last)
        at += count
    assert bool((out[n:] == 9.0).all())
    untouched = [i for i in range(8) if i not in slots]
    assert torch.equal(host(state[untouched]), before[untouched])


def sigmoid_case(rng, heads, groups, dim, vdim, rot_dims, news, pasts, dtype, mixing):
    """Random projections of whole sequences (past and new tokens), filed and prepared step by step as the engine would:
    first the past tokens as one step, then the new ones."""
    lens = [p + n for p, n in zip(pasts, news)]
    width = (heads + groups) * dim + groups * vdim
    proj = [rng.standard_normal((length, width)) * 1.5 for length in lens]
    other = [rng.standard_normal((length, groups * vdim)) for length in lens] if mixing else None
    qw, kw = 1.0 + 0.3 * rng.standard_normal(dim), 1.0 + 0.3 * rng.standard_normal(dim)
    table_width = -(-max(lens) // PAGE)
    freqs = plain.stretched_frequencies(rot_dims, 300.0, {"factor": 3.0, "low": 1.0, "high": 8.0, "original": 40})
    inv_freq = dev(freqs or [1.0])
    lam = 0.3
    pool = None
    outs = {}
    for phase, (lo_of, count_of) in enumerate(((lambda s: 0, lambda s: pasts[s]), (lambda s: pasts[s], lambda s: news[s]))):
        seqs = [s for s in range(len(lens)) if count_of(s) > 0]
        if not seqs:
            continue
        counts = [count_of(s) for s in seqs]
        seq_start, positions, token_seq, past, pages, n_pages = step_layout([lo_of(s) for s in seqs], counts, table_width)
        # (every sequence keeps its pages from one phase to the next: the same scrambled table, its rows picked by sequence)
        _, _, _, _, all_pages, n_pages = step_layout([0] * len(lens), [1] * len(lens), table_width)
        pages = all_pages[torch.tensor(seqs, device=DEV)].contiguous()
        if pool is None:
            pool = torch.zeros((n_pages, groups, PAGE, dim + vdim), dtype=dtype, device=DEV)
        rows = dev(np.concatenate([proj[s][lo_of(s):lo_of(s) + count_of(s)] for s in seqs]), dtype)
        n = rows.shape[0]
        v_other = dev(np.concatenate([other[s][lo_of(s):lo_of(s) + count_of(s)] for s in seqs])) if mixing else None
        publish = torch.zeros((n, groups * vdim), dtype=torch.float32, device=DEV)
        kernels.sigmoid_attention_prep(rows, dev(qw), dev(kw), 1e-5, positions, token_seq, inv_freq, rot_dims, pages,
                                       table_width, pool, n_tokens=n, n_heads=heads, n_kv_heads=groups, dim=dim, vdim=vdim,
                                       mix=dev([lam]) if mixing else None, v_other=v_other, v_publish=publish)
        outs[phase] = (seqs, counts, rows, seq_start, past, pages, publish)
    return proj, other, qw, kw, freqs, lam, pool, table_width, outs


@pytest.mark.parametrize("dtype, tol", DTYPES)
@pytest.mark.parametrize("heads, groups, dim, vdim, rot_dims, window, keep, mixing", [
    (6, 2, 24, 16, 16, 40, 5, True),          # a window and kept positions inside one page
    (5, 1, 12, 10, 6, 70, 66, False),         # sizes that are no 16-byte pieces; kept positions past a page's border
    (16, 1, 128, 96, 48, 64, 0, True),        # a window of exactly one page, sixteen heads a key head
    (40, 1, 16, 8, 0, 3, 1, False),           # more heads a key head than a block's rows; no rotation
    (2, 2, 72, 130, 72, 0, 0, False),         # no window at all; wide values
    (3, 3, 8, 40, 8, 1, 200, True),           # a window of one token, more kept positions than any sequence is long
    (8, 2, 64, 64, 32, 100, 7, True),         # keys and values of one size the tcgen05 kernel takes; kept tiles before the window
    (4, 1, 128, 128, 128, 0, 0, False),       # the same at 128 channels, no window
    (6, 3, 64, 64, 64, 130, 129, False),      # kept positions that fill a tile of 128 and one more
    (6, 2, 128, 64, 32, 90, 3, True),         # the tcgen05 kernel with values half as wide as the keys
    (4, 4, 64, 128, 64, 200, 0, False),       # and twice as wide
])
def test_sigmoid_attention_in_prompts_and_in_single_tokens(dtype, tol, heads, groups, dim, vdim, rot_dims, window, keep,
                                                           mixing):
    """Fresh prompts, portions that continue a sequence, and single tokens, in one batch of unequal sequences, against
    the plain implementation's weights sigmoid(q . k * scale + bias) over exactly the positions it calls visible."""
    rng = np.random.default_rng(1)
    scale = 0.7 / math.sqrt(dim)
    bias = rng.standard_normal(heads)
    for pasts, news in (([0, 0, 0], [130, 1, 65]), ([64, 63, 129, 1], [1, 1, 1, 1]), ([30, 128], [70, 3]), ([0, 0], [700, 300]), ([200, 0, 5], [300, 130, 64])):
        proj, other, qw, kw, freqs, lam, pool, table_width, outs = sigmoid_case(rng, heads, groups, dim, vdim, rot_dims, news,
                                                                              pasts, dtype, mixing)
        seqs, counts, rows, seq_start, past, pages, publish = outs[1]
        n = rows.shape[0]
        out = torch.full((n + 1, heads * vdim), 9.0, dtype=dtype, device=DEV)
        kernels.sigmoid_attention(rows, out, pool, pages, table_width, seq_start, past, n_seqs=len(seqs), max_new=max(counts),
                                  n_heads=heads, n_kv_heads=groups, dim=dim, vdim=vdim, scale=scale, bias=dev(bias),
                                  window=window, keep_first=keep)
        assert bool((out[n:] == 9.0).all())
        at = 0
        for s, count in zip(seqs, counts):
            length = pasts[s] + news[s]
            p = torch.tensor(proj[s], dtype=torch.float64)
            if dtype == torch.bfloat16:
                p = p.to(torch.bfloat16).double()
            positions = torch.arange(length)
            q = plain.rotate_pairs(plain.norm_plain(p[:, :heads * dim].view(length, heads, dim), torch.tensor(qw), 1e-5),
                                   positions, freqs, "half")
            k = plain.rotate_pairs(plain.norm_plain(p[:, heads * dim:(heads + groups) * dim].view(length, groups, dim),
                                                    torch.tensor(kw), 1e-5), positions, freqs, "half")
            v = plain.rms_divide(p[:, (heads + groups) * dim:].view(length, groups, vdim), 1e-5)
            if mixing:
                v = (1.0 - lam) * v + lam * torch.tensor(other[s]).view(length, groups, vdim)
            np.testing.assert_allclose(host(publish[at:at + count]), v[pasts[s]:].reshape(count, -1), atol=tol, rtol=tol)
            seen = plain.visibility(length, window or None, keep)
            want = torch.zeros(length, heads, vdim, dtype=torch.float64)
            for h in range(heads):
                g = h // (heads // groups)
                want[:, h] = (torch.sigmoid(q[:, h] @ k[:, g].T * scale + bias[h]) * seen) @ v[:, g]
            want = want[pasts[s]:].reshape(count, -1)
            assert rel(host(out[at:at + count]), want) < tol, (pasts, news, s)
            at += count
        if dtype == torch.bfloat16 and any(pasts) and kernels.sigmoid_attention_tcgen05_supports(dim, vdim, rows.shape[1]):
            # portions that continue a sequence (and single tokens) through the tcgen05 kernel over the pages
            fast = torch.full((n + 1, heads * vdim), 9.0, dtype=dtype, device=DEV)
            kernels.sigmoid_attention_tcgen05(rows, fast, seq_start, past, n_seqs=len(seqs), max_new=max(counts),
                                              n_heads=heads, n_kv_heads=groups, head_dim=dim, v_dim=vdim, scale=scale,
                                              bias=dev(bias), window=window, keep_first=keep, pool=pool, table=pages,
                                              table_len=table_width)
            kernels.check_status(torch.device(DEV))
            assert rel(host(fast[:n]), host(out[:n])) < tol and bool((fast[n:] == 9.0).all())
        if dtype == torch.bfloat16 and not any(pasts):
            # the same prompts through the tensor-core kernel that reads keys and values from the step's own rows
            q = rows[:, :heads * dim].view(n, heads, dim)
            k = rows[:, heads * dim:(heads + groups) * dim].view(n, groups, dim)
            v = rows[:, (heads + groups) * dim:].view(n, groups, vdim)
            fast = torch.full((n + 1, heads, vdim), 9.0, dtype=dtype, device=DEV)
            if kernels.sigmoid_attention_tcgen05_supports(dim, vdim, rows.shape[1]):
                # keys and values of 64 or 128 channels a head each: tcgen05, the scores in tensor memory
                kernels.sigmoid_attention_tcgen05(rows, fast.view(n + 1, -1), seq_start, past, n_seqs=len(seqs),
                                                  max_new=max(counts), n_heads=heads, n_kv_heads=groups, head_dim=dim,
                                                  v_dim=vdim, scale=scale, bias=dev(bias), window=window, keep_first=keep)
                kernels.check_status(torch.device(DEV))
                assert rel(host(fast[:n]).reshape(n, -1), host(out[:n])) < tol and bool((fast[n:] == 9.0).all())
                fast.fill_(9.0)
            takes = kernels.sigmoid_attention_prompt_supports(q, k, v, fast[:n])
            assert takes == (dim % 8 == 0 and vdim % 8 == 0 and vdim <= 128)
            if takes:
                kernels.sigmoid_attention_prompt(q, k, v, fast[:n], seq_start, n_seqs=len(seqs), max_new=max(counts),
                                                 scale=scale, bias=dev(bias), window=window, keep_first=keep)
                assert rel(host(fast[:n]).reshape(n, -1), host(out[:n])) < tol and bool((fast[n:] == 9.0).all())


def latent_reference(q, rows, rank, scale, window, past):
    """q [new, heads, rank + rot], rows [length, rank + rot]: softmax over the visible rows, weighted sum of their latents."""
    length, new = rows.shape[0], q.shape[0]
    seen = plain.visibility(length, window or None, 0)[past:]
    scores = torch.einsum("thd,jd->thj", q, rows) * scale
    p = torch.softmax(scores.masked_fill(~seen[:, None, :], -math.inf), -1)
    return torch.einsum("thj,jc->thc", p, rows[:, :rank])


@pytest.mark.parametrize("dtype, tol", DTYPES)
@pytest.mark.parametrize("tensor_cores", [False, True])
@pytest.mark.parametrize("heads, rank, rot, window, splits", [(3, 48, 8, 33, 1), (6, 160, 16, 50, 1), (4, 32, 8, 64, 3),
                                                              (2, 40, 0, 1, 1), (5, 64, 32, 200, 4)])
def test_latent_attention_sees_its_window_only(dtype, tol, tensor_cores, heads, rank, rot, window, splits):
    """The window in the multiply-add kernel and in the tensor-core kernel, with the keys cut into runs and not, for
    portions that continue a sequence and for single tokens, the first visible key at and beside a page's border."""
    rng = np.random.default_rng(2)
    dk = rank + rot
    scale = 2.0 / math.sqrt(dk)
    for pasts, news in (([0, 0], [150, 2]), ([64 + window - 1, 63, 300], [1, 1, 1]), ([100, 7], [70, 40])):
        lens = [p + n for p, n in zip(pasts, news)]
        table_width = -(-max(lens) // PAGE)
        seq_start, _, _, past, pages, n_pages = step_layout(pasts, news, table_width)
        pool = torch.zeros((n_pages, PAGE, dk), dtype=dtype, device=DEV)
        stored = []
        for s, length in enumerate(lens):
            rows = dev(rng.standard_normal((length, dk)), dtype)
            stored.append(host(rows))
            for j in range(length):
                pool[int(pages[s, j // PAGE]), j % PAGE] = rows[j]
        n = sum(news)
        q = dev(rng.standard_normal((n, heads * dk)), dtype)
        out = torch.full((n + 1, heads * rank), 9.0, dtype=dtype, device=DEV)
        scratch = None
        if splits > 1:
            scratch = torch.zeros(kernels.latent_attention_scratch_floats(n, heads, rank, splits), dtype=torch.float32,
                                  device=DEV)
        kernels.latent_attention(q, out, pool, pages, table_width, seq_start, past, n_tokens=n, n_seqs=len(news),
                                 max_new=max(news), n_heads=heads, rank=rank, rot=rot, scale=scale, n_splits=splits,
                                 scratch=scratch, tensor_cores=tensor_cores, window=window)
        assert bool((out[n:] == 9.0).all())
        at = 0
        for s, count in enumerate(news):
            want = latent_reference(host(q[at:at + count]).view(count, heads, dk), stored[s], rank, scale, window, pasts[s])
            assert rel(host(out[at:at + count]).view(count, heads, rank), want) < tol, (pasts, news, s)
            at += count


@pytest.mark.parametrize("window", [0, 1, 50, 64, 100])
def test_attention_of_fresh_prompts_sees_its_window_only(window):
    """The tensor-core kernel for prompts that start a sequence (bfloat16), with key tiles before the window skipped."""
    rng = np.random.default_rng(3)
    heads, dq, dv, news = 3, 40, 24, [200, 1, 70]
    n = sum(news)
    q, k, v = (dev(rng.standard_normal((n, heads, d)), torch.bfloat16) for d in (dq, dq, dv))
    out = torch.zeros((n, heads, dv), dtype=torch.bfloat16, device=DEV)
    if not kernels.sink_attention_supports(q, k, v, None, out):
        pytest.skip("the kernel does not take these views")
    seq_start = ints(np.concatenate([[0], np.cumsum(news)]))
    scale = 1.5 / math.sqrt(dq)
    kernels.sink_attention(q, k, v, out, seq_start, n_seqs=len(news), max_new=max(news), scale=scale, window=window)
    at = 0
    for count in news:
        seen = plain.visibility(count, window or None, 0)
        scores = torch.einsum("thd,jhd->htj", host(q[at:at + count]), host(k[at:at + count])) * scale
        p = torch.softmax(scores.masked_fill(~seen[None], -math.inf), -1)
        want = torch.einsum("htj,jhc->thc", p, host(v[at:at + count]))
        assert rel(host(out[at:at + count]), want) < 3e-2
        at += count


@pytest.mark.parametrize("dtype, tol", DTYPES)
@pytest.mark.parametrize("n, width, stored, identity, top, inner", [(70, 96, 6, 2, 2, 40), (5, 72, 1, 2, 1, 20),
                                                                    (300, 64, 7, 5, 4, 12), (33, 80, 8, 0, 3, 96)])
def test_softmax_router_and_experts_without_a_gate(dtype, tol, n, width, stored, identity, top, inner):
    """Route, sort, both products and the weighted sum, as the part runs them, against the plain implementation; tokens
    whose choice hangs on less than rounding are left out of the comparison."""
    rng = np.random.default_rng(4)
    routes = stored + identity
    x32 = dev(rng.standard_normal((n, width)))
    x = x32.to(dtype)
    router = dev(rng.standard_normal((routes, width)) * 0.3, dtype)
    correction = dev(rng.standard_normal(routes) * 0.1)
    w_in = dev(rng.standard_normal((stored, inner, width)) * width ** -0.5, dtype)
    w_out = dev(rng.standard_normal((stored, width, inner)) * inner ** -0.5, dtype)
    ids = torch.zeros((n, top), dtype=torch.int32, device=DEV)
    weights = torch.zeros((n, top), dtype=torch.float32, device=DEV)
    kernels.moe_route(x, router, ids, weights, n_tokens=n, top=top, rule="softmax", choice_bias=correction, normalise=False)
    pairs = n * top
    offsets, tile_first = (torch.zeros(routes + 1, dtype=torch.int32, device=DEV) for _ in range(2))
    order, place = (torch.zeros(pairs, dtype=torch.int32, device=DEV) for _ in range(2))
    kernels.moe_sort(ids, offsets, tile_first, order, place, pairs=pairs, n_experts=routes)
    hidden = torch.zeros((pairs, inner), dtype=dtype, device=DEV)
    kernels.moe_expert(True, x, w_in, hidden, offsets, tile_first, order, None, pairs=pairs, top=top, activation="gelu_erf",
                       gated=False)
    part = torch.zeros((pairs, width), dtype=torch.float32, device=DEV)
    kernels.moe_expert(False, hidden, w_out, part, offsets, tile_first, order, weights, pairs=pairs, top=top)
    out = torch.zeros((n, width), dtype=torch.float32, device=DEV)
    kernels.moe_combine(part, place, out, n_tokens=n, top=top, ids=ids, weights=weights, identity_input=x32, n_stored=stored)
    w = {"router": host(router), "correction": host(correction)}
    for e in range(stored):
        w[f"e{e}.up"], w[f"e{e}.down"] = host(w_in[e]), host(w_out[e])
    mlp = {"router": {"experts": stored, "identity": identity, "top": top}}
    want = plain.routed_experts(host(x32) if dtype == torch.float32 else host(x), w, mlp)
    choice = torch.softmax(host(x) @ host(router).T, -1) + host(correction)
    ranked = choice.sort(-1, descending=True).values
    # (both sides sum the same rounded operands in 32-bit and more: a choice is sure where the gap is far above that)
    sure = (ranked[:, top - 1] - ranked[:, top]) > 1e-4 if top < routes else torch.ones(n, dtype=torch.bool)
    assert int(sure.sum()) > 0.9 * n
    # the chosen experts themselves, where the choice is sure: by score plus correction, the weights without it
    scores = torch.softmax(host(x) @ host(router).T, -1)
    for t in torch.nonzero(sure).flatten().tolist():
        assert sorted(ids[t].tolist()) == sorted(choice[t].topk(top).indices.tolist())
        np.testing.assert_allclose(host(weights[t]), scores[t, ids[t].long().cpu()], rtol=20 * tol, atol=tol)
    assert rel(host(out)[sure], want[sure]) < 2 * tol


def test_norm_added_with_a_factor_and_handed_on_as_it_is():
    rng = np.random.default_rng(5)
    n, width = 7, 90
    x, stream, weight = dev(rng.standard_normal((n, width))), dev(rng.standard_normal((n, width))), dev(rng.standard_normal(width))
    before = host(stream).clone()
    rounded = torch.full((n + 1, width), 9.0, dtype=torch.bfloat16, device=DEV)
    kernels.rmsnorm_add(x, weight, stream, 1e-4, n_rows=n, factor=0.35, next_out=rounded)
    want = before + 0.35 * plain.norm_plain(host(x), host(weight), 1e-4)
    assert rel(host(stream), want) < 1e-5
    assert torch.equal(rounded[:n], stream.to(torch.bfloat16)) and bool((rounded[n:] == 9.0).all())
