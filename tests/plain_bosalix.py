"""Bosalix written out plainly: one function per mechanism, float64 on the CPU, a sequence at a time, token loops
where a loop says it best.  Shares no code with the package; the tests compare the package's kernels and engine
with these functions.

A model is (config, tensors): the configuration as a dictionary and the checkpoint's tensors by name.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_divide(x, eps):
    """x over the root of (its mean square plus eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_plain(x, weight, eps):
    return rms_divide(x, eps) * weight


def norm_around_zero(x, weight, eps):
    """The gain is kept minus one."""
    return rms_divide(x, eps) * (1.0 + weight)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def token_shift(h, shift, before=None):
    """Row t becomes h[t] + (h[t-1] - h[t]) * shift with the rows as they came in; the row before the first is
    `before` (zeros for a sequence's first token).  Returns the new rows and the last incoming row."""
    prev = torch.zeros_like(h)
    prev[1:] = h[:-1]
    if before is not None:
        prev[0] = before
    return h + (prev - h) * shift, h[-1].clone()


def plain_frequencies(dims, base):
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def stretched_frequencies(dims, base, scaling):
    """Long wavelengths are stretched by `factor`, short ones kept, a linear blend between the two bounds."""
    out = []
    for f in plain_frequencies(dims, base):
        if scaling is None:
            out.append(f)
            continue
        factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


def rotate_pairs(x, positions, freqs, layout):
    """x [tokens, vectors, length]: the first 2 * len(freqs) channels of every vector are turned, pair i by the angle
    position * freqs[i]; `layout` "interleaved" pairs (2i, 2i+1), "half" pairs (i, i + len(freqs))."""
    half = len(freqs)
    out = x.clone()
    if half == 0:
        return out
    angle = positions.to(F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]       # [tokens, half]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    if layout == "interleaved":
        u, v = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = u * cos - v * sin
        out[..., 1:2 * half:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:2 * half]
        out[..., :half] = u * cos - v * sin
        out[..., half:2 * half] = v * cos + u * sin
    return out


def visible(i, j, size, keep_first):
    """May position i attend position j?"""
    if j > i:
        return False
    if size is None:
        return True
    return i - j < size or j < keep_first


def visibility(n, size, keep_first):
    """[n, n] of booleans: row i, column j."""
    return torch.tensor([[visible(i, j, size, keep_first) for j in range(n)] for i in range(n)])


def latent_attention(h, w, m, eps):
    """h [tokens, width] of one sequence from its first token; w: the mixer's tensors by short name."""
    n = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(n)
    cq = norm_plain(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(n, heads, dim + rot)
    down = h @ w["dkv"].T
    c = norm_plain(down[:, :rank], w["dkv.norm"], eps)
    freqs = plain_frequencies(m["rot"]["dims"], m["rot"]["base"])
    shared = rotate_pairs(down[:, rank:].view(n, 1, rot), positions, freqs, "interleaved")[:, 0]
    q_rot = rotate_pairs(q[..., dim:], positions, freqs, "interleaved")
    k_plain = (c @ w["uk"].T).view(n, heads, dim)
    v = (c @ w["uv"].T).view(n, heads, vdim)
    size = m.get("mask", {}).get("size") if m.get("mask") else None
    seen = visibility(n, size, 0)
    out = torch.zeros(n, heads, vdim, dtype=F64)
    for head in range(heads):
        scores = (q[:, head, :dim] @ k_plain[:, head].T + q_rot[:, head] @ shared.T) * m["scale"]      # [query, key]
        p = torch.softmax(scores.masked_fill(~seen, -math.inf), -1)
        out[:, head] = p @ v[:, head]
    return out.reshape(n, heads * vdim) @ w["o"].T


def gated_attention_values(h, w, m, eps):
    """The values of the sigmoid attention as they leave their norm: [tokens, kv_heads, vdim]."""
    n = h.shape[0]
    v = (h @ w["v"].T + w["v.b"]).view(n, m["kv_heads"], m["vdim"])
    return rms_divide(v, eps)


def sigmoid_attention(h, w, m, eps, v_first=None):
    """Returns (the mixer's output, the values it attended over)."""
    n = h.shape[0]
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(n)
    q = norm_plain((h @ w["q"].T + w["q.b"]).view(n, heads, dim), w["q.norm"], eps)
    k = norm_plain((h @ w["k"].T + w["k.b"]).view(n, groups, dim), w["k.norm"], eps)
    freqs = stretched_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q, k = rotate_pairs(q, positions, freqs, "half"), rotate_pairs(k, positions, freqs, "half")
    v = gated_attention_values(h, w, m, eps)
    if v_first is not None:
        lam = w["vmix"]
        v = (1.0 - lam) * v + lam * v_first
    mask = m.get("mask") or {}
    size, keep = mask.get("size"), mask.get("keep_first", 0)
    seen = visibility(n, size, keep)
    out = torch.zeros(n, heads, vdim, dtype=F64)
    for head in range(heads):
        g = head // (heads // groups)
        weights = torch.sigmoid((q[:, head] @ k[:, g].T) * m["scale"] + w["pb"][head])      # [query, key], not normalised
        out[:, head] = (weights * seen) @ v[:, g]
    return out.reshape(n, heads * vdim) @ w["o"].T + w["o.b"], v


def routed_experts(h, w, mlp):
    """Softmax router over the stored and the identity experts; a token's `top` choices by score plus correction,
    weighted by the bare scores, not renormalised."""
    router = mlp["router"]
    stored, identity, top = router["experts"], router.get("identity", 0), router["top"]
    scores = torch.softmax(h @ w["router"].T, -1)
    choice = scores + w["correction"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(stored + identity), key=lambda e: (-float(choice[t, e]), e))[:top]
        for e in order:
            if e >= stored:
                out[t] += scores[t, e] * h[t]
            else:
                out[t] += scores[t, e] * (w[f"e{e}.down"] @ gelu_erf(w[f"e{e}.up"] @ h[t]))
    return out


def as_f64(value):
    return value.to(F64) if isinstance(value, torch.Tensor) else torch.as_tensor(value, dtype=F64)


def layer_tensors(tensors, i, part):
    prefix = f"l{i}.{part}."
    return {k[len(prefix):]: as_f64(v) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, keep_layers=False):
    """Logits [tokens, vocab] of one sequence (and the stream after every layer)."""
    eps, mult = config["norm"]["eps"], config["residual_mult"]
    x = as_f64(tensors["embed"])[torch.tensor(tokens)] * config["embedding"]["scale"]
    v_first = None
    stream = []
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        h, _ = token_shift(x, as_f64(tensors[f"l{i}.shift"]))
        w = layer_tensors(tensors, i, "mix")
        if layer["type"] == "latent_attention":
            mixed = latent_attention(h, w, m, eps)
        else:
            mixing = bool(m.get("v_mix"))
            mixed, v = sigmoid_attention(h, w, m, eps, v_first if mixing else None)
            if mixing and v_first is None:
                v_first = v
        x = x + mult * norm_around_zero(mixed, as_f64(tensors[f"l{i}.norm1"]), eps)
        if layer.get("mlp") is not None:
            y = routed_experts(x, layer_tensors(tensors, i, "mlp"), layer["mlp"])
            x = x + mult * norm_around_zero(y, as_f64(tensors[f"l{i}.norm2"]), eps)
        stream.append(x.clone())
    logits = norm_around_zero(x, as_f64(tensors["final.norm"]), eps) @ as_f64(tensors["head"]).T
    return (logits, torch.stack(stream)) if keep_layers else logits.numpy()
