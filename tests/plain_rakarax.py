"""Rakarax in plain NumPy, float64, whole sequences, no cache: the oracle of the Rakarax tests.

One function per mechanism, written from the design's equations; nothing here is shared with the library.  `weights`
maps checkpoint names to arrays (matrices stored [out, in]); `config` is the config.json dictionary.
"""
from __future__ import annotations

import numpy as np


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the gain minus one."""
    return rms_unit(x, eps) * (1.0 + w)


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return np.logaddexp(0.0, x)


def causal_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u], axis=0)
    y = np.zeros_like(u)
    for j in range(taps):
        y += padded[j:j + u.shape[0]] * w[:, j]
    return y if bias is None else y + bias


def rotate_half(x, positions, dims, base):
    """x [T, H, D]: channel i < dims/2 is paired with channel i + dims/2; the rest passes."""
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    angle = positions[:, None].astype(np.float64) * freq[None, :]
    c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def retention(h, w, p, m, eps):
    """The mixer 'retention' over one sequence h [T, width]; p is the tensors' prefix, m the mixer's configuration."""
    T = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, heads, dim)
    k = (h @ w[p + "k"].T).reshape(T, heads, dim)
    v = (h @ w[p + "v"].T).reshape(T, heads, vdim)
    q = rotate_half(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half(k, pos, m["rot"]["dims"], m["rot"]["base"]) * dim ** -0.5
    out = np.zeros((T, heads, vdim))
    for a in range(heads):
        S = np.zeros((dim, vdim))
        for t in range(T):
            S = m["decay"][a] * S + np.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    out = rms_unit(out, eps).reshape(T, heads * vdim)
    return (out * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def conv_attention(h, w, p, m, eps):
    """The left half of the mixer 'parallel': windowed softmax attention whose values are its keys."""
    T = h.shape[0]
    H, G, dim = m["heads"], m["kv_heads"], m["dim"]
    q = causal_conv(h @ w[p + "q"].T, w[p + "q.conv"]).reshape(T, H, dim)
    k = causal_conv(h @ w[p + "k"].T, w[p + "k.conv"]).reshape(T, G, dim)
    v = k
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    scores = np.zeros((H, T, T))
    for a in range(H):
        s = (q[:, a] @ k[:, a // (H // G)].T) * m["scale"] * w[p + "temp"][a]
        s = m["softcap"] * np.tanh(s / m["softcap"])
        scores[a] = s - 2.0 ** (-8.0 * (a + 1) / H) * (i - j)
    scores = np.einsum("hg,gij->hij", w[p + "talk"], scores)
    seen = (j <= i) & (i - j < m["mask"]["size"])
    scores = np.where(seen[None], scores, -np.inf)
    scores -= scores.max(axis=-1, keepdims=True)
    weights = np.exp(scores)
    weights /= weights.sum(axis=-1, keepdims=True)
    out = np.stack([weights[a] @ v[:, a // (H // G)] for a in range(H)], axis=1).reshape(T, H * m["vdim"])
    return (out * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def selective_scan(h, w, p, m):
    """The right half of the mixer 'parallel'."""
    T = h.shape[0]
    inner, n_state, rank = m["inner"], m["state"], m["dt_rank"]
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, w[p + "conv"], w[p + "conv.b"]))
    low = x @ w[p + "x"].T
    dt = softplus(low[:, :rank] @ w[p + "dt"].T + w[p + "dt.b"])
    B, C = low[:, rank:rank + n_state], low[:, rank + n_state:]
    A = -np.exp(w[p + "A_log"])
    S = np.zeros((inner, n_state))
    y = np.zeros((T, inner))
    for t in range(T):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[p + "D"] * x[t]
    return (y * silu(z)) @ w[p + "o"].T


def poly_norm_ff(h, w, p, eps):
    z = h @ w[p + "up"].T
    a, b, c, e = w[p + "act"]
    act = a * rms_unit(z, eps) + b * rms_unit(z * z, eps) + c * rms_unit(z * z * z, eps) + e
    return act @ w[p + "down"].T


def mixer(h, w, layer, p, eps):
    m = layer["mixer"]
    if layer["type"] == "retention":
        return retention(h, w, p + "mix.", m, eps)
    if layer["type"] == "parallel":
        return (m["left_scale"] * conv_attention(h, w, p + "mix.left.", m["left"], eps)
                + m["right_scale"] * selective_scan(h, w, p + "mix.right.", m["right"]))
    raise ValueError(layer["type"])


def forward(config, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer run)."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    tokens = np.asarray(tokens)
    x = w["embed"][tokens] + w["pos"][np.arange(len(tokens))]
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        x = x + offset_norm(mixer(offset_norm(x, w[p + "norm1"], eps), w, layer, p, eps), w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            x = x + offset_norm(poly_norm_ff(offset_norm(x, w[p + "norm2"], eps), w, p + "mlp.", eps), w[p + "norm2b"], eps)
        after.append(x)
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(after)) if return_layers else logits
