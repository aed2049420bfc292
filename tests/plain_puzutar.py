"""A plain, slow restatement of the Puzutar design in float64 numpy: one function per mechanism, whole
sequences at a time, no cache and no batching.  It shares nothing with the engine; the tests compare the
engine's logits with it.

A model is (config, weights): `config` is the dictionary of the design's config.json, `weights` maps the
file's tensor names to arrays.

Notation: x is the residual stream [n, width]; h the normalised rows; position p counts from 0.
"""
import math

import numpy as np


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def rms(v, eps):
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def grouped_rms_norm(x, w, groups, eps):
    n, width = x.shape
    parts = x.reshape(n, groups, width // groups)
    return rms(parts, eps).reshape(n, width) * w


def token_shift(h, mu):
    """Row t becomes h_t + (h_{t-1} - h_t) * mu, with zeros before the first row."""
    prev = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (prev - h) * mu


def xielu(z, p, q):
    a_pos = softplus(p)
    a_neg = 0.5 + softplus(q)
    zn = np.minimum(z, 0.0)
    return np.where(z > 0, a_pos * z * z + 0.5 * z, a_neg * (np.expm1(zn) - zn) + 0.5 * z)


def dense_ff(h, W, prefix):
    z = h @ W[prefix + "up"].T + W[prefix + "up.b"]
    p, q = (float(v) for v in W[prefix + "act"])
    return xielu(z, p, q) @ W[prefix + "down"].T + W[prefix + "down.b"]


def rotate_half(v, positions, base, dims):
    """Rotates the first `dims` entries of the last axis; entry i pairs with entry i + dims/2."""
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = positions[:, None].astype(np.float64) * freq[None, :]
    shape = (len(positions),) + (1,) * (v.ndim - 2) + (half,)
    cos, sin = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = v[..., :half], v[..., half:dims]
    return np.concatenate([a * cos - b * sin, b * cos + a * sin, v[..., dims:]], axis=-1)


def latent_and_key(h, W, prefix, m, eps):
    """What a layer with a down projection of its own leaves for keys and values: the normalised latent and
    the rotated key part shared by all heads."""
    rank, rot = m["kv_rank"], m["rot_dim"]
    d = h @ W[prefix + "dkv"].T
    c = rms(d[:, :rank], eps) * W[prefix + "dkv.norm"]
    kr = rotate_half(d[:, rank:rank + rot], np.arange(len(h)), m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, W, prefix, m, c, kr):
    n = len(h)
    H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ W[prefix + "q"].T).reshape(n, H, dim + rot)
    q_plain = q[..., :dim]
    q_rot = rotate_half(q[..., dim:], np.arange(n), m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ W[prefix + "uk"].T).reshape(n, H, dim)
    v = (c @ W[prefix + "uv"].T).reshape(n, H, vdim)
    scores = (np.einsum("ihd,jhd->hij", q_plain, k_plain) + np.einsum("ihd,jd->hij", q_rot, kr)) * m["scale"]
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    seen = (i - j >= 0)
    if m.get("mask") is not None:
        seen &= (i - j < m["mask"]["size"])
    scores = np.where(seen[None], scores, -np.inf)
    scores -= scores.max(axis=-1, keepdims=True)
    wts = np.exp(scores)
    wts /= wts.sum(axis=-1, keepdims=True)
    out = np.einsum("hij,jhv->ihv", wts, v).reshape(n, H * vdim)
    return out @ W[prefix + "o"].T


def token_side(x, tokens, W, layer, dim, eps):
    p = f"l{layer}.side."
    e = W["side.embed"][tokens, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ W[p + "gate"].T) * e
    y = g @ W[p + "proj"].T
    return x + rms(y, eps) * W[p + "norm"]


def forward(config, weights, tokens, return_layers=False, trace=None):
    """Logits [n, vocab] of a whole sequence (and the residual stream after every layer).  `trace`, a list, receives
    (name, rows) after every mechanism of every layer."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    tokens = np.asarray(tokens, dtype=np.int64)
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    x = W["embed"][tokens]
    kept = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        assert layer["type"] == "latent_attention"
        m = layer["mixer"]
        note = (lambda name, rows: trace.append((name, rows.copy()))) if trace is not None else (lambda name, rows: None)
        h = grouped_rms_norm(x, W[f"l{i}.norm1"], groups, eps)
        note("norm", h)
        hm = token_shift(h, W[f"l{i}.shift"])
        note("shift", hm)
        if m.get("kv_from") is None:
            kept[i] = latent_and_key(hm, W, f"l{i}.mix.", m, eps)
        c, kr = kept[i if m.get("kv_from") is None else m["kv_from"]]
        y = latent_attention(hm, W, f"l{i}.mix.", m, c, kr)
        note("mixer", x + y)
        if layer.get("mlp") is not None:
            assert layer["mlp"]["kind"] == "dense"
            y = y + dense_ff(h, W, f"l{i}.mlp.")
            note("feed_forward", x + y)
        x = x + y
        if config.get("token_side") is not None:
            x = token_side(x, tokens, W, i, config["token_side"]["dim"], eps)
            note("token_input", x)
        after.append(x.copy())
    logits = grouped_rms_norm(x, W["final.norm"], groups, eps) @ W["embed"].T
    return (logits, np.stack(after)) if return_layers else logits
