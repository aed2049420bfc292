"""A plain, slow restatement of the Vosurax design in float64 numpy: one function per mechanism, whole
sequences at a time, token by token where the design has a recurrence, no cache and no batching.  It shares
nothing with the engine; the tests compare the engine's logits with it.

A model is (config, weights): `config` is the dictionary of the design's config.json, `weights` maps the
file's tensor names to arrays.

Notation: x is the residual stream [n, width]; h a block's normalised input; position p counts from 0.
"""
import math

import numpy as np


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def log_sigmoid(z):
    return -(np.log1p(np.exp(-np.abs(z))) + np.maximum(-z, 0.0))


def rms(v, eps):
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def block_norm(x, w, eps):
    """The blocks' and the model's norm: the gain is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def rotate_half(v, positions, base, dims):
    """Rotates the first `dims` entries of the last axis of v [n, heads, d]; entry i pairs with entry i + dims/2."""
    half = dims // 2
    if half == 0:
        return v.copy()
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    out = v.copy()
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


# ---- mixer: retention ------------------------------------------------------------------------------------

def retention(h, W, p, m, eps, trace=None):
    """Linear attention with one fixed decay per head: S_t = g S_{t-1} + k_t v_t^T, o_t = S_t^T q_t."""
    n = h.shape[0]
    H, D, E = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q = (h @ W[p + "q"].T).reshape(n, H, D)
    k = (h @ W[p + "k"].T).reshape(n, H, D)
    v = (h @ W[p + "v"].T).reshape(n, H, E)
    rot = m.get("rot") or {}
    dims = rot.get("dims", 0)
    if dims:
        q = rotate_half(q, pos, rot["base"], dims)
        k = rotate_half(k, pos, rot["base"], dims)
    k = k * D ** -0.5
    o = np.zeros((n, H, E))
    for a in range(H):
        S = np.zeros((D, E))
        g = float(m["decay"][a])
        for t in range(n):
            S = g * S + np.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    y = rms(o, eps).reshape(n, H * E) * silu(h @ W[p + "g"].T)
    if trace is not None:
        trace["retention.heads"] = o.reshape(n, H * E)
    return y @ W[p + "o"].T


# ---- mixer: two side by side -------------------------------------------------------------------------------

def chunk_attention(h, W, p, m, eps, trace=None):
    """Softmax attention with grouped keys/values, RMS-normed queries and keys, no rotation, an output gate, and a
    mask in chunks counted from position 0: i sees j <= i in the same chunk."""
    n = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(n, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(n, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(n, G, E)
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    size = (m.get("mask") or {}).get("size", 0)
    i = np.arange(n)
    see = i[None, :] <= i[:, None]
    if size:
        see &= (i[None, :] // size) == (i[:, None] // size)
    out = np.zeros((n, H, E))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        s = np.where(see, s, -np.inf)
        w = np.exp(s - s.max(axis=1, keepdims=True))
        w /= w.sum(axis=1, keepdims=True)
        out[:, a] = w @ v[:, g]
    if trace is not None:
        trace["attention.heads"] = out.reshape(n, H * E)
    y = out.reshape(n, H * E) * sigmoid(h @ W[p + "g"].T)
    return y @ W[p + "o"].T


START_MAX = 0.0      # where the running maximum of a gated memory starts
FLOOR = True         # whether exp(-m) bounds the gated memory's divisor from below (tests switch it off to show that it matters)


def matrix_memory(h, W, p, m, eps, trace=None):
    """A matrix memory per head with exponential input gate and a running maximum that starts at 0."""
    n = h.shape[0]
    H, D, E, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ W[p + "q"].T).reshape(n, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).reshape(n, H, D)
    v = (h @ W[p + "v"].T).reshape(n, H, E)
    gi = cap * np.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)
    gf = log_sigmoid(cap * np.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    o = np.zeros((n, H, E))
    for a in range(H):
        S, z, mx = np.zeros((D, E)), np.zeros(D), START_MAX
        for t in range(n):
            new = max(gf[t, a] + mx, gi[t, a])
            keep, take = math.exp(gf[t, a] + mx - new), math.exp(gi[t, a] - new)
            S = keep * S + take * np.outer(k[t, a], v[t, a])
            z = keep * z + take * k[t, a]
            mx = new
            o[t, a] = (S.T @ q[t, a]) / (max(abs(float(z @ q[t, a])), math.exp(-mx) if FLOOR else 0.0) + 1e-6)
    if trace is not None:
        trace["memory.heads"] = o.reshape(n, H * E)
    y = rms(o, eps).reshape(n, H * E) * W[p + "norm"] * sigmoid(h @ W[p + "g"].T)
    return y @ W[p + "o"].T


def side_by_side(h, W, p, m, eps, trace=None):
    left = chunk_attention(h, W, p + "left.", m["left"], eps, trace)
    right = matrix_memory(h, W, p + "right.", m["right"], eps, trace)
    if trace is not None:
        trace["left"], trace["right"] = left, right
    return 0.5 * (rms(left, eps) * W[p + "left.out"] + rms(right, eps) * W[p + "right.out"])


# ---- feed-forwards -------------------------------------------------------------------------------------------

def dense_ff(h, W, p):
    return gelu_tanh(h @ W[p + "up"].T) @ W[p + "down"].T


def gated_ff(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def routed_ff(h, W, p, mlp, trace=None):
    """Every row goes to its `top` experts with the largest sigmoid scores; the score scales the expert's input."""
    n = h.shape[0]
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = sigmoid(h @ W[p + "router"].T)
    order = np.argsort(-s, axis=1, kind="stable")[:, :top]
    y = np.zeros((n, W[p + "e0.down"].shape[0]))
    for t in range(n):
        for e in order[t]:
            y[t] += gated_ff(s[t, e] * h[t:t + 1], W, f"{p}e{e}.")[0]
    if trace is not None:
        trace["experts"] = order
        trace["scores"] = s
        trace["routed_only"] = y.copy()
    if mlp.get("shared"):
        y += gated_ff(h, W, p + "shared.")
    return y


# ---- the model -------------------------------------------------------------------------------------------------

def run_order(config):
    """(layer, pass) in the order the layers run: layers start .. stop-1 are run `times` times in a row."""
    L = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(L)]
    out = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        out += [(i, t) for i in range(loop["start"], loop["stop"])]
    out += [(i, None) for i in range(loop["stop"], L)]
    return out


def layer_forward(x, W, config, i, trace=None):
    eps = config["norm"]["eps"]
    lc = config["layers"][i]
    p = f"l{i}."
    h = block_norm(x, W[p + "norm1"], eps)
    if lc["type"] == "retention":
        x = x + retention(h, W, p + "mix.", lc["mixer"], eps, trace)
    elif lc["type"] == "parallel":
        x = x + side_by_side(h, W, p + "mix.", lc["mixer"], eps, trace)
    else:
        raise ValueError(lc["type"])
    if trace is not None:
        trace["mixer"] = x
    mlp = lc.get("mlp")
    if mlp:
        h = block_norm(x, W[p + "norm2"], eps)
        if mlp["kind"] == "dense":
            x = x + dense_ff(h, W, p + "mlp.")
        elif mlp["kind"] == "moe":
            y = routed_ff(h, W, p + "mlp.", mlp, trace)
            if trace is not None:
                trace["routed"] = x + trace.pop("routed_only")
            x = x + y
        else:
            raise ValueError(mlp["kind"])
    return x


def forward(config, W, tokens, traces=None):
    """Logits [n, vocab] of one sequence; `traces`, when a list, receives one dictionary per layer run."""
    x = W["embed"][np.asarray(tokens)]
    loop = config.get("loop")
    for i, t in run_order(config):
        if t is not None and i == loop["start"]:
            x = x + W["loop.step"][t]
        trace = {} if traces is not None else None
        x = layer_forward(x, W, config, i, trace)
        if traces is not None:
            trace["out"] = x
            traces.append(trace)
    y = block_norm(x, W["final.norm"], config["norm"]["eps"])
    return y @ W["head"].T
