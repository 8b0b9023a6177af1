"""A plain, slow statement of the Totatar decoder in numpy float64, one function per mechanism,
for the tests to hold the engine against. It shares no code with the package: it reads a
config dict of the architecture's own keys and a dict of weight arrays by checkpoint name, and
runs a whole sequence at once, token after token where a mechanism is a recurrence (no cache,
no state carried between calls).

Notation: n tokens, width d; a mixer's input is X [n, d]; query heads H, key/value heads G,
key size a, value size b; a recurrent state is S.
"""
from __future__ import annotations

import math

import numpy as np


# ----------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """The model's norm: unit rms times (1 + w): the weight is zero-centred."""
    return unit_rms(x, eps) * (1.0 + w)


def group_norm(x, gain, eps, groups):
    """The last axis cut into `groups` equal consecutive parts, each brought to unit rms, the
    whole then multiplied by the plain gain."""
    n, d = x.shape
    return unit_rms(x.reshape(n, groups, d // groups), eps).reshape(n, d) * gain


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_interleaved(x, positions, rot):
    """x [n, heads, size]: within the first rot['dims'] channels, channel 2i pairs with 2i + 1
    and the pair turns by position * base^(-2i/dims) / factor; the rest pass."""
    if rot is None:
        return x
    dims, base = rot["dims"], float(rot["base"])
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    out = x.copy()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            ang = p * (base ** (-2.0 * i / dims) / factor)
            c, s = math.cos(ang), math.sin(ang)
            u, v = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            out[t, :, 2 * i] = u * c - v * s
            out[t, :, 2 * i + 1] = v * c + u * s
    return out


# ----------------------------------------------------------------------------------- mixers
def sink_window_attention(q, k, v, scale, window, sink):
    """q [n, H, a], k [n, G, a], v [n, G, b] -> [n, H, b]. Query i reads keys j with
    0 <= i - j < window (window None: every earlier key); the softmax's denominator also holds
    exp(sink_h), which has no value."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = max(s.max(), sink[h]) if sink is not None else s.max()
            e = np.exp(s - m)
            den = e.sum() + (math.exp(sink[h] - m) if sink is not None else 0.0)
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def same(x):
    return x


def softmax_branch(X, W, p, m, eps, rnd=same):
    """The softmax-attention side of a parallel mixer: biased projections, rotation, window,
    sink, output product. `rnd` rounds what a 16-bit engine stores in 16 bits."""
    n = X.shape[0]
    H, G, a, b = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = (rnd(X @ W[p + "q"].T) + W[p + "q.b"]).reshape(n, H, a)
    k = (rnd(X @ W[p + "k"].T) + W[p + "k.b"]).reshape(n, G, a)
    v = rnd(rnd(X @ W[p + "v"].T) + W[p + "v.b"]).reshape(n, G, b)
    pos = list(range(n))
    q, k = rnd(rotate_interleaved(q, pos, m.get("rot"))), rnd(rotate_interleaved(k, pos, m.get("rot")))
    window = (m.get("mask") or {}).get("size")
    scale = m["scale"] if m.get("scale") is not None else a ** -0.5
    o = sink_window_attention(q, k, v, scale, window, W.get(p + "sink"))
    return rnd(o.reshape(n, H * b)) @ W[p + "o"].T


def decayed_linear_attention(q, k, v, decay):
    """q, k [n, H, a], v [n, H, b], one fixed decay per head: S <- decay S + k v^T, o = S^T q."""
    n, H, a = q.shape
    out = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        S = np.zeros((a, v.shape[2]))
        for t in range(n):
            S = decay[h] * S + np.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def linear_branch(X, W, p, m, eps, rnd=same):
    """The linear-attention side: q, k, v through silu, the recurrence, one norm over all the
    heads together with a plain gain, a sigmoid gate, the output product."""
    n = X.shape[0]
    H, a, b = m["heads"], m["dim"], m.get("vdim", m["dim"])
    q = silu(rnd(X @ W[p + "q"].T)).reshape(n, H, a)
    k = silu(rnd(X @ W[p + "k"].T)).reshape(n, H, a)
    v = silu(rnd(X @ W[p + "v"].T)).reshape(n, H, b)
    o = decayed_linear_attention(q, k, v, m["decay"]).reshape(n, H * b)
    o = group_norm(o, W[p + "norm"], eps, 1) * sigmoid(rnd(X @ W[p + "g"].T))
    return rnd(o) @ W[p + "o"].T


def parallel_mixer(X, W, p, m, eps, rnd=same):
    return m.get("left_scale", 1.0) * softmax_branch(X, W, p + "left.", m["left"], eps, rnd) + \
        m.get("right_scale", 1.0) * linear_branch(X, W, p + "right.", m["right"], eps, rnd)


def causal_conv(x, w, bias):
    """x [n, c], w [c, taps]: y_t = bias + sum_j w[:, taps-1-j] x_(t-j), zeros before t = 0."""
    n, c = x.shape
    taps = w.shape[1]
    y = np.tile(bias, (n, 1)).astype(np.float64)
    for j in range(taps):
        if j < n:
            y[j:] += x[:n - j] * w[:, taps - 1 - j]
    return y


def selective_scan(x, dt, A, B, C, D, heads_per_group):
    """x [n, H, b], dt [n, H], B and C [n, G, N]: S <- exp(-A dt) S + dt B x^T (S [N, b]),
    y = S^T C + D x."""
    n, H, b = x.shape
    N = B.shape[2]
    y = np.zeros((n, H, b))
    for h in range(H):
        g = h // heads_per_group
        S = np.zeros((N, b))
        for t in range(n):
            S = math.exp(-A[h] * dt[t, h]) * S + dt[t, h] * np.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * x[t, h]
    return y


def state_space_mixer(X, W, p, m, eps, rnd=same):
    n = X.shape[0]
    H, b, N, G = m["heads"], m["vdim"], m["state"], m.get("groups", 1)
    inner = H * b
    z_all = rnd(X @ W[p + "in"].T)
    z = z_all[:, :inner]
    xbc = z_all[:, inner:2 * inner + 2 * G * N]
    dt = softplus(z_all[:, 2 * inner + 2 * G * N:] + W[p + "dt_bias"])
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].reshape(n, H, b)
    B = xbc[:, inner:inner + G * N].reshape(n, G, N)
    C = xbc[:, inner + G * N:].reshape(n, G, N)
    y = selective_scan(x, dt, np.exp(W[p + "A_log"]), B, C, W[p + "D"], H // G).reshape(n, inner)
    y = group_norm(y * silu(z), W[p + "norm"], eps, m.get("norm_groups", 1))
    return rnd(y) @ W[p + "o"].T


# ----------------------------------------------------------------------------- feed-forwards
def gated(X, W, p, act, rnd=same):
    return rnd(act(rnd(X @ W[p + "gate"].T)) * rnd(X @ W[p + "up"].T)) @ W[p + "down"].T


def routed(X, W, p, mlp, rnd=same):
    """Each token's `top` experts by router logit, weighted by the softmax over those logits
    alone, plus the shared expert."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = X @ W[p + "router"].T + W[p + "router.b"]
    out = np.zeros_like(X)
    for t in range(X.shape[0]):
        order = sorted(range(E), key=lambda e: (-logits[t, e], e))[:top]
        w = np.exp(logits[t, order] - logits[t, order].max())
        w /= w.sum()
        for e, we in zip(order, w):
            out[t] += we * gated(X[t:t + 1], W, f"{p}e{e}.", silu, rnd)[0]
    if mlp.get("shared"):
        out += gated(X, W, p + "shared.", silu, rnd)
    return out


def feed_forward(X, W, p, mlp, rnd=same):
    if mlp["kind"] == "dense":
        return gated(X, W, p, gelu_tanh, rnd)
    return routed(X, W, p, mlp, rnd)


# ------------------------------------------------------------------------------------ model
def forward(cfg, W, tokens, layer_outputs=None, rnd=same):
    """Logits [n, vocab] of a whole sequence. `layer_outputs`, a list, gets the stream after
    every layer. With `rnd` (a rounding to a 16-bit type) the sublayers' inputs, the
    projections' results and what the last products read are rounded, as a 16-bit engine
    stores them; the stream, the norms, the softmax and the recurrences stay as they are."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)].astype(np.float64)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rnd(offset_norm(x, W[p + "norm1"], eps))
        if layer["type"] == "parallel":
            y = parallel_mixer(h, W, p + "mix.", layer["mixer"], eps, rnd)
        elif layer["type"] == "mamba2":
            y = state_space_mixer(h, W, p + "mix.", layer["mixer"], eps, rnd)
        else:
            raise ValueError(layer["type"])
        x = x + offset_norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(rnd(offset_norm(x, W[p + "norm2"], eps)), W, p + "mlp.", layer["mlp"], rnd)
            x = x + offset_norm(y, W[p + "norm2b"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    return rnd(offset_norm(x, W["final.norm"], eps)) @ W["embed"].T


def greedy(cfg, W, prompt, n):
    """The n tokens that follow `prompt` when the largest logit is taken every time (ties: the
    lower id)."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(np.argmax(forward(cfg, W, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out
