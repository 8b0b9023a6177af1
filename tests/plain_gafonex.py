"""A plain, slow statement of the Gafonex decoder in numpy float64, one function per mechanism,
for the tests to hold the engine against. It shares no code with the package: it reads a
config dict of the architecture's own keys and a dict of weight arrays by checkpoint name, and
runs a whole sequence at once with dense matrices (no cache, no state carried between calls).

Notation: n tokens, width d; a mixer's input is X [n, d]; heads H, key/value heads G, key
size a, value size b.
"""
from __future__ import annotations

import math

import numpy as np


# ----------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def group_norm(x, gain, eps, groups):
    """The last axis cut into `groups` equal consecutive parts, each brought to unit rms, the
    whole then multiplied by the gain."""
    n, d = x.shape
    parts = x.reshape(n, groups, d // groups)
    return unit_rms(parts, eps).reshape(n, d) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def soft_cap(z, cap):
    return cap * np.tanh(z / cap)


def rotary_frequencies(rot):
    """Frequencies of the rot['dims'] / 2 pairs and the factor on cos and sin."""
    dims, base = rot["dims"], float(rot["base"])
    freq = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return freq, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    out = np.empty_like(freq)
    for i in range(dims // 2):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = freq[i] / factor * ramp + freq[i] * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [n, heads, size]: channel i < dims/2 pairs with channel i + dims/2; the rest pass."""
    if rot is None:
        return x
    dims = rot["dims"]
    half = dims // 2
    freq, mag = rotary_frequencies(rot)
    out = x.copy()
    for t, p in enumerate(positions):
        for i in range(half):
            ang = p * freq[i]
            c, s = math.cos(ang) * mag, math.sin(ang) * mag
            u, v = x[t, :, i], x[t, :, i + half]
            out[t, :, i] = u * c - v * s
            out[t, :, i + half] = v * c + u * s
    return out


# ----------------------------------------------------------------------------------- mixers
def attention_weights(q, k, scale):
    """q [n, H, a], k [n, G, a] -> causal softmax weights [H, n, n]."""
    n, H, _ = q.shape
    G = k.shape[1]
    w = np.zeros((H, n, n))
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            s = np.array([np.dot(q[i, h], k[j, g]) * scale for j in range(i + 1)])
            e = np.exp(s - s.max())
            w[h, i, :i + 1] = e / e.sum()
    return w


def mix_heads(w, table):
    """w [H, n, n] -> sum_g table[h, g] w[g]."""
    return np.einsum("hg,gij->hij", table, w)


def same(x):
    return x


def attention_mixer(X, m, W, prefix, eps, positions, shared, rnd=same):
    """`shared` is a dict carried through the layers of one forward: the first layer with
    v_mix leaves its values there, the later ones blend theirs with them. `rnd` rounds what a
    16-bit engine would store (projections, cached keys and values, the heads' outputs)."""
    n = X.shape[0]
    H, G, a = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    b = m.get("vdim", a)
    q = rnd(X @ W[prefix + "q"].T).reshape(n, H, a)
    k = rnd(X @ W[prefix + "k"].T).reshape(n, G, a)
    v = rnd(X @ W[prefix + "v"].T).reshape(n, G, b)
    q = unit_rms(q, eps) * W[prefix + "q.norm"]
    k = unit_rms(k, eps) * W[prefix + "k.norm"]
    q, k = rnd(rotate(q, positions, m.get("rot"))), rnd(rotate(k, positions, m.get("rot")))
    v = unit_rms(v, eps)
    if m.get("v_mix"):
        if "values" in shared:
            lam = float(W[prefix + "vmix"])
            v = (1.0 - lam) * v + lam * shared["values"]
        else:
            shared["values"] = v
    v = rnd(v)
    w = mix_heads(attention_weights(q, k, float(m["scale"])), W[prefix + "talk"])
    out = np.zeros((n, H, b))
    for h in range(H):
        out[:, h, :] = w[h] @ v[:, h // (H // G), :]
    return rnd(out.reshape(n, H * b)) @ W[prefix + "o"].T


def retention_outputs(q, k, v, decay):
    """q, k [n, H, a], v [n, H, b]: S <- decay S + k v^T from zero, o = S^T q, token by token."""
    n, H, a = q.shape
    b = v.shape[2]
    out = np.zeros((n, H, b))
    for h in range(H):
        S = np.zeros((a, b))
        for t in range(n):
            S = decay[h] * S + np.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def retention_mixer(X, m, W, prefix, eps, positions, rnd=same):
    n = X.shape[0]
    H, a = m["heads"], m["dim"]
    b = m.get("vdim", a)
    q = rotate(rnd(X @ W[prefix + "q"].T).reshape(n, H, a), positions, m.get("rot"))
    k = rotate(rnd(X @ W[prefix + "k"].T).reshape(n, H, a), positions, m.get("rot")) * a ** -0.5
    v = rnd(X @ W[prefix + "v"].T).reshape(n, H, b)
    o = unit_rms(retention_outputs(q, k, v, m["decay"]), eps).reshape(n, H * b)
    z = rnd(X @ W[prefix + "g"].T)
    return rnd(o * (z / (1.0 + np.exp(-z)))) @ W[prefix + "o"].T


def feed_forward(X, W, prefix, rnd=same):
    gate, up = rnd(X @ W[prefix + "gate"].T), rnd(X @ W[prefix + "up"].T)
    return rnd(np.maximum(gate, 0.0) * up) @ W[prefix + "down"].T


# ------------------------------------------------------------------------------- the model
def forward(cfg, W, tokens, layers_out=None, rnd=same):
    """Logits [n, vocab] of one sequence from position 0; `layers_out` (a list) collects the
    stream after every layer. With `rnd` (a rounding to a 16-bit type) the sublayers' inputs
    and what they store are rounded as an engine with 16-bit activations would, the stream,
    the norms, the softmax and the recurrence staying exact: how far that moves the logits is
    the yardstick for such an engine."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    positions = list(range(len(tokens)))
    x = W["embed"][np.asarray(tokens)]
    shared = {}
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        if layer["type"] == "attention":
            y = attention_mixer(rnd(x), layer["mixer"], W, pre + "mix.", eps, positions, shared, rnd)
        else:
            y = retention_mixer(rnd(x), layer["mixer"], W, pre + "mix.", eps, positions, rnd)
        x = x + group_norm(y, W[pre + "norm1"], eps, groups) * W[pre + "ls1"]
        if layer.get("mlp"):
            y = feed_forward(rnd(x), W, pre + "mlp.", rnd)
            x = x + group_norm(y, W[pre + "norm2"], eps, groups) * W[pre + "ls2"]
        if layers_out is not None:
            layers_out.append(x.copy())
    z = rnd(group_norm(x, W["final.norm"], eps, groups)) @ W["head"].T
    if cfg.get("logit_softcap"):
        z = soft_cap(z, cfg["logit_softcap"])
    return z


def greedy(cfg, W, prompt, n_new):
    """Greedy continuation, the whole sequence run again for every token; ties go to the
    lowest id."""
    tokens, out = list(prompt), []
    for _ in range(n_new):
        z = forward(cfg, W, tokens)[-1]
        nxt = int(np.argmax(z))
        out.append(nxt)
        tokens.append(nxt)
    return out
