"""A plain, slow implementation of the Fusazen decoder: the oracle of its tests.

Whole sequences, no cache, no batching, numpy only, float64, one function per mechanism.  It shares
no code with the library (the model folder is read with ``plain_llama.read_safetensors``, which is test
code as well).

Notation: ``x`` is the residual stream [T, W]; a matrix is stored [out, in] and applied as ``x @ M.T``;
the T tokens stand at positions 0..T-1.

The design, restated:

* embedding: row of the table times ``embedding.scale``;
* a layer is x += mixer(c(n1(x))) and then, if it has a feed-forward, x += ff(n2(x)), where n1, n2 are RMS
  norms with a weight and c(h) = h + (a causal convolution of h over time, per channel, ``canon.taps`` taps);
* mixers: ``general_delta`` (a matrix state per head with a decay per key channel and a rank-one removal
  along the unit key), ``attention`` (two softmax maps per head whose difference is taken, rotated on the
  first ``rot.dims`` entries of each map, optionally on the keys and values another layer has made) and
  ``attention_2`` (RMS norm over the whole query and key rows, a learned factor per head, no positions);
  both kinds of attention see the keys of their own block of ``mask.size`` positions only;
* feed-forward: down(relu(up h + b)^2) + b;
* the last RMS norm and an untied head.
"""
from __future__ import annotations

import json
import os

import numpy as np

from plain_llama import read_safetensors


def read_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ----------------------------------------------------------------------------- small pieces

def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softmax_rows(z):
    z = z - np.max(z, axis=-1, keepdims=True)
    e = np.exp(z)
    return e / np.sum(e, axis=-1, keepdims=True)


def time_conv_add(h, taps_w):
    """h + conv(h): out[t, c] = h[t, c] + sum_j taps_w[c, j] * h[t - (K-1) + j, c], zeros before the start."""
    T, K = h.shape[0], taps_w.shape[1]
    out = np.array(h, dtype=np.float64, copy=True)
    for j in range(K):
        back = K - 1 - j
        if back < T:
            out[back:] += taps_w[None, :, j] * h[:T - back]
    return out


def rotate_halves(v, positions, base, dims):
    """The first ``dims`` entries of the last axis rotated in pairs (i, i + dims/2) by the angle
    position * base^(-2i/dims); the rest passes.  v: [T, heads, D]."""
    out = np.array(v, dtype=np.float64, copy=True)
    if dims == 0:
        return out
    half = dims // 2
    freq = float(base) ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    lo, hi = v[..., :half], v[..., half:dims]
    out[..., :half] = lo * c - hi * s
    out[..., half:dims] = hi * c + lo * s
    return out


def block_mask(T, size):
    """[T, T] True where key j is visible from query i: j <= i and both in the same block of ``size`` positions."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def masked_attention(q, k, v, scale, mask):
    """q [T, D], k [T, D], v [T, Dv] of one head -> [T, Dv]."""
    s = (q @ k.T) * scale
    s = np.where(mask, s, -np.inf)
    return softmax_rows(s) @ v


# ----------------------------------------------------------------------------- mixers

def _rotation(m):
    """(base, rotated entries) of a mixer; one without a rotation has none."""
    rot = m.get("rot")
    return (rot["base"], rot["dims"]) if rot else (1.0, 0)


def keys_values_diff(h, w, p, m):
    """Rotated keys [T, G, 2, D] and values [T, G, Dv] of a two-map attention layer."""
    T = h.shape[0]
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[p + "k"].T).reshape(T, G * 2, D)
    k = rotate_halves(k, np.arange(T), *_rotation(m)).reshape(T, G, 2, D)
    v = (h @ w[p + "v"].T).reshape(T, G, Dv)
    return k, v


def diff_attention(h, w, p, m, eps, kv):
    """Two softmax maps per head over the same values, o = a1 - lam * a2, then unit RMS per head and (1 - diff)."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H * 2, D)
    q = rotate_halves(q, np.arange(T), *_rotation(m)).reshape(T, H, 2, D)
    k, v = kv
    lam = np.exp(np.sum(w[p + "lq1"] * w[p + "lk1"])) - np.exp(np.sum(w[p + "lq2"] * w[p + "lk2"])) + m["diff"]
    mask = block_mask(T, m["mask"]["size"] if m.get("mask") else T)
    out = np.zeros((T, H, Dv))
    for hh in range(H):
        g = hh // (H // G)
        a1 = masked_attention(q[:, hh, 0], k[:, g, 0], v[:, g], m["scale"], mask)
        a2 = masked_attention(q[:, hh, 1], k[:, g, 1], v[:, g], m["scale"], mask)
        out[:, hh] = rms_unit(a1 - lam * a2, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def normed_attention(h, w, p, m, eps):
    """Attention without positions: whole-row RMS norms of q and k, a factor per head on the scores."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (rms_unit(h @ w[p + "q"].T, eps) * w[p + "q.norm"]).reshape(T, H, D)
    k = (rms_unit(h @ w[p + "k"].T, eps) * w[p + "k.norm"]).reshape(T, G, D)
    v = (h @ w[p + "v"].T).reshape(T, G, Dv)
    mask = block_mask(T, m["mask"]["size"] if m.get("mask") else T)
    out = np.zeros((T, H, Dv))
    for hh in range(H):
        g = hh // (H // G)
        out[:, hh] = masked_attention(q[:, hh], k[:, g], v[:, g], m["scale"] * float(w[p + "temp"][hh]), mask)
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def general_delta(h, w, p, m, eps, state=None):
    """Per head a state S [D, D]:  S <- diag(d) S - (a*u)(u^T S) + k v^T  (both terms from the old S),  o = S^T r,
    with d = exp(-exp(-1/2) * sigmoid(.)) per key channel, a = sigmoid(.) and u the unit key."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ w[p + "r"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, D)
    d = np.exp(-np.exp(-0.5) * sigmoid(np.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).reshape(T, H, D)
    a = sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).reshape(T, H, D)
    u = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    S = np.zeros((H, D, D)) if state is None else state
    o = np.zeros((T, H, D))
    for t in range(T):
        for hh in range(H):
            old = S[hh]
            S[hh] = d[t, hh][:, None] * old - np.outer(a[t, hh] * u[t, hh], u[t, hh] @ old) + np.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ r[t, hh]
    o = rms_unit(o, eps).reshape(T, H * D) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def feed_forward(h, w, p):
    z = np.maximum(h @ w[p + "up"].T + w[p + "up.b"], 0.0)
    return (z * z) @ w[p + "down"].T + w[p + "down.b"]


# ----------------------------------------------------------------------------- the model

def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after every layer."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    made = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rms_unit(x, eps) * w[p + "norm1"]
        h = time_conv_add(h, w[p + "canon1"])
        if layer["type"] == "general_delta":
            x = x + general_delta(h, w, p + "mix.", m, eps)
        elif layer["type"] == "attention":
            if m.get("kv_from") is None:
                made[i] = keys_values_diff(h, w, p + "mix.", m)
                kv = made[i]
            else:
                kv = made[m["kv_from"]]
            x = x + diff_attention(h, w, p + "mix.", m, eps, kv)
        elif layer["type"] == "attention_2":
            x = x + normed_attention(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        if layer["mlp"] is not None:
            x = x + feed_forward(rms_unit(x, eps) * w[p + "norm2"], w, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.copy())
    return (rms_unit(x, eps) * w["final.norm"]) @ w["head"].T


def generate_greedy(cfg, w, prompt, n_new):
    """The ``n_new`` tokens a greedy loop appends to ``prompt`` (first maximum wins), recomputing everything each time."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(np.argmax(forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]
