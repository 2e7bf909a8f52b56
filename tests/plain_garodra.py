"""A plain, slow implementation of the Garodra decoder: the oracle of its tests.

Whole sequences, no cache, no batching, numpy only, float64 by default, one function per
mechanism.  It shares no code with the library (the model folder is read with the few lines
of ``plain_llama.read_safetensors``, which is test code as well).

Notation: ``x`` is the residual stream [T, W]; a matrix is stored [out, in] and applied as
``x @ M.T``; ``T`` tokens at positions 0..T-1.

The design, restated:

* embedding: row of the table times ``embedding.scale``;
* every norm is a Dynamic Tanh, y = tanh(alpha x) * w + b (no statistics);
* a layer is x += post1(mixer(pre1(x))), then, if it has a feed-forward, x += post2(ff(pre2(x)));
* mixers: a gated delta rule with short convolutions, or attention through a low-rank latent
  with one shared rotated key part;
* feed-forwards: a gated dense one (tanh GELU) or routed experts (SiLU) with the softmax taken over
  the chosen experts' logits only;
* a span of layers may run several times over with the same weights; every pass but the first adds
  the embedding output again, and every pass adds its own learned vector, before its first layer.
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

def dyt(x, w, prefix):
    """Dynamic Tanh: tanh(alpha * x) * weight + bias."""
    return np.tanh(float(w[prefix + ".alpha"]) * x) * w[prefix] + w[prefix + ".b"]


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return np.logaddexp(0.0, z)


def softmax(z):
    z = z - np.max(z, axis=-1, keepdims=True)
    e = np.exp(z)
    return e / np.sum(e, axis=-1, keepdims=True)


def rotate_pairs(v, positions, base, dims):
    """Neighbouring pairs (2i, 2i+1) of the first ``dims`` entries of the last axis turned by the angle
    position * base^(-2i/dims); the rest passes.  v: [T, ..., D]."""
    out = np.array(v, dtype=v.dtype, copy=True)
    i = np.arange(dims // 2)
    freq = np.asarray(base, dtype=np.float64) ** (-2.0 * i / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]         # [T, dims/2]
    shape = (v.shape[0],) + (1,) * (v.ndim - 2) + (dims // 2,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def causal_conv(x, taps_w):
    """Per-channel causal convolution over time.  x [T, C], taps_w [C, K]; the last column multiplies the
    current token, the one before it the token before, and so on; zeros before the start."""
    T, C = x.shape
    K = taps_w.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C), dtype=x.dtype), x], axis=0)
    out = np.zeros_like(x)
    for j in range(K):
        out += padded[j:j + T] * taps_w[:, j][None, :]
    return out


# ----------------------------------------------------------------------------- mixers

def delta_mixer(h, w, p, m, eps):
    """Gated delta rule.  h [T, W]; ``p`` the tensor prefix ('l3.mix'); ``m`` the mixer's sizes."""
    T = h.shape[0]
    H, Hk, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + ".q"].T, w[p + ".q.conv"])).reshape(T, Hk, D)
    k = silu(causal_conv(h @ w[p + ".k"].T, w[p + ".k.conv"])).reshape(T, Hk, D)
    v = silu(causal_conv(h @ w[p + ".v"].T, w[p + ".v.conv"])).reshape(T, H, Dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + ".b"].T)                                              # [T, H]
    decay = np.exp(-np.exp(w[p + ".A_log"])[None, :] * softplus(h @ w[p + ".a"].T + w[p + ".dt_bias"][None, :]))
    gate = silu(h @ w[p + ".g"].T).reshape(T, H, Dv)
    out = np.zeros((T, H, Dv), dtype=h.dtype)
    rep = H // Hk
    for hh in range(H):
        S = np.zeros((D, Dv), dtype=h.dtype)
        kh = hh // rep
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, kh])
            S = S + np.outer(k[t, kh], u)
            out[t, hh] = S.T @ q[t, kh]
    out = rms_unit(out, eps) * w[p + ".norm"][None, None, :] * gate
    return out.reshape(T, H * Dv) @ w[p + ".o"].T


def latent_attention_mixer(h, w, p, m, eps, positions):
    """Attention whose keys and values come from one low-rank latent per token plus one rotated key part
    that all heads share.  Written the long way round: every head's keys and values are made explicitly."""
    T = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_unit(h @ w[p + ".dq"].T, eps) * w[p + ".dq.norm"]
    q = (cq @ w[p + ".uq"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], positions, m["rot"]["base"], m["rot"]["dims"])
    down = h @ w[p + ".dkv"].T
    c = rms_unit(down[:, :C], eps) * w[p + ".dkv.norm"]
    k_rot = rotate_pairs(down[:, C:], positions, m["rot"]["base"], m["rot"]["dims"])   # [T, R], one for all heads
    k_plain = (c @ w[p + ".uk"].T).reshape(T, H, D)
    v = (c @ w[p + ".uv"].T).reshape(T, H, Dv)
    out = np.zeros((T, H, Dv), dtype=h.dtype)
    mask = np.tril(np.ones((T, T), dtype=bool))
    for hh in range(H):
        s = (q_plain[:, hh] @ k_plain[:, hh].T + q_rot[:, hh] @ k_rot.T) * m["scale"]
        s = np.where(mask, s, -np.inf)
        out[:, hh] = softmax(s) @ v[:, hh]
    return out.reshape(T, H * Dv) @ w[p + ".o"].T


# ----------------------------------------------------------------------------- feed-forwards

def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + ".gate"].T) * (h @ w[p + ".up"].T)) @ w[p + ".down"].T


def choose_experts(logits, top):
    """Indices of the ``top`` largest logits per row (ties: the lower index first) and the softmax over them."""
    order = np.argsort(-logits, axis=-1, kind="stable")[:, :top]
    chosen = np.take_along_axis(logits, order, axis=-1)
    return order, softmax(chosen)


def moe_ff(h, w, p, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, wt = choose_experts(h @ w[p + ".router"].T, top)
    out = np.zeros((h.shape[0], w[p + ".e0.down"].shape[0]), dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = f"{p}.e{int(idx[t, j])}"
            a = silu(h[t] @ w[e + ".gate"].T) * (h[t] @ w[e + ".up"].T)
            out[t] += wt[t, j] * (a @ w[e + ".down"].T)
    return out


# ----------------------------------------------------------------------------- the model

def layer_order(cfg):
    """[(layer index, pass number or None)] in run order, with the pass number set on the first layer of a pass."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["times"] <= 1 and False:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        for i in range(a, b):
            order.append((i, t if i == a else None))
    order += [(i, None) for i in range(b, n)]
    return order


def run_layer(x, w, i, layer, eps, positions):
    p = f"l{i}"
    h = dyt(x, w, p + ".norm1")
    if layer["type"] == "delta":
        y = delta_mixer(h, w, p + ".mix", layer["mixer"], eps)
    elif layer["type"] == "latent_attention":
        y = latent_attention_mixer(h, w, p + ".mix", layer["mixer"], eps, positions)
    else:
        raise ValueError(layer["type"])
    x = x + dyt(y, w, p + ".norm1b")
    mlp = layer.get("mlp")
    if mlp is not None:
        h = dyt(x, w, p + ".norm2")
        y = dense_ff(h, w, p + ".mlp") if mlp["kind"] == "dense" else moe_ff(h, w, p + ".mlp", mlp)
        x = x + dyt(y, w, p + ".norm2b")
    return x


def forward(cfg, w, tokens, dtype=np.float64, return_states=False):
    """Logits [T, vocab] of one whole sequence; with ``return_states`` also the stream after every layer run."""
    w = {k: np.asarray(v, dtype=dtype) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    positions = np.arange(len(tokens))
    x0 = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    x = x0.copy()
    states = []
    for i, t in layer_order(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t][None, :]
        x = run_layer(x, w, i, cfg["layers"][i], eps, positions)
        states.append(x.copy())
    logits = dyt(x, w, "final.norm") @ w["head"].T
    return (logits, states) if return_states else logits


def generate_greedy(cfg, w, prompt, max_new, dtype=np.float64):
    toks, out = list(prompt), []
    for _ in range(max_new):
        nxt = int(np.argmax(forward(cfg, w, toks, dtype)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
