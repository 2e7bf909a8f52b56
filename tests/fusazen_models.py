"""Small Fusazen configurations and weights for the tests: sizes unlike one another (and unlike any model the
library ships numbers for), and weights large enough that every mechanism matters."""
import json
import os

import numpy as np


def delta(heads, dim, rank=None):
    m = {"heads": heads, "dim": dim}
    if rank is not None:
        m["rank"] = rank
    return m


def diff_att(heads, kv_heads, dim, vdim, chunk, rot_dims, base=10000.0, diff=0.5, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "mask": {"size": chunk},
         "rot": {"base": base, "dims": rot_dims}, "scale": float(scale if scale is not None else dim ** -0.5)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def normed_att(heads, kv_heads, dim, vdim, chunk, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
            "scale": float(scale if scale is not None else 1.0 / dim)}


def config(width, vocab, taps, layers, scale=2.0, eps=1e-5):
    return {"architecture": "Fusazen", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "canon": {"taps": taps},
            "layers": [{"type": t, "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}} for t, m, ff in layers]}


# one mechanism at a time
DELTA_ONLY = config(40, 83, 3, [("general_delta", delta(3, 12, rank=5), None)])              # a head size for the general kernel
DELTA_REG = config(64, 90, 2, [("general_delta", delta(2, 32, rank=8), None)])               # the state's columns in registers
DIFF_ONLY = config(48, 97, 4, [("attention", diff_att(4, 2, 12, 20, 37, 6, base=300.0, diff=0.3), None)])
NORMED_ONLY = config(36, 71, 1, [("attention_2", normed_att(3, 3, 10, 14, 50), None)])       # one tap: the convolution is a scale
MLP_ONLY = config(32, 61, 2, [("general_delta", delta(1, 8, rank=3), 72)])
# keys and values of another layer, with layers in between; a second pair behind it
SHARED = config(56, 120, 3, [("attention", diff_att(2, 1, 16, 24, 64, 16, diff=0.7), 40),
                             ("general_delta", delta(2, 16, rank=4), None),
                             ("attention", diff_att(2, 1, 16, 24, 20, 16, diff=0.2, kv_from=0), 48),
                             ("attention", diff_att(3, 3, 8, 8, 100, 0, diff=0.5), None),
                             ("attention_2", normed_att(4, 2, 8, 6, 33), 24),
                             ("attention", diff_att(3, 3, 8, 8, 7, 0, diff=0.4, kv_from=3), 16)], scale=1.5)
# all three mixers, blocks of positions that are no multiple of a cache page and smaller than one
MIXED = config(48, 101, 5, [("attention_2", normed_att(2, 1, 24, 12, 90), 64),
                            ("general_delta", delta(3, 16, rank=6), 80),
                            ("attention", diff_att(6, 2, 8, 16, 5, 4, base=77.0, diff=0.6), None),
                            ("general_delta", delta(1, 24, rank=2), 32)], eps=1e-4, scale=0.7)
# sizes of the kind the fast kernels take (multiples of 64), several layers
WIDE = config(128, 300, 4, [("attention", diff_att(4, 2, 64, 64, 128, 32), 256),
                            ("general_delta", delta(2, 64, rank=16), 192),
                            ("attention_2", normed_att(4, 4, 64, 64, 64), 128),
                            ("attention", diff_att(4, 2, 64, 64, 200, 32, kv_from=0), 256),
                            ("general_delta", delta(1, 128, rank=8), None),
                            ("attention_2", normed_att(8, 2, 32, 64, 256), 64)], scale=1.0)
# sizes that fit no fast kernel: rows of odd byte counts, head counts that divide nothing, a rotation of two entries
ODD = config(36, 77, 2, [("general_delta", delta(3, 10, rank=7), 10),
                         ("attention", diff_att(5, 5, 6, 7, 11, 2, base=50.0, diff=0.25), 22),
                         ("attention_2", normed_att(5, 1, 6, 9, 3), None)], scale=0.9, eps=1e-6)
CONFIGS = {"odd": ODD, "delta": DELTA_ONLY, "delta_reg": DELTA_REG, "diff": DIFF_ONLY, "normed": NORMED_ONLY, "mlp": MLP_ONLY,
           "shared": SHARED, "mixed": MIXED, "wide": WIDE}


def make_weights(cfg, seed, keep_state=False):
    """name -> float32 array.  ``keep_state``: decays next to one and weak removal, so that a state that is lost or cut
    anywhere changes everything after it."""
    rng = np.random.default_rng(seed)
    W, V, K = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    w = {}

    def mat(name, out, inp, gain=1.0):
        w[name] = (rng.standard_normal((out, inp)) * gain / np.sqrt(inp)).astype(np.float32)

    def vec(name, n, mean=0.0, std=1.0):
        w[name] = (mean + std * rng.standard_normal(n)).astype(np.float32)

    w["embed"] = rng.standard_normal((V, W)).astype(np.float32)
    mat("head", V, W, 2.0)
    vec("final.norm", W, 1.0, 0.2)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        vec(p + "norm1", W, 1.0, 0.2)
        w[p + "canon1"] = (rng.standard_normal((W, K)) / np.sqrt(K)).astype(np.float32)
        if layer["type"] == "general_delta":
            H, D = m["heads"], m["dim"]
            N, R = H * D, m.get("rank") or max(1, W // 16)
            for n, gain in (("r", 2.0), ("k", 2.0), ("v", 2.0), ("a", 1.0), ("g", 2.0)):
                mat(p + "mix." + n, N, W, gain)
            mat(p + "mix.w1", R, W, 2.0)
            mat(p + "mix.w2", N, R, 0.1 if keep_state else 2.0)
            vec(p + "mix.w0", N, -9.0 if keep_state else 0.0, 0.1 if keep_state else 1.0)
            vec(p + "mix.a.b", N, -6.0 if keep_state else 0.0, 0.1 if keep_state else 1.0)
            vec(p + "mix.norm", N, 1.0, 0.2)
            mat(p + "mix.o", W, N)
        else:
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            maps = 2 if layer["type"] == "attention" else 1
            mat(p + "mix.q", H * maps * D, W, 3.0)
            if m.get("kv_from") is None:
                mat(p + "mix.k", G * maps * D, W, 3.0)
                mat(p + "mix.v", G * Dv, W, 2.0)
            mat(p + "mix.o", W, H * Dv)
            if maps == 2:
                for n in ("lq1", "lk1", "lq2", "lk2"):
                    vec(p + "mix." + n, D, 0.0, 0.5 / np.sqrt(np.sqrt(D)))
            else:
                vec(p + "mix.q.norm", H * D, 1.0, 0.3)
                vec(p + "mix.k.norm", G * D, 1.0, 0.3)
                w[p + "mix.temp"] = rng.uniform(0.5, 3.0, H).astype(np.float32)
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            vec(p + "norm2", W, 1.0, 0.2)
            mat(p + "mlp.up", F, W, 2.0)
            vec(p + "mlp.up.b", F, 0.0, 0.5)
            mat(p + "mlp.down", W, F)
            vec(p + "mlp.down.b", W, 0.0, 0.3)
    return w


def write_model(folder, cfg, weights, storage="F32"):
    """config.json and model.safetensors; ``storage`` F32 or BF16.  Returns the weights as the file holds them."""
    import torch
    from llmi_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    dt = {"F32": torch.float32, "BF16": torch.bfloat16}[storage]
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(dt) for k, v in weights.items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    return {k: t.float().numpy().astype(np.float64) for k, t in tensors.items()}
