"""Small Garodra configurations and weights for the tests: sizes unlike one another, and weights large enough
that every mechanism matters (the library's own random folders draw matrices at 0.02, which leaves a tanh norm in
its linear range and a router undecided)."""
import json
import os

import numpy as np


def att(heads, dim, rot_dim, vdim, kv_rank, q_rank, rot_dims=None, base=10000.0, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5),
            "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(width, vocab, layers, loop=None, scale=2.0, eps=1e-5):
    c = {"architecture": "Garodra", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
         "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# one mechanism at a time
ATT_ONLY = config(48, 97, [("latent_attention", att(3, 20, 12, 10, 24, 16, rot_dims=8), None)])
DELTA_ONLY = config(40, 83, [("delta", delta(4, 2, 24, 20, 4), None)])
DELTA_REG = config(64, 90, [("delta", delta(2, 2, 64, 48, 2), None)])          # the state's columns in registers
DENSE_ONLY = config(32, 61, [("delta", delta(1, 1, 16, 16, 1), dense(72))])     # one tap: a convolution that is a scale
MOE_ONLY = config(56, 120, [("latent_attention", att(2, 16, 8, 16, 16, 24), moe(40, 5, 2))])
MOE_ALL = config(32, 50, [("latent_attention", att(1, 8, 4, 8, 8, 8), moe(24, 3, 3)),      # every expert chosen
                          ("delta", delta(2, 1, 8, 8, 3), moe(16, 6, 1))])                 # one expert chosen
# loops: layers ahead of the span, in it and behind it; a span of one layer; a span run once
LOOPED = config(48, 101, [("delta", delta(2, 1, 16, 24, 3), dense(64)),
                          ("latent_attention", att(4, 12, 8, 12, 20, 28), moe(32, 4, 2)),
                          ("delta", delta(3, 3, 20, 12, 5), None),
                          ("latent_attention", att(2, 24, 16, 8, 32, 12, rot_dims=16, base=500.0), dense(80))],
                loop=(1, 3, 3), scale=1.5)
LOOP_ONE = config(32, 64, [("latent_attention", att(2, 8, 8, 8, 12, 12), dense(48))], loop=(0, 1, 4))
LOOP_ONCE = config(32, 64, [("delta", delta(2, 2, 32, 16, 2), None), ("latent_attention", att(2, 8, 8, 8, 12, 12), None)],
                   loop=(0, 2, 1))
# sizes of the kind the fast kernels take (multiples of 64), several layers
WIDE = config(128, 300, [("latent_attention", att(4, 64, 32, 64, 128, 64), dense(256)),
                         ("delta", delta(4, 2, 128, 64, 4), moe(128, 8, 3)),
                         ("latent_attention", att(8, 32, 32, 32, 64, 64), moe(64, 4, 2)),
                         ("delta", delta(2, 1, 64, 128, 3), dense(192))], loop=(0, 2, 2), scale=1.0)
# sizes that fit no fast kernel: rows of odd byte counts, head counts that divide nothing, a rotation of two entries
ODD = config(36, 77, [("delta", delta(3, 3, 12, 10, 2), moe(10, 3, 2)),
                      ("latent_attention", att(5, 6, 4, 7, 10, 9, rot_dims=2, base=77.0), dense(22)),
                      ("latent_attention", att(1, 10, 0, 3, 6, 5), None)], loop=(0, 2, 2), scale=0.7, eps=1e-4)      # the last: no rotated part at all
CONFIGS = {"odd": ODD, "att": ATT_ONLY, "delta": DELTA_ONLY, "delta_reg": DELTA_REG, "dense": DENSE_ONLY, "moe": MOE_ONLY,
           "moe_all": MOE_ALL, "looped": LOOPED, "loop_one": LOOP_ONE, "loop_once": LOOP_ONCE, "wide": WIDE}


def make_weights(cfg, seed, keep_state=False):
    """name -> float32 array.  ``keep_state``: decays next to one and strong writes, so that a state that is lost or
    cut anywhere changes everything after it."""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]
    w = {}

    def mat(name, out, inp, gain=1.0):
        w[name] = (rng.standard_normal((out, inp)) * gain / np.sqrt(inp)).astype(np.float32)

    def norm(name, n=W):
        w[name] = (1.0 + 0.2 * rng.standard_normal(n)).astype(np.float32)
        w[name + ".b"] = (0.2 * rng.standard_normal(n)).astype(np.float32)
        w[name + ".alpha"] = np.float32(rng.uniform(0.4, 1.2))

    w["embed"] = rng.standard_normal((V, W)).astype(np.float32)
    mat("head", V, W, 2.0)
    norm("final.norm")
    if "loop" in cfg:
        w["loop.step"] = (0.5 * rng.standard_normal((cfg["loop"]["times"], W))).astype(np.float32)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        norm(p + "norm1")
        norm(p + "norm1b")
        if layer["type"] == "latent_attention":
            H, D, R, Dv, C, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            mat(p + "mix.dq", Q, W)
            w[p + "mix.dq.norm"] = (1.0 + 0.2 * rng.standard_normal(Q)).astype(np.float32)
            mat(p + "mix.uq", H * (D + R), Q, 3.0)
            mat(p + "mix.dkv", C + R, W, 2.0)
            w[p + "mix.dkv.norm"] = (1.0 + 0.2 * rng.standard_normal(C)).astype(np.float32)
            mat(p + "mix.uk", H * D, C, 2.0)
            mat(p + "mix.uv", H * Dv, C)
            mat(p + "mix.o", W, H * Dv)
        else:
            H, Hk, D, Dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", Hk * D), ("k", Hk * D), ("v", H * Dv)):
                mat(p + "mix." + n, rows, W, 2.0)
                w[p + f"mix.{n}.conv"] = (rng.standard_normal((rows, K)) / np.sqrt(K)).astype(np.float32)
            mat(p + "mix.b", H, W, 2.0)
            mat(p + "mix.a", H, W)
            if keep_state:
                w[p + "mix.A_log"] = np.full(H, -9.0, dtype=np.float32)
                w[p + "mix.b"] += 0.0
            else:
                w[p + "mix.A_log"] = np.log(rng.uniform(0.05, 2.0, H)).astype(np.float32)
            w[p + "mix.dt_bias"] = rng.standard_normal(H).astype(np.float32)
            w[p + "mix.norm"] = (1.0 + 0.2 * rng.standard_normal(Dv)).astype(np.float32)
            mat(p + "mix.g", H * Dv, W, 2.0)
            mat(p + "mix.o", W, H * Dv)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        norm(p + "norm2")
        norm(p + "norm2b")
        if mlp["kind"] == "dense":
            mat(p + "mlp.gate", mlp["ff"], W, 2.0)
            mat(p + "mlp.up", mlp["ff"], W)
            mat(p + "mlp.down", W, mlp["ff"])
        else:
            F = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                mat(p + f"mlp.e{e}.gate", F, W, 2.0)
                mat(p + f"mlp.e{e}.up", F, W)
                mat(p + f"mlp.e{e}.down", W, F, 1.0 + e)          # experts that differ in size as well
            mat(p + "mlp.router", mlp["router"]["experts"], W, 3.0)
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
