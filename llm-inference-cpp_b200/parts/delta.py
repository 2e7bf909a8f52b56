"""Mixer ``delta``: the gated delta rule, a recurrent layer with a matrix state per head.

Per token, from the layer's input h: q, k (``kv_heads`` heads of ``dim``) and v (``heads`` heads of ``vdim``) by
projections without bias, each then through a short causal convolution over time (per channel, ``conv`` taps, no
bias) and silu; q and k made unit vectors per head (q also times dim^-1/2); a write strength beta = sigmoid(W_b h)
and a decay g = exp(-exp(A_log) * softplus(W_a h + dt_bias)) per head.  Query/key head of head h: h // (heads /
kv_heads).  Per head, in this order:

    S <- g S;   u = beta (v - Sᵀ k);   S <- S + k uᵀ;   o = Sᵀ q

then o / rms(o) (over vdim) * weight * silu(W_g h), and W_o.  The state of a sequence — S [heads, dim, vdim] and the
last conv-1 inputs of the convolution, all fp32 — lives in the cache's state slab (S column by column), zero at the start; everything
behind the projections is fp32 (csrc/delta_rule.cu).
"""
from __future__ import annotations

import torch

from ..cache.storage import StateRequest
from ..ops import kernels
from .registry import FreeDim, TensorDecl, part


@part("mixer", "delta")
class GatedDeltaRule:
    """params: ``width``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` (taps), ``eps`` (of the output's RMS norm).
    tensors: ``q``, ``k`` [kv_heads*dim, width], ``v`` [heads*vdim, width], ``q.conv``, ``k.conv``, ``v.conv`` [channels,
    conv], ``b``, ``a`` [heads, width], ``A_log``, ``dt_bias`` [heads], ``g`` [heads*vdim, width], ``norm`` [vdim],
    ``o`` [width, heads*vdim]."""
    stores_output = True

    @classmethod
    def declare(cls, spec):
        p = spec.params
        W, H, Hk, D, Dv, K = p["width"], p["heads"], p["kv_heads"], p["dim"], p["vdim"], p["conv"]
        return {"q": TensorDecl((Hk * D, W)), "q.conv": TensorDecl((Hk * D, K)), "k": TensorDecl((Hk * D, W)),
                "k.conv": TensorDecl((Hk * D, K)), "v": TensorDecl((H * Dv, W)), "v.conv": TensorDecl((H * Dv, K)),
                "b": TensorDecl((H, W)), "A_log": TensorDecl((H,), "bias"), "norm": TensorDecl((Dv,), "norm_scale"),
                "a": TensorDecl((H, W)), "dt_bias": TensorDecl((H,), "bias"), "g": TensorDecl((H * Dv, W)),
                "o": TensorDecl((W, H * Dv))}

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self.width, self.H, self.Hk = int(p["width"]), int(p["heads"]), int(p["kv_heads"])
        self.D, self.Dv, self.taps, self.eps = int(p["dim"]), int(p["vdim"]), int(p["conv"]), float(p["eps"])
        if self.H % self.Hk:
            raise ValueError("delta: heads must be a multiple of kv_heads")
        self.dims = (self.H, self.Hk, self.D, self.Dv, self.taps)
        self.n_conv = 2 * self.Hk * self.D + self.H * self.Dv
        # one product for all six projections: rows [q | k | v | b | a | gate]
        self.w_in = rt.to_compute(torch.cat([tensors[n] for n in ("q", "k", "v", "b", "a", "g")], dim=0))
        self.conv_w = rt.to_f32(torch.cat([tensors[n + ".conv"] for n in ("q", "k", "v")], dim=0))
        self.a_log, self.dt_bias = rt.to_f32(tensors["A_log"]), rt.to_f32(tensors["dt_bias"])
        self.w_norm = rt.to_f32(tensors["norm"])
        self.w_o = rt.to_compute(tensors["o"])
        self.state_floats = kernels.delta_state_floats(*self.dims)

    def cache_request(self):
        return StateRequest((self.state_floats,), torch.float32)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    @property
    def takes_padding_rows(self) -> bool:
        return True          # every kernel skips token rows and sequences of no slot

    def forward(self, h, x, ctx, binding, store: bool = False) -> bool:
        T = h.shape[0]
        rt, H, Dv = self.rt, self.H, self.Dv
        n_in = self.n_conv + 2 * H + H * Dv
        proj = rt.scratch("delta_proj", (T, n_in), torch.float32)
        kernels.linear(h, self.w_in, proj, None, kernels.OUT_STORE_F32)
        prep = rt.scratch("delta_prep", (T, self.n_conv + 2 * H), torch.float32)
        o_raw = rt.scratch("delta_o", (T, H * Dv), torch.float32)
        state = binding.group.data[binding.index]
        kernels.delta_step(proj, self.dims, self.conv_w, self.a_log, self.dt_bias, state, ctx, prep, o_raw,
                           write_state=binding.writes)
        heads = rt.scratch("attn_out", (T, H * Dv))
        kernels.delta_finish(o_raw, proj[:, self.n_conv + 2 * H:], self.w_norm, self.eps, H, Dv, ctx, heads)
        kernels.linear(heads, self.w_o, x, None, kernels.OUT_STORE_F32 if store else kernels.OUT_ADD_F32)
        return False


@part("mixer", "general_delta")
class GeneralDeltaRule:
    """The delta rule with a decay per key channel and a removal along the unit key.  Per token, from the layer's input
    h: r, k, v (``heads`` heads of ``dim``) by projections without bias; a decay per head and key channel through a
    low-rank path, d = exp(-exp(-1/2) * sigmoid(W2 tanh(W1 h) + w0)); a removal rate a = sigmoid(Wa h + a.b); the unit
    key u = k / sqrt(sum(k^2) + 1e-6).  Per head, both new terms read the old state:

        S <- diag(d) S - (a * u) (uᵀ S) + k vᵀ ;    o = Sᵀ r

    then o / rms(o) per head, times ``norm`` (a weight per entry of all heads), times sigmoid(Wg h), and W_o.  S
    [heads, dim, dim] lives in the cache's state slab (fp32, column by column, zero at the start); everything behind
    the projections is fp32 (csrc/dplr_delta.cu).

    params: ``width``, ``heads``, ``dim``, ``eps`` (of the output's RMS norm), optional ``rank`` (the low-rank path's
    size where random weights are drawn; a file's own size is read from its tensors).
    tensors: ``r``, ``k``, ``v``, ``a``, ``g`` [heads*dim, width], ``a.b``, ``w0``, ``norm`` [heads*dim], ``w1`` [rank,
    width], ``w2`` [heads*dim, rank], ``o`` [width, heads*dim]."""
    stores_output = True
    WALK_MAX_TOKENS = 16     # up to here the decay's low-rank path is walked inside the preparing kernel; beyond, a product

    @classmethod
    def declare(cls, spec):
        p = spec.params
        W, N = p["width"], p["heads"] * p["dim"]
        R = FreeDim(int(p.get("rank") or max(1, W // 16)))
        d = {n: TensorDecl((N, W)) for n in ("r", "k", "v", "a", "g")}
        d.update({"a.b": TensorDecl((N,), "bias"), "w0": TensorDecl((N,), "bias"), "norm": TensorDecl((N,), "norm_scale"),
                  "w1": TensorDecl((R, W)), "w2": TensorDecl((N, R)), "o": TensorDecl((W, N))})
        return d

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self.width, self.H, self.D, self.eps = int(p["width"]), int(p["heads"]), int(p["dim"]), float(p["eps"])
        self.R = int(tensors["w1"].shape[0])
        if tensors["w2"].shape[1] != self.R:
            raise ValueError(f"general_delta: w1 has {self.R} rows but w2 has {tensors['w2'].shape[1]} columns")
        # one product for all projections: rows [r | k | v | a | gate | low-rank path]
        self.w_in = rt.to_compute(torch.cat([tensors[n] for n in ("r", "k", "v", "a", "g", "w1")], dim=0))
        self.w2t = rt.to_f32(tensors["w2"]).t().contiguous()          # [rank, heads*dim]: for a handful of tokens, walked in the kernel
        self.w2 = rt.to_compute(tensors["w2"])                        # for many tokens: a product of its own
        self.w0, self.a_bias = rt.to_f32(tensors["w0"]), rt.to_f32(tensors["a.b"])
        self.w_norm = rt.to_f32(tensors["norm"])
        self.w_o = rt.to_compute(tensors["o"])

    def cache_request(self):
        return StateRequest((self.H * self.D * self.D,), torch.float32)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.w2t))

    @property
    def takes_padding_rows(self) -> bool:
        return True          # every kernel skips token rows and sequences of no slot

    defers_norm = True       # the output projection can fill the norm behind the mixer (``then_norm``)

    def forward(self, h, x, ctx, binding, store: bool = False, then_norm=None) -> bool:
        T = h.shape[0]
        rt, H, D = self.rt, self.H, self.D
        N = H * D
        proj = rt.scratch("delta_proj", (T, 5 * N + self.R), torch.float32)
        kernels.linear(h, self.w_in, proj, None, kernels.OUT_STORE_F32)
        prep = rt.scratch("delta_prep", (T, 3 * N), torch.float32)
        z = None
        if T > self.WALK_MAX_TOKENS:
            low = rt.scratch("delta_low", (T, self.R))
            kernels.tanh_rows(proj[:, 5 * N:], low)
            z = rt.scratch("delta_z", (T, N), torch.float32)
            kernels.linear(low, self.w2, z, None, kernels.OUT_STORE_F32)
        kernels.gdelta_prepare(proj, H, D, D, self.w2t, self.w0, self.a_bias, ctx, prep, z)
        o_raw = rt.scratch("delta_o", (T, N), torch.float32)
        kernels.dplr_recurrence(proj, prep, H, D, D, binding.group.data[binding.index], ctx, o_raw, write_state=binding.writes)
        heads = rt.scratch("attn_out", (T, N))
        kernels.delta_finish(o_raw, proj[:, 4 * N:5 * N], self.w_norm, self.eps, H, D, ctx, heads, kernels.GATE_SIGMOID)
        if store:
            kernels.linear(heads, self.w_o, x, None, kernels.OUT_STORE_F32)
            return False
        return kernels.linear(heads, self.w_o, x, None, kernels.OUT_ADD_F32, then_norm)
