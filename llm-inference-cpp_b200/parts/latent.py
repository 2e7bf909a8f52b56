"""Mixer ``latent_attention``: causal attention whose keys and values come from one low-rank latent per token.

Per token the layer computes, from its input h:

* a query latent, RMS-normed, expanded to H heads of ``dim`` plain + ``rot_dim`` rotated entries;
* a key/value latent c of rank ``kv_rank``, RMS-normed, and ONE rotated key part r of ``rot_dim`` entries that all heads
  share (not normed);
* head h's key is [Uk_h c | r], its value Uv_h c; score = (q_plain . Uk_h c + q_rot . r) * scale; softmax; W_o.

Only [c | r] is cached: one row of kv_rank + rot_dim entries per token (a key-only cache group with one head).  The
expansions are folded into the query and the output, (Uk_hᵀ q_plain) . c and Uv_h (Σ p c), so that attention runs over
the cached rows directly, the same way for a prompt and for a single token.  Norms, scores, softmax and the rotation's
angles are fp32; the rotation pairs neighbouring entries (2i, 2i+1) with angle pos * base^(-2i/dims).
"""
from __future__ import annotations

import numpy as np
import torch

from ..cache.storage import KVRequest
from ..ops import kernels
from .registry import TensorDecl, part


@part("mixer", "latent_attention")
class LatentAttention:
    """params: ``width``, ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``q_rank``, ``scale``, ``rot_base``,
    ``rot_dims`` (how many of the rot_dim entries are rotated), ``eps`` (of the two RMS norms).
    tensors: ``dq`` [q_rank, width], ``dq.norm`` [q_rank], ``uq`` [heads*(dim+rot_dim), q_rank], ``dkv`` [kv_rank+rot_dim,
    width], ``dkv.norm`` [kv_rank], ``uk`` [heads*dim, kv_rank], ``uv`` [heads*vdim, kv_rank], ``o`` [width, heads*vdim]."""
    stores_output = True

    @classmethod
    def declare(cls, spec):
        p = spec.params
        W, H, D, R, Dv, C, Q = p["width"], p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"], p["q_rank"]
        return {"dq": TensorDecl((Q, W)), "dq.norm": TensorDecl((Q,), "norm_scale"), "uq": TensorDecl((H * (D + R), Q)),
                "dkv": TensorDecl((C + R, W)), "dkv.norm": TensorDecl((C,), "norm_scale"), "uk": TensorDecl((H * D, C)),
                "uv": TensorDecl((H * Dv, C)), "o": TensorDecl((W, H * Dv))}

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self.width, self.H, self.D, self.R = int(p["width"]), int(p["heads"]), int(p["dim"]), int(p["rot_dim"])
        self.Dv, self.C, self.Q = int(p["vdim"]), int(p["kv_rank"]), int(p["q_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.rot_dims = int(p.get("rot_dims", self.R))
        if self.rot_dims % 2 or self.rot_dims > self.R:
            raise ValueError("latent_attention: rot_dims must be even and at most rot_dim")
        i = np.arange(self.rot_dims // 2, dtype=np.float64)
        inv = np.power(np.float64(p["rot_base"]), -2.0 * i / max(self.rot_dims, 1)).astype(np.float32)
        self.inv_freq = torch.from_numpy(inv if inv.size else np.zeros(1, np.float32)).to(rt.device)
        # one product for both down-projections: rows [query latent | kv latent | shared key part]
        self.w_down = rt.to_compute(torch.cat([tensors["dq"], tensors["dkv"]], dim=0))
        self.w_qnorm, self.w_cnorm = rt.to_f32(tensors["dq.norm"]), rt.to_f32(tensors["dkv.norm"])
        self.w_uq = rt.to_compute(tensors["uq"])
        # per head: Uk_hᵀ [C, D] (folded into the query) and Uv_h [Dv, C] (applied to the context)
        self.w_uk_t = rt.to_compute(tensors["uk"].reshape(self.H, self.D, self.C).transpose(1, 2).contiguous())
        self.w_uv = rt.to_compute(tensors["uv"].reshape(self.H, self.Dv, self.C).contiguous())
        self.w_o = rt.to_compute(tensors["o"])

    def cache_request(self):
        return KVRequest(1, self.C + self.R, 0, values=False)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_down, self.w_uq, self.w_uk_t, self.w_uv, self.w_o))

    @property
    def takes_padding_rows(self) -> bool:
        return True          # every kernel skips token rows of no sequence

    def forward(self, h, x, ctx, binding, store: bool = False) -> bool:
        T = h.shape[0]
        rt, H, D, R, C, Q, Dv = self.rt, self.H, self.D, self.R, self.C, self.Q, self.Dv
        g = binding.group
        pages = ctx.pages_of(g)
        cache = g.k[binding.index]
        down = rt.scratch("latent_down", (T, Q + C + R), torch.float32)
        kernels.linear(h, self.w_down, down, None, kernels.OUT_STORE_F32)
        cq = rt.scratch("latent_cq", (T, Q))
        kernels.latent_prepare(down, Q, C, R, self.w_qnorm, self.w_cnorm, self.eps, self.inv_freq, self.rot_dims, ctx, pages,
                               g.page_size, cache, cq, write_kv=binding.writes)
        q = rt.scratch("latent_q", (T, H * (D + R)))
        kernels.linear(cq, self.w_uq, q)
        qa = rt.scratch("latent_qa", (T, H * (C + R)))
        kernels.linear_batched(q, D + R, self.w_uk_t, qa, C + R, D)
        kernels.latent_q_rotate(q, D, qa, C, R, H, self.inv_freq, self.rot_dims, ctx)
        lat = rt.scratch("latent_ctx", (T, H * C))
        kernels.attention_latent(qa, lat, cache, ctx, pages, g.page_size, H, C, R, self.scale, rt=rt)
        heads = rt.scratch("attn_out", (T, H * Dv))
        kernels.linear_batched(lat, C, self.w_uv, heads, Dv, C)
        kernels.linear(heads, self.w_o, x, None, kernels.OUT_STORE_F32 if store else kernels.OUT_ADD_F32)
        return False
