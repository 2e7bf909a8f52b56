"""Parts of the family ``conv``: something that reshapes a sublayer's input over time and keeps, per sequence, the
inputs it still needs.  Interface: ``cache_request() -> StateRequest | None`` and ``forward(h, ctx, binding) -> h'``
(same shape and type as ``h``; ``binding`` is the part's own place in the cache's state slab).  Optional:
``forward_from_stream(x, norm, ctx, binding) -> h' | None`` — the norm ahead and the part in one kernel where that
exists.

``causal_add``:  h'[t] = h[t] + sum_j w[:, j] * h[t - (taps-1) + j]  per channel, zeros before a sequence's start, no
bias.  The last taps-1 inputs of a sequence are its state (fp32, zero when a slot is handed out); the sum is fp32
(csrc/short_conv.cu).
"""
from __future__ import annotations

import os

import torch

from ..cache.storage import StateRequest
from ..ops import kernels
from .registry import TensorDecl, part


_FUSE = os.environ.get("LLMI_FUSE_CONV", "1") != "0"      # 0: the norm ahead always as a kernel of its own (for measurements)


@part("conv", "causal_add")
class CausalConvAdd:
    """params: ``width``, ``taps``.  tensors (the prefix is the tensor's full name): ``""`` [width, taps]."""
    takes_padding_rows = True       # rows of no sequence get zeros and touch no state

    @classmethod
    def declare(cls, spec):
        return {"": TensorDecl((spec.params["width"], spec.params["taps"]))}

    def __init__(self, spec, tensors, rt, **_):
        self.rt = rt
        self.width, self.taps = int(spec.params["width"]), int(spec.params["taps"])
        if self.taps < 1:
            raise ValueError("causal_add: needs at least one tap")
        self.weight = rt.to_f32(tensors[""]).t().contiguous()        # [taps, width]: neighbouring channels side by side
        self._no_state = None

    def cache_request(self):
        return StateRequest((max(self.taps - 1, 1) * self.width,), torch.float32)

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward_from_stream(self, x, norm, ctx, binding):
        """The norm ahead and this part in one kernel, where that exists: a step in which every sequence brings one
        token, behind an RMS norm with a weight.  Returns h', or None (then the caller runs the norm and :meth:`forward`)."""
        if not (_FUSE and ctx.decode and getattr(norm, "kind", None) == "rms" and norm.width == self.width):
            return None
        out = self.rt.scratch("conv_out", (x.shape[0], self.width))
        kernels.norm_conv_token(x, norm.weight, norm.eps, self.weight, binding.group.data[binding.index], ctx, out)
        return out

    def forward(self, h, ctx, binding):
        out = self.rt.scratch("conv_out", tuple(h.shape), h.dtype)
        kernels.conv_add(h, self.weight, binding.group.data[binding.index], ctx, out)
        return out
