"""Feed-forward ``routed_experts``: a mixture of small gated feed-forwards of which every token runs a few.

Router logits z = W_r h in fp32; the ``top`` experts with the largest logits are chosen (ties: the lower index) and
weighted by the softmax over the CHOSEN logits only; the output is the weighted sum of the chosen experts' outputs,
each W_down (act(W_gate h) * (W_up h)) without biases, summed in the order of the choice.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from .registry import TensorDecl, part


@part("ffn", "routed_experts")
class RoutedExperts:
    """params: ``width``, ``inner`` (of one expert), ``experts``, ``top``, optional ``activation`` (default ``silu``).
    tensors: ``router`` [experts, width] and per expert i ``e<i>.gate``, ``e<i>.up`` [inner, width], ``e<i>.down``
    [width, inner]."""
    takes_padding_rows = True       # the router marks token rows of no sequence; they get zeros
    stores_output = True

    @classmethod
    def declare(cls, spec):
        p = spec.params
        W, F = p["width"], p["inner"]
        d = {}
        for i in range(p["experts"]):
            d.update({f"e{i}.gate": TensorDecl((F, W)), f"e{i}.up": TensorDecl((F, W)), f"e{i}.down": TensorDecl((W, F))})
        d["router"] = TensorDecl((p["experts"], W))
        return d

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self.width, self.inner, self.E, self.top = int(p["width"]), int(p["inner"]), int(p["experts"]), int(p["top"])
        if not (1 <= self.top <= self.E):
            raise ValueError("routed_experts: top must be between 1 and the number of experts")
        activation = p.get("activation", "silu")
        if activation not in kernels.ACTIVATIONS:
            raise ValueError(f"routed_experts: unknown activation {activation!r}")
        self.act = kernels.ACTIVATIONS[activation]
        self.w_router = rt.to_compute(tensors["router"])
        self.w_gate = rt.to_compute(torch.stack([tensors[f"e{i}.gate"] for i in range(self.E)]))
        self.w_up = rt.to_compute(torch.stack([tensors[f"e{i}.up"] for i in range(self.E)]))
        self.w_down = rt.to_compute(torch.stack([tensors[f"e{i}.down"] for i in range(self.E)]))

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_router, self.w_gate, self.w_up, self.w_down))

    def forward(self, h, x, ctx, store: bool = False) -> bool:
        T = h.shape[0]
        rt = self.rt
        logits = rt.scratch("router_logits", (T, self.E), torch.float32)
        kernels.linear(h, self.w_router, logits, None, kernels.OUT_STORE_F32)
        idx = rt.scratch("router_choice", (T, self.top), torch.int32)
        wt = rt.scratch("router_weight", (T, self.top), torch.float32)
        kernels.moe_route(logits, self.top, ctx, idx, wt)
        y = x if store else rt.scratch("experts_out", tuple(x.shape), torch.float32)
        if kernels.moe_grouped_applies(h, self.width, self.inner, self.E):
            kernels.moe_experts_grouped(h, self.w_gate, self.w_up, self.w_down, idx, wt, self.act, rt, y)
        else:
            a = rt.scratch("experts_act", (T, self.top, self.inner), torch.float32)
            kernels.moe_experts_streamed(h, self.w_gate, self.w_up, self.w_down, idx, wt, self.act, a, y)
        if not store:
            x += y
        return False
