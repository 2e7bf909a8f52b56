"""Feed-forward parts.  ``swiglu``: x += (act(h·Wgᵀ) ⊙ (h·Wuᵀ))·Wdᵀ, no biases, act = silu
(src/model/transformer.cpp:288-292; silu(z) = z / (1 + exp(-z)), src/model/kernels.cpp:148) unless the
parameter ``activation`` names another one (``gelu_tanh``: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z³)))).
Gate and up are stored as one matrix [gate; up] so that one product serves both."""
from __future__ import annotations

import torch

from ..ops import kernels
from .registry import TensorDecl, part


@part("ffn", "swiglu")
class SwiGLU:
    """params: ``width``, ``inner``, optional ``activation`` (``silu``, ``gelu_tanh``), optional ``names`` (the local
    tensor names of gate, up and down; default ``gate_proj.weight`` and so on)."""
    takes_padding_rows = True       # token rows of no sequence (a step padded to a shape) do no harm: rows are treated alone
    stores_output = True            # forward(..., store=True) overwrites x instead of adding to it
    DEFAULT_NAMES = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")

    @classmethod
    def declare(cls, spec):
        w, f = spec.params["width"], spec.params["inner"]
        g, u, d = spec.params.get("names", cls.DEFAULT_NAMES)
        return {g: TensorDecl((f, w)), u: TensorDecl((f, w)), d: TensorDecl((w, f))}

    def __init__(self, spec, tensors, rt, **_):
        self.rt = rt
        self.width, self.inner = int(spec.params["width"]), int(spec.params["inner"])
        g_name, u_name, d_name = spec.params.get("names", self.DEFAULT_NAMES)
        gate, up = tensors[g_name], tensors[u_name]
        activation = spec.params.get("activation", "silu")
        if activation not in kernels.ACTIVATIONS:
            raise ValueError(f"swiglu: unknown activation {activation!r} (known: {sorted(kernels.ACTIVATIONS)})")
        self.act = kernels.ACTIVATIONS[activation]
        # The tensor-core product can finish silu(gate)·up itself when gate and up rows alternate;
        # otherwise the rows are [gate; up] and a gating kernel follows the product.
        self.fused_gate = (rt.dtype == torch.bfloat16 and self.width % 8 == 0 and not kernels._FORCE_SIMT
                           and self.act in kernels.FUSED_GATE_MODES)
        if self.fused_gate:
            self.w_gate_up = rt.to_compute(torch.stack([gate, up], dim=1).reshape(2 * self.inner, self.width))
        else:
            self.w_gate_up = rt.to_compute(torch.cat([gate, up], dim=0))
        self.w_down = rt.to_compute(tensors[d_name])

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    defers_norm = True

    def forward(self, h, x, ctx, then_norm=None, store: bool = False) -> bool:
        T = h.shape[0]
        act = self.rt.scratch("ffn_act", (T, self.inner))
        if self.fused_gate and kernels.gemm_tc_eligible(getattr(h, "h", h), self.w_gate_up):
            kernels.gemm_bf16(h, self.w_gate_up, act, None, kernels.FUSED_GATE_MODES[self.act])
        else:
            if self.fused_gate:
                raise kernels.KernelError("swiglu: activations are not aligned for the tensor-core product")
            gate_up = self.rt.scratch("ffn_gate_up", (T, 2 * self.inner))
            kernels.linear(h, self.w_gate_up, gate_up)
            kernels.swiglu(gate_up, act, self.act)
        return kernels.linear(act, self.w_down, x, None, kernels.OUT_STORE_F32 if store else kernels.OUT_ADD_F32, then_norm)


@part("ffn", "mlp")
class DenseMLP:
    """x += act(h·Wuᵀ + bu)·Wdᵀ + bd: a feed-forward without a gate.  params: ``width``, ``inner``, ``activation`` (``relu2``:
    the square of relu), optional ``bias`` (default True), optional ``names`` (the local names of the two matrices,
    default ``up`` and ``down``; a bias is its matrix's name + ``.b``)."""
    takes_padding_rows = True       # rows are treated alone
    stores_output = True

    @classmethod
    def declare(cls, spec):
        w, f = spec.params["width"], spec.params["inner"]
        u, d = spec.params.get("names", ("up", "down"))
        out = {u: TensorDecl((f, w)), d: TensorDecl((w, f))}
        if spec.params.get("bias", True):
            out.update({u + ".b": TensorDecl((f,), "bias"), d + ".b": TensorDecl((w,), "bias")})
        return out

    def __init__(self, spec, tensors, rt, **_):
        self.rt = rt
        self.width, self.inner = int(spec.params["width"]), int(spec.params["inner"])
        u, d = spec.params.get("names", ("up", "down"))
        activation = spec.params.get("activation", "relu2")
        if activation not in kernels.PLAIN_ACTIVATIONS:
            raise ValueError(f"mlp: unknown activation {activation!r} (known: {sorted(kernels.PLAIN_ACTIVATIONS)})")
        self.act = kernels.PLAIN_ACTIVATIONS[activation]
        self.w_up, self.w_down = rt.to_compute(tensors[u]), rt.to_compute(tensors[d])
        bias = spec.params.get("bias", True)
        self.b_up = rt.to_f32(tensors[u + ".b"]) if bias else None
        self.b_down = rt.to_f32(tensors[d + ".b"]) if bias else None

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down))

    defers_norm = True       # takes a deferred norm as its input, and its down projection can fill the next one

    def forward(self, h, x, ctx, then_norm=None, store: bool = False) -> bool:
        T = h.shape[0]
        act = self.rt.scratch("ffn_act", (T, self.inner))
        kernels.linear(h, self.w_up, act, self.b_up, kernels.PLAIN_ACTIVATION_MODES[self.act])      # the activation rides on the product
        if store:
            kernels.linear(act, self.w_down, x, self.b_down, kernels.OUT_STORE_F32)
            return False
        return kernels.linear(act, self.w_down, x, self.b_down, kernels.OUT_ADD_F32, then_norm)
