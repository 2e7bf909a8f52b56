"""What a pass over a looped span of layers adds to the stream ahead of its first layer.

A model may run a span of its layers several times in a row with the same weights (each pass keeps a cache or
state of its own: the schedule names the layer once per pass).  ``loop_pass`` is the part that marks the start of
pass ``index``: every pass but the first adds the embedding output again (the stream as it was before the first
layer of the model), and every pass then adds its own learned vector, row ``index`` of the table ``step``
[passes, width].  fp32, rows alone.
"""
from __future__ import annotations

from ..ops import kernels
from .registry import TensorDecl, part


@part("pass_entry", "loop_pass")
class LoopPass:
    """params: ``width``, ``passes``, ``index``, optional ``tensor`` (local name of the table; default ``step``)."""
    takes_padding_rows = True       # elementwise: rows are treated alone

    @classmethod
    def declare(cls, spec):
        return {spec.params.get("tensor", "step"): TensorDecl((spec.params["passes"], spec.params["width"]), "bias")}

    def __init__(self, spec, tensors, rt, **_):
        self.index = int(spec.params["index"])
        if not (0 <= self.index < int(spec.params["passes"])):
            raise ValueError("loop_pass: index out of range")
        table = rt.to_f32(tensors[spec.params.get("tensor", "step")])
        self.vector = table[self.index].contiguous()
        self.needs_embedding_output = self.index > 0

    def forward(self, x, x0, ctx) -> None:
        kernels.stream_add(x, x0 if self.needs_embedding_output else None, self.vector)
