"""The Garodra decoder as a recipe of parts.

Embedding rows times a constant; layers of the arrangement ``prepost`` (a Dynamic Tanh norm ahead of and behind each
sublayer); a mixer per layer, ``latent_attention`` or ``delta``; a feed-forward per layer, gated dense with the tanh
GELU, routed experts with silu, or none; a span of layers that may run several times with the same weights, each pass
with a cache or state of its own and a ``loop_pass`` entry ahead of its first layer; a last Dynamic Tanh and an untied
head.  Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.step``, and per layer i ``l<i>.norm1`` (ahead of the
mixer), ``l<i>.norm1b`` (behind it), ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from ..config.garodra import ARCHITECTURE, GarodraConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 24        # the design sets no limit: positions are angles computed on the fly, and a state has no length


def _mixer(c: GarodraConfig, layer, prefix: str) -> PartSpec:
    m = layer.mixer
    if layer.type == "latent_attention":
        return PartSpec("latent_attention", {
            "width": c.width, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
            "q_rank": m.q_rank, "scale": m.scale, "rot_base": m.rot_base, "rot_dims": m.rot_dims, "eps": c.norm_eps}, prefix)
    return PartSpec("delta", {"width": c.width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
                              "conv": m.conv, "eps": c.norm_eps}, prefix)


def _ffn(c: GarodraConfig, mlp, prefix: str) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("swiglu", {"width": c.width, "inner": mlp.ff, "activation": "gelu_tanh",
                                   "names": ("gate", "up", "down")}, prefix)
    return PartSpec("routed_experts", {"width": c.width, "inner": mlp.ff, "experts": mlp.experts, "top": mlp.top,
                                       "activation": "silu"}, prefix)


def garodra_model_spec(c: GarodraConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("dyt", {"width": c.width}, name)
    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        more = [("mixer_post", "norm", norm(p + "norm1b"))]
        if layer.mlp is not None:
            more.append(("ffn_post", "norm", norm(p + "norm2b")))
        layers.append(LayerSpec(
            block="prepost", mixer_norm=norm(p + "norm1"), mixer=_mixer(c, layer, p + "mix."),
            ffn_norm=norm(p + "norm2") if layer.mlp is not None else None,
            ffn=_ffn(c, layer.mlp, p + "mlp.") if layer.mlp is not None else None, more=tuple(more)))
    n = len(c.layers)
    schedule = [ScheduleEntry(i) for i in range(c.loop_start if c.has_loop else n)]
    if c.has_loop:
        for t in range(c.loop_times):
            for i in range(c.loop_start, c.loop_stop):
                before = None
                if i == c.loop_start:
                    before = PartSpec("loop_pass", {"width": c.width, "passes": c.loop_times, "index": t}, "loop.")
                schedule.append(ScheduleEntry(i, before=before))
        schedule += [ScheduleEntry(i) for i in range(c.loop_stop, n)]
    return ModelSpec(
        architecture=c.architecture, vocab_size=c.vocab, width=c.width, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_table", {"vocab": c.vocab, "width": c.width, "scale": c.embedding_scale,
                                           "tensor": "embed"}, ""),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": c.vocab, "width": c.width, "tied": False, "tensor": "head"}, ""),
        stop_ids=())


register_architecture(Architecture(ARCHITECTURE, GarodraConfig.from_dict, garodra_model_spec))
