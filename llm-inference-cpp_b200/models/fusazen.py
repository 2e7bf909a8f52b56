"""The Fusazen decoder as a recipe of parts.

Embedding rows times a constant; layers of the arrangement ``prenorm`` with RMS norms and a short causal convolution
(``causal_add``) on what the mixer reads; a mixer per layer — ``general_delta``, ``diff_attention`` (rotated on the
first entries of every map, optionally on another layer's keys and values) or ``qk_normed_attention``, both kinds of
attention masked to blocks of positions —; a feed-forward per layer (``mlp`` with the square of relu and biases) or
none; a last RMS norm and an untied head.  Tensor names: ``embed``, ``head``, ``final.norm`` and per layer i
``l<i>.norm1``, ``l<i>.canon1``, ``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.mlp.*``.

A layer that reads layer j's keys and values becomes a scheduled call with ``cache_of`` = j: it writes nothing into
that cache and keeps only the convolution's state of its own.
"""
from __future__ import annotations

from ..config.fusazen import ARCHITECTURE, FusazenConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 24        # the design sets no limit: angles are computed on the fly, and a state has no length


def _mixer(c: FusazenConfig, layer, prefix: str) -> PartSpec:
    m = layer.mixer
    if layer.type == "general_delta":
        return PartSpec("general_delta", {"width": c.width, "heads": m.heads, "dim": m.dim, "eps": c.norm_eps,
                                          "rank": m.rank}, prefix)
    sizes = {"width": c.width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
             "eps": c.norm_eps, "chunk": m.chunk}
    if layer.type == "attention":
        position = (PartSpec("rotary_half", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base})
                    if m.rot_dims else PartSpec("none"))
        return PartSpec("diff_attention", {**sizes, "diff": m.diff, "shares_kv": m.kv_from is not None,
                                           "position": position}, prefix)
    return PartSpec("qk_normed_attention", sizes, prefix)


def fusazen_model_spec(c: FusazenConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("rms", {"width": c.width, "eps": c.norm_eps, "tensor": ""}, name)
    layers, schedule = [], []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        layers.append(LayerSpec(
            block="prenorm", mixer_norm=norm(p + "norm1"), mixer=_mixer(c, layer, p + "mix."),
            ffn_norm=norm(p + "norm2") if layer.ff else None,
            ffn=PartSpec("mlp", {"width": c.width, "inner": layer.ff, "activation": "relu2"}, p + "mlp.") if layer.ff else None,
            more=(("mixer_conv", "conv", PartSpec("causal_add", {"width": c.width, "taps": c.taps}, p + "canon1")),)))
        schedule.append(ScheduleEntry(i, cache_of=getattr(layer.mixer, "kv_from", None)))
    return ModelSpec(
        architecture=c.architecture, vocab_size=c.vocab, width=c.width, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_table", {"vocab": c.vocab, "width": c.width, "scale": c.embedding_scale,
                                           "tensor": "embed"}, ""),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": c.vocab, "width": c.width, "tied": False, "tensor": "head"}, ""),
        stop_ids=())


register_architecture(Architecture(ARCHITECTURE, FusazenConfig.from_dict, fusazen_model_spec))
