"""Typed configuration of the Garodra decoder.

config.json names the design with ``"architecture": "Garodra"`` and gives every size and every constant that can
differ between models of the design:

* ``vocab``, ``width``; ``embedding.scale``; ``norm.eps`` (the eps of every RMS norm inside a mixer);
* ``layers``: a list, one entry per layer, with ``type`` (``delta`` or ``latent_attention``), ``mixer`` (that mixer's
  sizes) and ``mlp`` (``null`` for a layer without a feed-forward, else ``kind`` ``dense`` with ``ff``, or ``kind``
  ``moe`` with ``expert.ff``, ``router.experts`` and ``router.top``);
* ``loop`` (optional): layers ``start`` .. ``stop``-1 run ``times`` times in a row.

Nothing here has a default that stands in for a missing size: a missing or ill-typed key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .llama import MAX_DIM, MAX_LAYERS, MAX_VOCAB, ConfigError

ARCHITECTURE = "Garodra"


def _obj(root: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = root.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f'config: {where}"{key}" must be an object')
    return v


def _uint(root: Mapping[str, Any], key: str, where: str, limit: int = MAX_DIM, least: int = 1) -> int:
    v = root.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < least or v > limit:
        raise ConfigError(f'config: {where}"{key}" must be an integer in {least}..{limit}')
    return v


def _number(root: Mapping[str, Any], key: str, where: str, positive: bool = True) -> float:
    v = root.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f'config: {where}"{key}" must be a {"positive " if positive else ""}number')
    return float(v)


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class DeltaSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class FeedForwardSizes:
    kind: str                  # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class GarodraLayer:
    type: str                  # "latent_attention" | "delta"
    mixer: Any
    mlp: Optional[FeedForwardSizes]


@dataclass(frozen=True)
class GarodraConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, root: Mapping[str, Any]) -> "GarodraConfig":
        vocab = _uint(root, "vocab", "", MAX_VOCAB)
        width = _uint(root, "width", "")
        scale = _number(_obj(root, "embedding", ""), "scale", "embedding.", positive=False)
        eps = _number(_obj(root, "norm", ""), "eps", "norm.")
        raw = root.get("layers")
        if not isinstance(raw, list) or not raw or len(raw) > MAX_LAYERS:
            raise ConfigError(f'config: "layers" must be a list of 1..{MAX_LAYERS} layers')
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config: layers[{i}] must be an object")
            kind = entry.get("type")
            m = _obj(entry, "mixer", where)
            mw = where + "mixer."
            if kind == "latent_attention":
                rot = _obj(m, "rot", mw)
                rot_dim = _uint(m, "rot_dim", mw, least=0)
                rot_dims = _uint(rot, "dims", mw + "rot.", least=0)
                if rot_dims % 2 or rot_dims > rot_dim:
                    raise ConfigError(f'config: {mw}rot."dims" must be even and at most "rot_dim"')
                mixer = LatentAttentionSizes(
                    heads=_uint(m, "heads", mw), dim=_uint(m, "dim", mw), rot_dim=rot_dim, vdim=_uint(m, "vdim", mw),
                    kv_rank=_uint(m, "kv_rank", mw), q_rank=_uint(m, "q_rank", mw), scale=_number(m, "scale", mw),
                    rot_base=_number(rot, "base", mw + "rot."), rot_dims=rot_dims)
            elif kind == "delta":
                mixer = DeltaSizes(heads=_uint(m, "heads", mw), kv_heads=_uint(m, "kv_heads", mw), dim=_uint(m, "dim", mw),
                                   vdim=_uint(m, "vdim", mw), conv=_uint(m, "conv", mw, 16))
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f'config: {mw}"heads" is not a multiple of "kv_heads"')
            else:
                raise ConfigError(f'config: {where}"type" must be "latent_attention" or "delta", not {kind!r}')
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f'config: {where}"mlp" must be an object or null')
                fw = where + "mlp."
                if mlp.get("kind") == "dense":
                    mlp = FeedForwardSizes("dense", _uint(mlp, "ff", fw))
                elif mlp.get("kind") == "moe":
                    router = _obj(mlp, "router", fw)
                    experts = _uint(router, "experts", fw + "router.", 256)
                    top = _uint(router, "top", fw + "router.", 32)
                    if top > experts:
                        raise ConfigError(f'config: {fw}router."top" is larger than "experts"')
                    mlp = FeedForwardSizes("moe", _uint(_obj(mlp, "expert", fw), "ff", fw + "expert."), experts, top)
                else:
                    raise ConfigError(f'config: {fw}"kind" must be "dense" or "moe"')
            layers.append(GarodraLayer(kind, mixer, mlp))
        start, stop, times = 0, 0, 1
        loop = root.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError('config: "loop" must be an object or null')
            start = _uint(loop, "start", "loop.", len(layers), least=0)
            stop = _uint(loop, "stop", "loop.", len(layers), least=0)
            times = _uint(loop, "times", "loop.", 1024)
            if stop < start:
                raise ConfigError('config: loop."stop" is before loop."start"')
        return cls(vocab=vocab, width=width, embedding_scale=scale, norm_eps=eps, layers=tuple(layers),
                   loop_start=start, loop_stop=stop, loop_times=times)

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start
