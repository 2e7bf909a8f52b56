"""Typed configuration of the Fusazen decoder.

config.json names the design with ``"architecture": "Fusazen"`` and gives every size and every constant that can
differ between models of the design:

* ``vocab``, ``width``; ``embedding.scale``; ``norm.eps`` (of every RMS norm); ``canon.taps`` (taps of the short
  convolution ahead of every mixer);
* ``layers``: a list, one entry per layer, with ``type`` (``general_delta``, ``attention`` or ``attention_2``), ``mixer``
  (that mixer's sizes) and ``mlp`` (``null`` for a layer without a feed-forward, else ``kind`` ``dense`` with ``ff``).
  An ``attention`` mixer may name with ``kv_from`` an earlier layer of its kind whose keys and values it reads.

Nothing here has a default that stands in for a missing size: a missing or ill-typed key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .garodra import _number, _obj, _uint
from .llama import MAX_LAYERS, MAX_VOCAB, ConfigError

ARCHITECTURE = "Fusazen"
MAX_TAPS = 16


@dataclass(frozen=True)
class DeltaSizes:
    heads: int
    dim: int
    rank: int = 0            # 0: not given (a file's tensors decide; random weights take a default)


@dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int               # positions per block of the mask (0: no mask beyond causality)
    diff: float = 0.0        # (two-map attention only)
    rot_base: float = 0.0
    rot_dims: int = 0
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class FusazenLayer:
    type: str                # "general_delta" | "attention" | "attention_2"
    mixer: Any
    ff: int                  # 0: no feed-forward


@dataclass(frozen=True)
class FusazenConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    taps: int
    layers: tuple
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, root: Mapping[str, Any]) -> "FusazenConfig":
        vocab = _uint(root, "vocab", "", MAX_VOCAB)
        width = _uint(root, "width", "")
        scale = _number(_obj(root, "embedding", ""), "scale", "embedding.", positive=False)
        eps = _number(_obj(root, "norm", ""), "eps", "norm.")
        taps = _uint(_obj(root, "canon", ""), "taps", "canon.", MAX_TAPS)
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
            if kind == "general_delta":
                mixer = DeltaSizes(heads=_uint(m, "heads", mw), dim=_uint(m, "dim", mw),
                                   rank=_uint(m, "rank", mw) if m.get("rank") is not None else 0)
            elif kind in ("attention", "attention_2"):
                heads, kv_heads = _uint(m, "heads", mw), _uint(m, "kv_heads", mw)
                if heads % kv_heads:
                    raise ConfigError(f'config: {mw}"heads" is not a multiple of "kv_heads"')
                # a mixer without "mask" (or with null) sees all earlier positions; one without "rot" is not rotated
                chunk = _uint(_obj(m, "mask", mw), "size", mw + "mask.", 1 << 30) if m.get("mask") is not None else 0
                common = dict(heads=heads, kv_heads=kv_heads, dim=_uint(m, "dim", mw), vdim=_uint(m, "vdim", mw),
                              scale=_number(m, "scale", mw), chunk=chunk)
                if kind == "attention":
                    rot = _obj(m, "rot", mw) if m.get("rot") is not None else {"dims": 0, "base": 1.0}
                    rot_dims = _uint(rot, "dims", mw + "rot.", least=0)
                    if rot_dims % 2 or rot_dims > common["dim"]:
                        raise ConfigError(f'config: {mw}rot."dims" must be even and at most "dim"')
                    kv_from = m.get("kv_from")
                    if kv_from is not None:
                        kv_from = _uint(m, "kv_from", mw, MAX_LAYERS, least=0)
                        src = layers[kv_from] if kv_from < i else None
                        if src is None or src.type != "attention" or src.mixer.kv_from is not None:
                            raise ConfigError(f'config: {mw}"kv_from" must name an earlier "attention" layer with keys and '
                                              f'values of its own')
                        s = src.mixer
                        if (s.kv_heads, s.dim, s.vdim) != (kv_heads, common["dim"], common["vdim"]):
                            raise ConfigError(f'config: {mw}"kv_from": layer {kv_from} keeps keys and values of other sizes')
                    diff = _number(m, "diff", mw, positive=False)
                    mixer = AttentionSizes(**common, diff=diff, rot_base=_number(rot, "base", mw + "rot."), rot_dims=rot_dims,
                                           kv_from=kv_from)
                else:
                    mixer = AttentionSizes(**common)
            else:
                raise ConfigError(f'config: {where}"type" must be "general_delta", "attention" or "attention_2", not {kind!r}')
            mlp = entry.get("mlp")
            ff = 0
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f'config: {where}"mlp" must be an object or null')
                if mlp.get("kind") != "dense":
                    raise ConfigError(f'config: {where}mlp."kind" must be "dense"')
                ff = _uint(mlp, "ff", where + "mlp.")
            layers.append(FusazenLayer(kind, mixer, ff))
        return cls(vocab=vocab, width=width, embedding_scale=scale, norm_eps=eps, taps=taps, layers=tuple(layers))
