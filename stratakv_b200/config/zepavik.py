"""Typed configuration of the Zepavik decoder, read from its ``config.json``.

The file names the design under ``architecture`` and nests its sizes::

    {"architecture": "Zepavik", "vocab": V, "width": W, "max_positions": P, "logit_scale": s,
     "norm": {"eps": e},
     "embedding": {"bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": c, "mask": {"size": w}},
                 "mlp": {"kind": "dense", "ff": F} | null}, ...]}

Every size and every constant that differs between models of the design comes from there; layers may differ
from one another in all of their numbers.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError, _need, _optional

ARCHITECTURE = "Zepavik"
MIXERS = ("attention",)
MLP_KINDS = ("dense",)


def _section(raw: Mapping[str, Any], key: str, where: str, required: bool = True) -> Optional[Mapping[str, Any]]:
    value = raw.get(key)
    if value is None:
        if required:
            raise ConfigError(f"config.json: {where}'{key}' is missing")
        return None
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return value


def _positive(value: int, what: str) -> int:
    if value <= 0:
        raise ConfigError(f"config.json: {what} must be positive, got {value}")
    return value


@dataclass(frozen=True)
class ZepavikBigram:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class ZepavikLayer:
    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                    # mask.size; 0: no mask beyond the causal one
    ff: int                        # 0: the layer has no feed-forward
    mlp_kind: str = "dense"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], index: int) -> "ZepavikLayer":
        where = f"layers[{index}]."
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: layers[{index}] must be an object")
        kind = _need(raw, "type", str)
        if kind not in MIXERS:
            raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design ({', '.join(MIXERS)})")
        mixer = _section(raw, "mixer", where)
        heads = _positive(_need(mixer, "heads", int), where + "mixer.heads")
        kv_heads = _positive(_optional(mixer, "kv_heads", int, heads), where + "mixer.kv_heads")
        if heads % kv_heads != 0:
            raise ConfigError(f"config.json: {where}mixer.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        dim = _positive(_need(mixer, "dim", int), where + "mixer.dim")
        vdim = _positive(_optional(mixer, "vdim", int, dim), where + "mixer.vdim")
        mask = _section(mixer, "mask", where + "mixer.", required=False)
        window = _optional(mask, "size", int, 0) if mask is not None else 0
        if window < 0:
            raise ConfigError(f"config.json: {where}mixer.mask.size must not be negative")
        mlp = _section(raw, "mlp", where, required=False)
        ff, mlp_kind = 0, "dense"
        if mlp is not None:
            mlp_kind = _optional(mlp, "kind", str, "dense")
            if mlp_kind not in MLP_KINDS:
                raise ConfigError(f"config.json: {where}mlp.kind '{mlp_kind}' is not a feed-forward of this design")
            ff = _positive(_need(mlp, "ff", int), where + "mlp.ff")
        return cls(kind, heads, kv_heads, dim, vdim, _need(mixer, "scale", float), window, ff, mlp_kind)

    def to_dict(self) -> dict:
        mixer = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.window:
            mixer["mask"] = {"size": self.window}
        return {"type": self.type, "mixer": mixer,
                "mlp": {"ff": self.ff, "kind": self.mlp_kind} if self.ff else None}


@dataclass(frozen=True)
class ZepavikConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    logit_scale: float
    bigram: Optional[ZepavikBigram]
    layers: Tuple[ZepavikLayer, ...]
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZepavikConfig":
        vocab = _positive(_need(raw, "vocab", int), "vocab")
        width = _positive(_need(raw, "width", int), "width")
        max_positions = _positive(_need(raw, "max_positions", int), "max_positions")
        norm = _section(raw, "norm", "")
        bigram = None
        embedding = _section(raw, "embedding", "", required=False)
        pair = _section(embedding, "bigram", "embedding.", required=False) if embedding is not None else None
        if pair is not None:
            bigram = ZepavikBigram(_positive(_need(pair, "buckets", int), "embedding.bigram.buckets"),
                                   _need(pair, "mul_prev", int), _need(pair, "mul_cur", int))
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        return cls(vocab, width, max_positions, _need(norm, "eps", float), _optional(raw, "logit_scale", float, 1.0),
                   bigram, tuple(ZepavikLayer.from_dict(layer, i) for i, layer in enumerate(layers)))

    def to_dict(self) -> dict:
        raw = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "max_positions": self.max_positions, "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.bigram is not None:
            raw["embedding"] = {"bigram": {"buckets": self.bigram.buckets, "mul_prev": self.bigram.mul_prev,
                                           "mul_cur": self.bigram.mul_cur}}
        return raw
