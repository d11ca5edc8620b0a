"""Typed configuration of the Povusun decoder, read from its ``config.json``.

The file names the design under ``architecture`` and lists its layers, each with its own mixer and sizes::

    {"architecture": "Povusun", "vocab": V, "width": W, "norm": {"eps": e}, "token_side": {"dim": s} | absent,
     "layers": [
       {"type": "attention",
        "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": c, "softcap": cap,
                  "q_temp": {"coef": a, "every": n}, "kv_from": j},
        "mlp": {"kind": "dense", "ff": F, "limit": l} | null},
       {"type": "latent_attention", "mixer": {"heads": H, "dim": d, "vdim": dv, "kv_rank": r, "scale": c}, "mlp": ...},
       {"type": "rglru", "mixer": {"width": C, "blocks": B, "conv": taps}, "mlp": ...}]}

``softcap``, ``q_temp`` and ``kv_from`` may be absent (no cap, no temperature, keys and values of the layer's own).
Every size and every constant that differs between models of the design comes from there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError, _need, _optional
from .zepavik import _positive, _section

ARCHITECTURE = "Povusun"
MIXERS = ("attention", "latent_attention", "rglru")
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class PovusunMlp:
    ff: int
    limit: float
    kind: str = "dense"

    def to_dict(self) -> dict:
        return {"ff": self.ff, "kind": self.kind, "limit": self.limit}


@dataclass(frozen=True)
class PovusunLayer:
    """One layer.  Which fields count depends on ``type``: attention uses heads, kv_heads, dim, vdim, scale, softcap
    (0: none), q_temp_coef / q_temp_every (every 0: none) and kv_from (None: its own keys and values); latent
    attention heads, dim, vdim, kv_rank, scale; rglru channels, blocks, taps."""
    type: str
    mlp: Optional[PovusunMlp]
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    scale: float = 0.0
    softcap: float = 0.0
    q_temp_coef: float = 0.0
    q_temp_every: int = 0
    kv_from: Optional[int] = None
    kv_rank: int = 0
    channels: int = 0
    blocks: int = 0
    taps: int = 0

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], index: int) -> "PovusunLayer":
        where = f"layers[{index}]."
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: layers[{index}] must be an object")
        kind = _need(raw, "type", str)
        if kind not in MIXERS:
            raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design ({', '.join(MIXERS)})")
        mixer = _section(raw, "mixer", where)
        mlp_raw = _section(raw, "mlp", where, required=False)
        mlp = None
        if mlp_raw is not None:
            mlp_kind = _optional(mlp_raw, "kind", str, "dense")
            if mlp_kind not in MLP_KINDS:
                raise ConfigError(f"config.json: {where}mlp.kind '{mlp_kind}' is not a feed-forward of this design")
            mlp = PovusunMlp(_positive(_need(mlp_raw, "ff", int), where + "mlp.ff"),
                             _need(mlp_raw, "limit", float), mlp_kind)
            if not mlp.limit > 0.0:
                raise ConfigError(f"config.json: {where}mlp.limit must be positive, got {mlp.limit}")
        if kind == "rglru":
            channels = _positive(_need(mixer, "width", int), where + "mixer.width")
            blocks = _positive(_need(mixer, "blocks", int), where + "mixer.blocks")
            if channels % blocks != 0:
                raise ConfigError(f"config.json: {where}mixer.width ({channels}) must be a multiple of blocks ({blocks})")
            return cls(kind, mlp, channels=channels, blocks=blocks,
                       taps=_positive(_need(mixer, "conv", int), where + "mixer.conv"))
        heads = _positive(_need(mixer, "heads", int), where + "mixer.heads")
        dim = _positive(_need(mixer, "dim", int), where + "mixer.dim")
        vdim = _positive(_optional(mixer, "vdim", int, dim), where + "mixer.vdim")
        scale = _need(mixer, "scale", float)
        if kind == "latent_attention":
            return cls(kind, mlp, heads=heads, dim=dim, vdim=vdim, scale=scale,
                       kv_rank=_positive(_need(mixer, "kv_rank", int), where + "mixer.kv_rank"))
        kv_heads = _positive(_optional(mixer, "kv_heads", int, heads), where + "mixer.kv_heads")
        if heads % kv_heads != 0:
            raise ConfigError(f"config.json: {where}mixer.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        softcap = mixer.get("softcap")
        softcap = 0.0 if softcap is None else _need(mixer, "softcap", float)
        if softcap < 0.0:
            raise ConfigError(f"config.json: {where}mixer.softcap must not be negative")
        coef, every = 0.0, 0
        temp = _section(mixer, "q_temp", where + "mixer.", required=False)
        if temp is not None:
            coef = _need(temp, "coef", float)
            every = _positive(_need(temp, "every", int), where + "mixer.q_temp.every")
        kv_from = mixer.get("kv_from")
        if kv_from is not None:
            kv_from = _need(mixer, "kv_from", int)
            if not 0 <= kv_from < index:
                raise ConfigError(f"config.json: {where}mixer.kv_from ({kv_from}) must name an earlier layer")
        return cls(kind, mlp, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, softcap=softcap,
                   q_temp_coef=coef, q_temp_every=every, kv_from=kv_from)

    def to_dict(self) -> dict:
        if self.type == "rglru":
            mixer = {"blocks": self.blocks, "conv": self.taps, "width": self.channels}
        elif self.type == "latent_attention":
            mixer = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "scale": self.scale, "vdim": self.vdim}
        else:
            mixer = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
            if self.softcap:
                mixer["softcap"] = self.softcap
            if self.q_temp_every:
                mixer["q_temp"] = {"coef": self.q_temp_coef, "every": self.q_temp_every}
            if self.kv_from is not None:
                mixer["kv_from"] = self.kv_from
        return {"type": self.type, "mixer": mixer, "mlp": self.mlp.to_dict() if self.mlp is not None else None}


@dataclass(frozen=True)
class PovusunConfig:
    vocab: int
    width: int
    norm_eps: float
    side_dim: int                      # 0: no per-layer token input
    layers: Tuple[PovusunLayer, ...]
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "PovusunConfig":
        vocab = _positive(_need(raw, "vocab", int), "vocab")
        width = _positive(_need(raw, "width", int), "width")
        norm = _section(raw, "norm", "")
        side = _section(raw, "token_side", "", required=False)
        side_dim = _positive(_need(side, "dim", int), "token_side.dim") if side is not None else 0
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        parsed = tuple(PovusunLayer.from_dict(layer, i) for i, layer in enumerate(layers))
        for i, layer in enumerate(parsed):
            if layer.kv_from is None:
                continue
            source = parsed[layer.kv_from]
            if source.type != "attention" or source.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from names layer {layer.kv_from}, "
                                  "which has no keys and values of its own")
            if (source.kv_heads, source.dim, source.vdim) != (layer.kv_heads, layer.dim, layer.vdim):
                raise ConfigError(f"config.json: layers[{i}] uses the keys and values of layer {layer.kv_from} "
                                  "but differs from it in kv_heads, dim or vdim")
        return cls(vocab, width, _need(norm, "eps", float), side_dim, parsed)

    def to_dict(self) -> dict:
        raw = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers]}
        if self.side_dim:
            raw["token_side"] = {"dim": self.side_dim}
        return raw
