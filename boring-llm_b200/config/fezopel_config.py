"""Typed configuration of the Fezopel decoder, read from its own config.json keys.

    {"architecture": "Fezopel", "vocab": V, "width": d, "norm": {"eps": e},
     "layers": [{"type": "attention" | "gla" | "channel_delta", "mixer": {...}, "mlp": {"kind": "dense", "ff": n} | null}, ...]}

Every size and every constant that can differ between models of the design is a field; a layer's mixer has the keys
of its type (see the three mixer classes). Sizes that only the tensors' shapes give (the inner sizes of the products
in two factors) are optional keys here, `rank` and `gate_rank`: a checkpoint needs none of them, the random-weights
mode does.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass, field
from typing import Optional, Tuple, Union

from .model_config import ConfigError, _get, _positive, architecture_name


@dataclass(frozen=True)
class AttentionMixerConfig:
    """'attention': grouped-query attention with a norm over the whole q and k projections, rotation of the first
    `rot_dims` dimensions of each head in interleaved pairs, a window of `window` positions (0: none), a sink per head
    and a gate per head."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int
    rot_base: float
    rot_dims: int
    scale: float

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "mask": {"size": self.window}, "rot": {"base": self.rot_base, "dims": self.rot_dims}, "scale": self.scale}


@dataclass(frozen=True)
class GlaMixerConfig:
    """'gla': gated linear attention, decay sigmoid(z)^(1 / tau) per key channel."""
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int] = None

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.rank is not None:
            d["rank"] = self.rank
        return d


@dataclass(frozen=True)
class ChannelDeltaMixerConfig:
    """'channel_delta': the gated delta rule with a decay per head and key channel and short convolutions of `conv` taps."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    rank: Optional[int] = None
    gate_rank: Optional[int] = None

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.rank is not None:
            d["rank"] = self.rank
        if self.gate_rank is not None:
            d["gate_rank"] = self.gate_rank
        return d


MixerConfig = Union[AttentionMixerConfig, GlaMixerConfig, ChannelDeltaMixerConfig]


@dataclass(frozen=True)
class FezopelLayerConfig:
    type: str
    mixer: MixerConfig
    ff: int = 0                  # hidden size of the dense feed-forward, 0: the layer has none

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": {"kind": "dense", "ff": self.ff} if self.ff else None}


def _optional_rank(m: dict, key: str) -> Optional[int]:
    return _positive(key, _get(m, key, int)) if m.get(key) is not None else None


def _mixer(kind: str, m: dict, where: str) -> MixerConfig:
    heads = _positive(f"{where}.heads", _get(m, "heads", int))
    dim = _positive(f"{where}.dim", _get(m, "dim", int))
    vdim = _positive(f"{where}.vdim", _get(m, "vdim", int, dim))
    if kind == "attention":
        kv = _positive(f"{where}.kv_heads", _get(m, "kv_heads", int, heads))
        if heads % kv != 0:
            raise ConfigError(f"config.json: {where}: {heads} heads cannot share {kv} key/value heads")
        mask = m.get("mask") or {}
        window = _get(mask, "size", int, 0)
        if window < 0:
            raise ConfigError(f"config.json: {where}.mask.size must not be negative, got {window}")
        rot = m.get("rot") or {}
        rot_dims = _get(rot, "dims", int, 0)
        if rot_dims < 0 or rot_dims % 2 != 0 or rot_dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims ({rot_dims}) must be even and at most the head size {dim}")
        base = _get(rot, "base", float, 10000.0)
        if not base > 0:
            raise ConfigError(f"config.json: {where}.rot.base must be positive, got {base}")
        return AttentionMixerConfig(heads, kv, dim, vdim, window, float(base), rot_dims, float(_get(m, "scale", float, dim ** -0.5)))
    if kind == "gla":
        tau = _get(m, "tau", float)
        if not tau > 0:
            raise ConfigError(f"config.json: {where}.tau must be positive, got {tau}")
        return GlaMixerConfig(heads, dim, vdim, float(tau), _optional_rank(m, "rank"))
    if kind == "channel_delta":
        kv = _positive(f"{where}.kv_heads", _get(m, "kv_heads", int, heads))
        if heads % kv != 0:
            raise ConfigError(f"config.json: {where}: {heads} heads cannot share {kv} query/key heads")
        conv = _positive(f"{where}.conv", _get(m, "conv", int))
        return ChannelDeltaMixerConfig(heads, kv, dim, vdim, conv, _optional_rank(m, "rank"), _optional_rank(m, "gate_rank"))
    raise ConfigError(f"config.json: {where}: unknown layer type {kind!r} (attention, gla, channel_delta)")


@dataclass(frozen=True)
class FezopelConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    layers: Tuple[FezopelLayerConfig, ...]
    max_position_embeddings: int = 1 << 20      # the design has no position limit of its own; engines clamp to their cache
    eos_token_ids: Tuple[int, ...] = ()
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    ARCHITECTURES = ("Fezopel",)

    @classmethod
    def from_dict(cls, d: dict) -> "FezopelConfig":
        arch = architecture_name(d)
        vocab = _positive("vocab", _get(d, "vocab", int))
        width = _positive("width", _get(d, "width", int))
        eps = _get(_get(d, "norm", dict), "eps", float)
        if not eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        entries = _get(d, "layers", list)
        if not entries:
            raise ConfigError("config.json: 'layers' lists no layer")
        layers = []
        for i, e in enumerate(entries):
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = _get(e, "type", str)
            mixer = _mixer(kind, _get(e, "mixer", dict), f"layers[{i}].mixer")
            ff = 0
            mlp = e.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: layers[{i}].mlp must be an object or null")
                if _get(mlp, "kind", str, "dense") != "dense":
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind {mlp['kind']!r} is not supported (only 'dense')")
                ff = _positive(f"layers[{i}].mlp.ff", _get(mlp, "ff", int))
            layers.append(FezopelLayerConfig(kind, mixer, ff))
        known = {"architecture", "architectures", "model_type", "vocab", "width", "norm", "layers", "max_position_embeddings",
                 "eos_token_id"}
        unknown = sorted(k for k in d if k not in known and not k.startswith("_"))
        if unknown:
            warnings.warn(f"config.json: keys not used by {arch}: {', '.join(unknown)}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(x) for x in eos))
        return cls(architecture=arch, vocab_size=vocab, width=width, norm_eps=float(eps), layers=tuple(layers),
                   max_position_embeddings=_positive("max_position_embeddings", _get(d, "max_position_embeddings", int, 1 << 20)),
                   eos_token_ids=eos_ids, raw=dict(d))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": [l.to_dict() for l in self.layers]}
        if self.max_position_embeddings != 1 << 20:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
