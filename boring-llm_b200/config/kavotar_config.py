"""Typed configuration of the Kavotar decoder, read from its own config.json keys.

    {"architecture": "Kavotar", "vocab": V, "width": d, "norm": {"eps": e}, "logit_softcap": c,
     "layers": [{"type": "mlstm" | "parallel", "mixer": {...}, "mlp": {"kind": "moe", ...} | null}, ...]}

    mlstm mixer:     {"heads", "dim", "vdim", "gate_cap"}
    parallel mixer:  {"left":  {"heads", "kv_heads", "dim", "vdim", "mask": {"size"}, "rot": {"base", "dims"}, "scale"},
                      "right": {"heads", "dim"}}
    mlp:             {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "groups": {"count", "keep"}}}

Every size and every constant that can differ between models of the design is a field. The inner size of the decay's
two factors in the right mixer is given by the tensors' shapes; `rank` is an optional key for the random-weights mode.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass, field
from typing import Optional, Tuple, Union

from .model_config import ConfigError, _get, _positive, architecture_name


@dataclass(frozen=True)
class MatrixMemoryConfig:
    """'mlstm': a matrix memory per head with exponential gates; `gate_cap` bounds the gates' pre-activations."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    """The left half of 'parallel': grouped-query attention inside chunks of `chunk` positions (0: none), q/k norm per
    head, rotation of the first `rot_dims` dimensions of each head in halves, a temperature per head, mixed heads."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    chunk: int
    rot_base: float
    rot_dims: int
    scale: float

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "mask": {"size": self.chunk},
                "rot": {"base": self.rot_base, "dims": self.rot_dims}, "scale": self.scale}


@dataclass(frozen=True)
class ShiftedRecurrenceConfig:
    """The right half of 'parallel': a linear recurrence with token-shifted inputs; keys and values of `dim` per head."""
    heads: int
    dim: int
    rank: Optional[int] = None

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim}
        if self.rank is not None:
            d["rank"] = self.rank
        return d


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: ChunkedAttentionConfig
    right: ShiftedRecurrenceConfig

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class RoutedExpertsConfig:
    """'moe': `experts` SwiGLU experts of hidden size `ff`, `top` a token, in `groups` runs of which `keep` stay open."""
    ff: int
    experts: int
    top: int
    groups: int = 1
    keep: int = 1

    def to_dict(self):
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "top": self.top, "groups": {"count": self.groups, "keep": self.keep}}}


@dataclass(frozen=True)
class KavotarLayerConfig:
    type: str
    mixer: Union[MatrixMemoryConfig, ParallelMixerConfig]
    mlp: Optional[RoutedExpertsConfig] = None

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp is not None else None}


def _heads(m: dict, where: str):
    heads = _positive(f"{where}.heads", _get(m, "heads", int))
    dim = _positive(f"{where}.dim", _get(m, "dim", int))
    return heads, dim


def _mixer(kind: str, m: dict, where: str):
    if kind == "mlstm":
        heads, dim = _heads(m, where)
        cap = _get(m, "gate_cap", float)
        if not cap > 0:
            raise ConfigError(f"config.json: {where}.gate_cap must be positive, got {cap}")
        return MatrixMemoryConfig(heads, dim, _positive(f"{where}.vdim", _get(m, "vdim", int, dim)), float(cap))
    if kind == "parallel":
        l, r = _get(m, "left", dict), _get(m, "right", dict)
        heads, dim = _heads(l, where + ".left")
        kv = _positive(f"{where}.left.kv_heads", _get(l, "kv_heads", int, heads))
        if heads % kv != 0:
            raise ConfigError(f"config.json: {where}.left: {heads} heads cannot share {kv} key/value heads")
        chunk = _get(l.get("mask") or {}, "size", int, 0)
        if chunk < 0:
            raise ConfigError(f"config.json: {where}.left.mask.size must not be negative, got {chunk}")
        rot = l.get("rot") or {}
        rot_dims = _get(rot, "dims", int, 0)
        if rot_dims < 0 or rot_dims % 2 != 0 or rot_dims > dim:
            raise ConfigError(f"config.json: {where}.left.rot.dims ({rot_dims}) must be even and at most the head size {dim}")
        base = _get(rot, "base", float, 10000.0)
        if not base > 0:
            raise ConfigError(f"config.json: {where}.left.rot.base must be positive, got {base}")
        left = ChunkedAttentionConfig(heads, kv, dim, _positive(f"{where}.left.vdim", _get(l, "vdim", int, dim)), chunk,
                                      float(base), rot_dims, float(_get(l, "scale", float, dim ** -0.5)))
        rh, rd = _heads(r, where + ".right")
        rank = _positive(f"{where}.right.rank", _get(r, "rank", int)) if r.get("rank") is not None else None
        return ParallelMixerConfig(left, ShiftedRecurrenceConfig(rh, rd, rank))
    raise ConfigError(f"config.json: {where}: unknown layer type {kind!r} (mlstm, parallel)")


def _mlp(mlp, where: str) -> Optional[RoutedExpertsConfig]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where} must be an object or null")
    if _get(mlp, "kind", str, "moe") != "moe":
        raise ConfigError(f"config.json: {where}.kind {mlp['kind']!r} is not supported (only 'moe')")
    ff = _positive(f"{where}.expert.ff", _get(_get(mlp, "expert", dict), "ff", int))
    router = _get(mlp, "router", dict)
    experts = _positive(f"{where}.router.experts", _get(router, "experts", int))
    top = _positive(f"{where}.router.top", _get(router, "top", int))
    groups = router.get("groups") or {}
    count = _positive(f"{where}.router.groups.count", _get(groups, "count", int, 1))
    keep = _positive(f"{where}.router.groups.keep", _get(groups, "keep", int, count))
    if experts % count != 0 or keep > count:
        raise ConfigError(f"config.json: {where}.router: {experts} experts in {count} groups of which {keep} are kept")
    if top > keep * (experts // count):
        raise ConfigError(f"config.json: {where}.router: {top} experts a token, but only {keep * (experts // count)} can be chosen")
    return RoutedExpertsConfig(ff, experts, top, count, keep)


@dataclass(frozen=True)
class KavotarConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    logit_softcap: float
    layers: Tuple[KavotarLayerConfig, ...]
    max_position_embeddings: int = 1 << 20      # the design has no position limit of its own; engines clamp to their cache
    eos_token_ids: Tuple[int, ...] = ()
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    ARCHITECTURES = ("Kavotar",)

    @classmethod
    def from_dict(cls, d: dict) -> "KavotarConfig":
        arch = architecture_name(d)
        vocab = _positive("vocab", _get(d, "vocab", int))
        width = _positive("width", _get(d, "width", int))
        eps = _get(_get(d, "norm", dict), "eps", float)
        if not eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        cap = _get(d, "logit_softcap", float, 0.0)
        if cap < 0:
            raise ConfigError(f"config.json: logit_softcap must not be negative, got {cap}")
        entries = _get(d, "layers", list)
        if not entries:
            raise ConfigError("config.json: 'layers' lists no layer")
        layers = []
        for i, e in enumerate(entries):
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = _get(e, "type", str)
            layers.append(KavotarLayerConfig(kind, _mixer(kind, _get(e, "mixer", dict), f"layers[{i}].mixer"),
                                             _mlp(e.get("mlp"), f"layers[{i}].mlp")))
        known = {"architecture", "architectures", "model_type", "vocab", "width", "norm", "layers", "logit_softcap",
                 "max_position_embeddings", "eos_token_id"}
        unknown = sorted(k for k in d if k not in known and not k.startswith("_"))
        if unknown:
            warnings.warn(f"config.json: keys not used by {arch}: {', '.join(unknown)}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(x) for x in eos))
        return cls(architecture=arch, vocab_size=vocab, width=width, norm_eps=float(eps), logit_softcap=float(cap),
                   layers=tuple(layers),
                   max_position_embeddings=_positive("max_position_embeddings", _get(d, "max_position_embeddings", int, 1 << 20)),
                   eos_token_ids=eos_ids, raw=dict(d))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
             "logit_softcap": self.logit_softcap, "layers": [l.to_dict() for l in self.layers]}
        if self.max_position_embeddings != 1 << 20:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
