"""Typed configuration of the Viresun decoder: a stack of layers that each name their mixer
(windowed attention with a distance bias, or a Mamba-2 state-space mixer) and their
feed-forward (dense, routed, or none), possibly borrowing another layer's weights.

config.json gives every size and constant: ``vocab``, ``width``, ``norm.eps`` and ``layers``,
a list of ``{"type", "mixer": {...}, "mlp": {...} | null, "weights_of": j}`` (the last optional:
such a layer owns no tensors and computes with those of layer ``j``; what it caches per request
stays separate).  Nothing is defaulted
that the configuration must say; what a mechanism may leave out (a window, a query
temperature) is None.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError


def _int(d: Mapping[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"{where}.{key} must be an integer, got {v!r}")
    if int(v) < minimum:
        raise ConfigError(f"{where}.{key} must be at least {minimum}, got {v}")
    return int(v)


def _float(d: Mapping[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]                   # mask.size
    q_temp: Optional[Tuple[float, int]]     # (coef, every)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "AttentionMixerConfig":
        heads = _int(d, "heads", where)
        kv = _int(d, "kv_heads", where) if d.get("kv_heads") is not None else heads     # left out: one per query head
        if heads % kv:
            raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv} kv_heads")
        mask = d.get("mask") or None
        temp = d.get("q_temp") or None
        dim = _int(d, "dim", where)
        return cls(heads=heads, kv_heads=kv, dim=dim,
                   vdim=_int(d, "vdim", where) if d.get("vdim") is not None else dim,      # left out: the key's size
                   scale=_float(d, "scale", where),
                   window=_int(mask, "size", where + ".mask") if mask else None,
                   q_temp=(_float(temp, "coef", where + ".q_temp"), _int(temp, "every", where + ".q_temp"))
                   if temp else None)


@dataclass(frozen=True)
class Mamba2MixerConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "Mamba2MixerConfig":
        out = cls(heads=_int(d, "heads", where), vdim=_int(d, "vdim", where), state=_int(d, "state", where),
                  groups=_int(d, "groups", where) if d.get("groups") is not None else 1,
                  conv=_int(d, "conv", where),
                  norm_groups=_int(d, "norm_groups", where) if d.get("norm_groups") is not None else 1)
        if out.heads % out.groups:
            raise ConfigError(f"{where}: {out.heads} heads are not a multiple of {out.groups} groups")
        if (out.heads * out.vdim) % out.norm_groups:
            raise ConfigError(f"{where}: heads * vdim does not fall into {out.norm_groups} equal parts")
        return out


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                    # "dense" | "moe"
    ff: int                      # dense: the hidden size of the layer; moe: of one expert
    experts: int = 0
    top: int = 0
    limit: float = 0.0

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "FeedForwardConfig":
        kind = d.get("kind")
        if kind == "dense":
            return cls(kind="dense", ff=_int(d, "ff", where))
        if kind == "moe":
            expert, router = d.get("expert") or {}, d.get("router") or {}
            out = cls(kind="moe", ff=_int(expert, "ff", where + ".expert"),
                      experts=_int(router, "experts", where + ".router"), top=_int(router, "top", where + ".router"),
                      limit=_float(expert, "limit", where + ".expert"))
            if out.top > out.experts:
                raise ConfigError(f"{where}: {out.top} of {out.experts} experts cannot be chosen")
            if not out.limit > 0:
                raise ConfigError(f"{where}.expert.limit must be positive")
            return out
        raise ConfigError(f"{where}.kind {kind!r} is not known (dense, moe)")


@dataclass(frozen=True)
class ViresunLayerConfig:
    type: str                                   # "attention" | "mamba2"
    mixer: Any                                  # AttentionMixerConfig | Mamba2MixerConfig
    mlp: Optional[FeedForwardConfig]
    weights_of: Optional[int] = None


@dataclass(frozen=True)
class ViresunConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[ViresunLayerConfig, ...]
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    max_position_embeddings: int = 1 << 17      # the design sets no limit; block tables are made this wide

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ViresunConfig":
        norm = d.get("norm") or {}
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a list with at least one entry")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = L.get("type")
            if kind == "attention":
                mixer = AttentionMixerConfig.from_dict(L.get("mixer") or {}, where + ".mixer")
            elif kind == "mamba2":
                mixer = Mamba2MixerConfig.from_dict(L.get("mixer") or {}, where + ".mixer")
            else:
                raise ConfigError(f"{where}.type {kind!r} is not known (attention, mamba2)")
            mlp = FeedForwardConfig.from_dict(L["mlp"], where + ".mlp") if L.get("mlp") else None
            src = L.get("weights_of")
            if src is not None:
                src = _int(L, "weights_of", where, minimum=0)
                if src >= i or layers[src].weights_of is not None:
                    raise ConfigError(f"{where}.weights_of must name an earlier layer that has tensors of its own")
                if (layers[src].type, layers[src].mixer, layers[src].mlp) != (kind, mixer, mlp):
                    raise ConfigError(f"{where} borrows the tensors of layer {src} but describes another layer")
            layers.append(ViresunLayerConfig(kind, mixer, mlp, src))
        eps = _float(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError("norm.eps must be positive")
        width = _int(d, "width", "config")
        if width % 2:
            raise ConfigError("width must be even: sine and cosine entries of the position vector alternate")
        dtype = str(d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16").replace("torch.", "")
        return cls(vocab_size=_int(d, "vocab", "config"), hidden_size=width, norm_eps=eps, layers=tuple(layers),
                   torch_dtype=dtype,
                   max_position_embeddings=_int(d, "max_position_embeddings", "config")
                   if d.get("max_position_embeddings") is not None else 1 << 17)
