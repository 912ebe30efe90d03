"""Typed configuration of the Bivatar decoder: a stack of layers that each name their mixer
(attention through a shared latent with a rotated key part, or grouped-query attention behind a
sliding window that keeps a sequence's first tokens, with a linear distance penalty) and their
gated feed-forward (or none), the norms sitting on the sublayers' outputs.

config.json gives every size and constant: ``vocab``, ``width``, ``norm.eps``, ``residual_mult``,
``embedding.scale`` and ``layers``, a list of ``{"type", "mixer": {...}, "mlp": {...} | null}``.
A latent-attention mixer may say ``kv_from: j``: it has no down-projection to the latent and
reads what layer ``j`` keeps.  What a mechanism may leave out (a window, kept first tokens, a
frequency scaling, the feed-forward) is None or 0.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError
from .viresun_config import _float, _int


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]]      # (factor, original, fast, slow)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "RotationConfig":
        s = d.get("scaling") or None
        scaling = None
        if s:
            scaling = (_float(s, "factor", where + ".scaling"), _float(s, "original", where + ".scaling"),
                       _float(s, "fast", where + ".scaling"), _float(s, "slow", where + ".scaling"))
            if not (scaling[0] > 0 and scaling[1] > 0 and scaling[2] > 0 and scaling[3] > 0):
                raise ConfigError(f"{where}.scaling: factor, original, fast and slow must be positive")
        out = cls(dims=_int(d, "dims", where), base=_float(d, "base", where), scaling=scaling)
        if out.dims % 2:
            raise ConfigError(f"{where}.dims must be even: dimension i turns with dimension i + dims/2")
        if not out.base > 1:
            raise ConfigError(f"{where}.base must be above 1")
        return out


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int                    # unrotated query/key dimensions per head
    rot_dim: int                # rotated query/key dimensions per head; the key's are shared by all heads
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: RotationConfig
    kv_from: Optional[int]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "LatentMixerConfig":
        dim = _int(d, "dim", where)
        out = cls(heads=_int(d, "heads", where), dim=dim, rot_dim=_int(d, "rot_dim", where),
                  vdim=_int(d, "vdim", where) if d.get("vdim") is not None else dim,
                  kv_rank=_int(d, "kv_rank", where), q_rank=_int(d, "q_rank", where), scale=_float(d, "scale", where),
                  rot=RotationConfig.from_dict(d.get("rot") or {}, where + ".rot"),
                  kv_from=_int(d, "kv_from", where, minimum=0) if d.get("kv_from") is not None else None)
        if out.rot.dims > out.rot_dim:
            raise ConfigError(f"{where}: {out.rot.dims} rotated dimensions do not fit rot_dim {out.rot_dim}")
        return out


@dataclass(frozen=True)
class WindowMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]       # mask.size
    keep_first: int             # mask.keep_first

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "WindowMixerConfig":
        heads = _int(d, "heads", where)
        kv = _int(d, "kv_heads", where) if d.get("kv_heads") is not None else heads
        if heads % kv:
            raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv} kv_heads")
        mask = d.get("mask") or None
        dim = _int(d, "dim", where)
        window = _int(mask, "size", where + ".mask") if mask and mask.get("size") is not None else None
        keep = _int(mask, "keep_first", where + ".mask", minimum=0) if mask and mask.get("keep_first") is not None else 0
        return cls(heads=heads, kv_heads=kv, dim=dim, vdim=_int(d, "vdim", where) if d.get("vdim") is not None else dim,
                   scale=_float(d, "scale", where), window=window, keep_first=keep if window else 0)


@dataclass(frozen=True)
class DenseFeedForwardConfig:
    ff: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "DenseFeedForwardConfig":
        if d.get("kind", "dense") != "dense":
            raise ConfigError(f"{where}.kind {d.get('kind')!r} is not known (dense)")
        return cls(ff=_int(d, "ff", where))


@dataclass(frozen=True)
class BivatarLayerConfig:
    type: str                                   # "latent_attention" | "attention"
    mixer: Any                                  # LatentMixerConfig | WindowMixerConfig
    mlp: Optional[DenseFeedForwardConfig]


@dataclass(frozen=True)
class BivatarConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    layers: Tuple[BivatarLayerConfig, ...]
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    max_position_embeddings: int = 1 << 17      # the design sets no limit; block tables are made this wide

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BivatarConfig":
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a list with at least one entry")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = L.get("type")
            if kind == "latent_attention":
                mixer = LatentMixerConfig.from_dict(L.get("mixer") or {}, where + ".mixer")
                j = mixer.kv_from
                if j is not None:
                    if j >= i or layers[j].type != "latent_attention" or layers[j].mixer.kv_from is not None:
                        raise ConfigError(f"{where}.mixer.kv_from must name an earlier latent-attention layer that "
                                          f"has a down-projection of its own")
                    src = layers[j].mixer
                    if (src.kv_rank, src.rot_dim, src.rot) != (mixer.kv_rank, mixer.rot_dim, mixer.rot):
                        raise ConfigError(f"{where} reads what layer {j} keeps, but its kv_rank, rot_dim or rotation differ")
            elif kind == "attention":
                mixer = WindowMixerConfig.from_dict(L.get("mixer") or {}, where + ".mixer")
            else:
                raise ConfigError(f"{where}.type {kind!r} is not known (latent_attention, attention)")
            mlp = DenseFeedForwardConfig.from_dict(L["mlp"], where + ".mlp") if L.get("mlp") else None
            layers.append(BivatarLayerConfig(kind, mixer, mlp))
        eps = _float(d.get("norm") or {}, "eps", "norm")
        if not eps > 0:
            raise ConfigError("norm.eps must be positive")
        emb = d.get("embedding") or {}
        dtype = str(d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16").replace("torch.", "")
        return cls(vocab_size=_int(d, "vocab", "config"), hidden_size=_int(d, "width", "config"), norm_eps=eps,
                   residual_mult=_float(d, "residual_mult", "config") if d.get("residual_mult") is not None else 1.0,
                   embedding_scale=_float(emb, "scale", "embedding") if emb.get("scale") is not None else 1.0,
                   layers=tuple(layers), torch_dtype=dtype,
                   max_position_embeddings=_int(d, "max_position_embeddings", "config")
                   if d.get("max_position_embeddings") is not None else 1 << 17)
