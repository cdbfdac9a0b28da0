"""Typed configuration of the Vezalorn design, read from its config.json.

The file names the design with one string (`architecture`), gives the model's width and vocabulary, the embedding's
scale, the norm's eps and number of groups, and a list of layers: each entry has a `type` (which mixer), the mixer's
sizes (`mixer`) and its feed-forward (`mlp`: kind and width, or null for a layer without one). Every size and every
constant that can differ between models comes from the file; nothing has a default."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .errors import ConfigError
from .lfm2 import _get

MIXERS = ("latent_attention", "mingru")
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotationConfig

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "LatentAttentionConfig":
        rot = _get(d, "rot", dict)
        c = cls(*(_get(d, k, int) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank")), _get(d, "scale", float),
                RotationConfig(_get(rot, "base", float), _get(rot, "dims", int)))
        if min(c.heads, c.dim, c.vdim, c.kv_rank) < 1 or c.rot_dim < 0:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        if c.rot.dims % 2 or not 0 <= c.rot.dims <= c.rot_dim:
            raise ConfigError(f"config.json: {where}: rot.dims {c.rot.dims} must be even and at most rot_dim {c.rot_dim}")
        return c

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "scale": self.scale, "rot": {"base": self.rot.base, "dims": self.rot.dims}}


@dataclass(frozen=True)
class MinGruConfig:
    width: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MinGruConfig":
        c = cls(_get(d, "width", int))
        if c.width < 1:
            raise ConfigError(f"config.json: {where}: width must be positive")
        return c

    def to_dict(self) -> dict:
        return {"width": self.width}


@dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int

    def to_dict(self) -> dict:
        return {"kind": self.kind, "ff": self.ff}


@dataclass(frozen=True)
class VezalornLayer:
    type: str
    mixer: object                       # LatentAttentionConfig | MinGruConfig
    mlp: Optional[MlpConfig]

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class VezalornConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    norm_groups: int
    layers: tuple[VezalornLayer, ...]
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict) -> "VezalornConfig":
        emb, norm = _get(d, "embedding", dict), _get(d, "norm", dict)
        raw = _get(d, "layers", list)
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: {where} should be an object")
            kind = _get(entry, "type", str)
            mixer = _get(entry, "mixer", dict)
            if kind == "latent_attention":
                m = LatentAttentionConfig.from_dict(mixer, where)
            elif kind == "mingru":
                m = MinGruConfig.from_dict(mixer, where)
            else:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r}; known: {list(MIXERS)}")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}.mlp should be an object or null")
                mk = _get(mlp, "kind", str)
                if mk not in MLP_KINDS:
                    raise ConfigError(f"config.json: {where}: feed-forward kind {mk!r}; known: {list(MLP_KINDS)}")
                mlp = MlpConfig(mk, _get(mlp, "ff", int))
                if mlp.ff < 1:
                    raise ConfigError(f"config.json: {where}: ff must be positive")
            layers.append(VezalornLayer(kind, m, mlp))
        c = cls(_get(d, "vocab", int), _get(d, "width", int), _get(emb, "scale", float), _get(norm, "eps", float),
                _get(norm, "groups", int), tuple(layers), _get(d, "eos_token_id", int, None))
        if c.vocab < 1 or c.width < 1:
            raise ConfigError("config.json: vocab and width must be positive")
        if c.norm_groups < 1 or c.width % c.norm_groups:
            raise ConfigError(f"config.json: width {c.width} does not split into {c.norm_groups} equal norm groups")
        return c

    def to_dict(self) -> dict:
        d = {"architecture": "Vezalorn", "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
             "layers": [l.to_dict() for l in self.layers]}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
