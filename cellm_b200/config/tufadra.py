"""Typed configuration of the Tufadra design, read from its config.json.

The file names the design with one string (`architecture`) and gives the vocabulary, the model's width, the number
of learned position vectors (`max_positions`), the norms' eps, and a list of layers. A layer has a `type` (its
mixer: `attention`), the mixer's sizes and constants (`mixer`), its feed-forward (`mlp`: a mixture of experts, or
null for none), and may name an earlier layer whose weights it uses (`weights_of`; it keeps a cache of its own).
Every size and constant that can differ between models comes from the file. What the file leaves out does not
exist: an attention without `q_temp` has no query temperature, a router without `groups` chooses among all
experts, a feed-forward without `shared` has no shared expert."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .errors import ConfigError
from .lfm2 import _get

MIXERS = ("attention",)
MLP_KINDS = ("moe",)


@dataclass(frozen=True)
class QueryTemperature:
    coef: float
    every: int


@dataclass(frozen=True)
class TufadraAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: Optional[QueryTemperature]

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "TufadraAttention":
        qt = d.get("q_temp")
        if qt is not None:
            if not isinstance(qt, dict):
                raise ConfigError(f"config.json: {where}.mixer.q_temp should be an object")
            qt = QueryTemperature(_get(qt, "coef", float), _get(qt, "every", int))
            if qt.every < 1:
                raise ConfigError(f"config.json: {where}: q_temp.every must be positive")
        c = cls(*(_get(d, k, int) for k in ("heads", "kv_heads", "dim", "vdim")), _get(d, "scale", float), qt)
        if min(c.heads, c.kv_heads, c.dim, c.vdim) < 1:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: {c.heads} heads are not a multiple of {c.kv_heads} key/value heads")
        return c

    def to_dict(self) -> dict:
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.q_temp is not None:
            d["q_temp"] = {"coef": self.q_temp.coef, "every": self.q_temp.every}
        return d


@dataclass(frozen=True)
class TufadraMoe:
    ff: int
    experts: int
    top: int
    scale: float
    groups: int          # 1: no groups
    keep: int
    shared_ff: int       # 0: no shared expert
    has_groups: bool = True

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "TufadraMoe":
        kind = _get(d, "kind", str)
        if kind not in MLP_KINDS:
            raise ConfigError(f"config.json: {where}: feed-forward kind {kind!r}; known: {list(MLP_KINDS)}")
        router, expert = _get(d, "router", dict), _get(d, "expert", dict)
        groups = router.get("groups")
        count, keep = 1, 1
        if groups is not None:
            if not isinstance(groups, dict):
                raise ConfigError(f"config.json: {where}.mlp.router.groups should be an object")
            count, keep = _get(groups, "count", int), _get(groups, "keep", int)
        shared = d.get("shared")
        if shared is not None and not isinstance(shared, dict):
            raise ConfigError(f"config.json: {where}.mlp.shared should be an object or null")
        c = cls(_get(expert, "ff", int), _get(router, "experts", int), _get(router, "top", int), _get(router, "scale", float),
                count, keep, _get(shared, "ff", int) if shared is not None else 0, groups is not None)
        if c.ff < 1 or c.shared_ff < 0 or not 1 <= c.top <= c.experts:
            raise ConfigError(f"config.json: {where}: expert sizes must be positive and top at most the number of experts")
        if c.groups < 1 or c.experts % c.groups or not 1 <= c.keep <= c.groups:
            raise ConfigError(f"config.json: {where}: {c.experts} experts do not form {c.groups} equal groups of which {c.keep} are kept")
        if c.keep * (c.experts // c.groups) < c.top:
            raise ConfigError(f"config.json: {where}: {c.keep} groups of {c.experts // c.groups} experts cannot give {c.top} choices")
        return c

    def to_dict(self) -> dict:
        router = {"experts": self.experts, "scale": self.scale, "top": self.top}
        if self.has_groups:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        d = {"expert": {"ff": self.ff}, "kind": "moe", "router": router}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class TufadraLayer:
    type: str
    mixer: TufadraAttention
    mlp: Optional[TufadraMoe]
    weights_of: Optional[int] = None     # the layer whose tensors this one uses (None: its own)

    def to_dict(self) -> dict:
        d = {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None, "type": self.type}
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


@dataclass(frozen=True)
class TufadraConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: tuple[TufadraLayer, ...]
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict) -> "TufadraConfig":
        norm = _get(d, "norm", dict)
        raw = _get(d, "layers", list)
        layers: list[TufadraLayer] = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: {where} should be an object")
            kind = _get(entry, "type", str)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r}; known: {list(MIXERS)}")
            src = entry.get("weights_of")
            if src is not None:
                if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < len(raw) or src == i:
                    raise ConfigError(f"config.json: {where}: weights_of must name another layer, not {src!r}")
            mixer = TufadraAttention.from_dict(_get(entry, "mixer", dict), where)
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}.mlp should be an object or null")
                mlp = TufadraMoe.from_dict(mlp, where)
            layers.append(TufadraLayer(kind, mixer, mlp, src))
        for i, layer in enumerate(layers):           # a chain of references ends at the layer that has the tensors
            j, seen = layer.weights_of, {i}
            while j is not None and layers[j].weights_of is not None:
                if j in seen:
                    raise ConfigError(f"config.json: layers[{i}]: weights_of runs in a circle")
                seen.add(j)
                j = layers[j].weights_of
            if j is not None:               # the sizes and constants are those of the layer whose tensors it uses
                layers[i] = TufadraLayer(layers[j].type, layers[j].mixer, layers[j].mlp, j)
        c = cls(_get(d, "vocab", int), _get(d, "width", int), _get(d, "max_positions", int), _get(norm, "eps", float),
                tuple(layers), _get(d, "eos_token_id", int, None))
        if c.vocab < 1 or c.width < 1 or c.max_positions < 1:
            raise ConfigError("config.json: vocab, width and max_positions must be positive")
        return c

    def to_dict(self) -> dict:
        d = {"architecture": "Tufadra", "layers": [l.to_dict() for l in self.layers], "max_positions": self.max_positions,
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
