"""Typed configuration of the Pudinex decoder, read from its config.json.

The file is nested: `layers` is a list with one entry per layer (`type` names the mixer, `mixer` holds the mixer's
sizes and constants, `mlp` the feed-forward's or null), `embedding.scale`, `norm.eps` and `norm.groups`, `vocab`,
`width`. Every size and constant comes from there. A key the file does not have switches its feature off where that
makes sense (no `embedding`: rows as stored; no `norm.groups`: the whole row is one part; no `rot`: no rotation; no
`rot.scaling`: plain frequencies; no `softcap`: scores as they are; no `router.identity`: every expert has weights; no
`shared`: no shared expert; `mlp` null: no feed-forward) and is an error otherwise.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .bananex_config import _get
from .dupenex_config import _positive
from .model_config import ConfigError

MIXER_TYPES = ("attention", "hgrn2")
MAX_POSITIONS = 1 << 20  # the file gives no longest sequence: nothing in the model depends on one


@dataclass(frozen=True)
class YarnConfig:
    factor: float
    original: float
    fast: float
    slow: float

    @staticmethod
    def from_json(m, where):
        c = YarnConfig(_get(m, "factor", float, where), _get(m, "original", float, where), _get(m, "fast", float, where),
                       _get(m, "slow", float, where))
        if c.factor <= 0 or c.original <= 0 or c.fast <= 0 or c.slow <= 0:
            raise ConfigError(f"config.json `{where}`: factor, original, fast and slow must be positive")
        return c


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: Optional[float]
    softcap: Optional[float]
    rot_base: float
    rot_dims: int
    yarn: Optional[YarnConfig]

    @staticmethod
    def from_json(m, where):
        rot = m.get("rot")
        heads = _get(m, "heads", int, where)
        dim = _get(m, "dim", int, where)
        sc = rot.get("scaling") if rot else None
        c = SinkAttentionConfig(
            heads=heads, kv_heads=int(m["kv_heads"]) if m.get("kv_heads") is not None else heads, dim=dim,
            vdim=int(m["vdim"]) if m.get("vdim") is not None else dim,
            scale=float(m["scale"]) if m.get("scale") is not None else None,
            softcap=float(m["softcap"]) if m.get("softcap") else None,
            rot_base=_get(rot, "base", float, where + ".rot") if rot else 10000.0,
            rot_dims=_get(rot, "dims", int, where + ".rot") if rot else 0,
            yarn=YarnConfig.from_json(sc, where + ".rot.scaling") if sc else None)
        _positive(where, heads=c.heads, kv_heads=c.kv_heads, dim=c.dim, vdim=c.vdim)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json `{where}`: {c.kv_heads} kv_heads do not divide {c.heads} heads")
        if c.rot_dims % 2 or not 0 <= c.rot_dims <= c.dim:
            raise ConfigError(f"config.json `{where}.rot.dims` = {c.rot_dims} must be even and at most dim")
        if c.softcap is not None and c.softcap <= 0:
            raise ConfigError(f"config.json `{where}.softcap` must be positive")
        return c


@dataclass(frozen=True)
class ForgetGateConfig:
    heads: int
    dim: int
    vdim: int

    @staticmethod
    def from_json(m, where):
        c = ForgetGateConfig(_get(m, "heads", int, where), _get(m, "dim", int, where), _get(m, "vdim", int, where))
        _positive(where, heads=c.heads, dim=c.dim, vdim=c.vdim)
        return c


_MIXERS = {"attention": SinkAttentionConfig, "hgrn2": ForgetGateConfig}


@dataclass(frozen=True)
class MlpConfig:
    kind: str  # "dense" | "moe"
    ff: int  # of the dense layer, or of one expert
    limit: float = 0.0  # dense: the cap on gate and up
    experts: int = 0
    identity: int = 0
    top: int = 0
    shared: int = 0  # inner size of the shared expert, 0: none

    @staticmethod
    def from_json(m, where):
        kind = str(m.get("kind", "dense"))
        if kind == "dense":
            c = MlpConfig("dense", _get(m, "ff", int, where), limit=_get(m, "limit", float, where))
            if not c.limit > 0:
                raise ConfigError(f"config.json `{where}.limit` must be positive")
        elif kind == "moe":
            r, sh = m.get("router"), m.get("shared")
            c = MlpConfig("moe", _get(m.get("expert"), "ff", int, where + ".expert"),
                          experts=_get(r, "experts", int, where + ".router"), identity=int(r.get("identity") or 0),
                          top=_get(r, "top", int, where + ".router"),
                          shared=_get(sh, "ff", int, where + ".shared") if sh else 0)
            if c.experts < 0 or c.identity < 0 or c.shared < 0:
                raise ConfigError(f"config.json `{where}`: experts, identity and shared.ff must not be negative")
            if not 1 <= c.top <= c.experts + c.identity:
                raise ConfigError(f"config.json `{where}.router`: top = {c.top} must lie in 1..experts + identity = "
                                  f"{c.experts + c.identity}")
        else:
            raise ConfigError(f"config.json `{where}.kind` = `{kind}`; this engine knows: dense, moe")
        _positive(where, ff=c.ff)
        return c


@dataclass(frozen=True)
class PudinexLayer:
    type: str
    mixer: object
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class PudinexConfig:
    vocab: int
    width: int
    eps: float
    norm_groups: int
    embedding_scale: float
    layers: tuple

    @staticmethod
    def from_json(cfg: dict) -> "PudinexConfig":
        layers = cfg.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json `layers` must be a non-empty list")
        out = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]"
            kind = _get(entry, "type", str, where)
            if kind not in _MIXERS:
                raise ConfigError(f"config.json `{where}.type` = `{kind}`; this engine knows: {', '.join(MIXER_TYPES)}")
            if not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json is missing `{where}.mixer`")
            mlp = entry.get("mlp")
            out.append(PudinexLayer(kind, _MIXERS[kind].from_json(entry["mixer"], where + ".mixer"),
                                    MlpConfig.from_json(mlp, where + ".mlp") if mlp else None))
        norm = cfg.get("norm")
        emb = cfg.get("embedding") or {}
        c = PudinexConfig(vocab=_get(cfg, "vocab", int, ""), width=_get(cfg, "width", int, ""),
                          eps=_get(norm, "eps", float, "norm"), norm_groups=int(norm.get("groups") or 1),
                          embedding_scale=float(emb.get("scale", 1.0)), layers=tuple(out))
        if c.vocab < 1 or c.width < 1:
            raise ConfigError("config.json `vocab` and `width` must be positive")
        if c.norm_groups < 1 or c.width % c.norm_groups:
            raise ConfigError(f"config.json `norm.groups` = {c.norm_groups} must divide `width` = {c.width}")
        return c
