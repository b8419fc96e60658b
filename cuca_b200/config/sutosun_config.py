"""Typed configuration of the Sutosun decoder, read from its config.json.

The file is nested: `layers` is a list with one entry per layer (`type` names the mixer, `mixer` holds the mixer's
sizes and constants, `mlp` the feed-forward's or null, and `weights_of`: j says that the layer has no tensors of its
own and runs with layer j's), `norm.eps`, `logit_softcap`, `vocab`, `width`. Every size and constant comes from
there. A key the file does not have switches its feature off where that makes sense (no `q_temp`: queries as they
are; no `rot`: no rotation; no `rot.scaling`: plain frequencies; no `kv_heads`: one key head per query head; no `vdim`:
values as wide as keys; no `logit_softcap`: logits as they are; `mlp` null: no feed-forward) and is an error otherwise.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .bananex_config import _get
from .dupenex_config import _positive
from .model_config import ConfigError
from .pudinex_config import YarnConfig

MIXER_TYPES = ("attention", "retention", "latent_attention")
MAX_POSITIONS = 1 << 20  # the file gives no longest sequence: nothing in the model depends on one


@dataclass(frozen=True)
class RotConfig:
    base: float
    dims: int
    yarn: Optional[YarnConfig]

    @staticmethod
    def from_json(rot, where, most: int):
        """`most`: the size of what is rotated; `dims` is even and at most that."""
        if not rot:
            return None
        sc = rot.get("scaling")
        c = RotConfig(_get(rot, "base", float, where), _get(rot, "dims", int, where),
                      YarnConfig.from_json(sc, where + ".scaling") if sc else None)
        if c.dims % 2 or not 0 <= c.dims <= most:
            raise ConfigError(f"config.json `{where}.dims` = {c.dims} must be even and at most {most}")
        if not c.base > 0:
            raise ConfigError(f"config.json `{where}.base` must be positive")
        return c if c.dims else None


@dataclass(frozen=True)
class GatedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp_coef: Optional[float]
    q_temp_every: int

    @staticmethod
    def from_json(m, where):
        heads, dim = _get(m, "heads", int, where), _get(m, "dim", int, where)
        qt = m.get("q_temp")
        c = GatedAttentionConfig(
            heads=heads, kv_heads=int(m["kv_heads"]) if m.get("kv_heads") is not None else heads, dim=dim,
            vdim=int(m["vdim"]) if m.get("vdim") is not None else dim,
            scale=float(m["scale"]) if m.get("scale") is not None else dim ** -0.5,
            q_temp_coef=_get(qt, "coef", float, where + ".q_temp") if qt else None,
            q_temp_every=_get(qt, "every", int, where + ".q_temp") if qt else 0)
        _positive(where, heads=c.heads, kv_heads=c.kv_heads, dim=c.dim, vdim=c.vdim)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json `{where}`: {c.kv_heads} kv_heads do not divide {c.heads} heads")
        if qt and c.q_temp_every < 1:
            raise ConfigError(f"config.json `{where}.q_temp.every` must be positive")
        return c


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot: Optional[RotConfig]

    @staticmethod
    def from_json(m, where):
        heads, dim = _get(m, "heads", int, where), _get(m, "dim", int, where)
        decay = m.get("decay")
        if not isinstance(decay, list):
            raise ConfigError(f"config.json is missing the list `{where}.decay`")
        c = RetentionConfig(heads=heads, dim=dim, vdim=int(m["vdim"]) if m.get("vdim") is not None else dim,
                            decay=tuple(float(v) for v in decay),
                            rot=RotConfig.from_json(m.get("rot"), where + ".rot", dim))
        _positive(where, heads=c.heads, dim=c.dim, vdim=c.vdim)
        if len(c.decay) != c.heads:
            raise ConfigError(f"config.json `{where}.decay` has {len(c.decay)} entries for {c.heads} heads")
        return c


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Optional[RotConfig]

    @staticmethod
    def from_json(m, where):
        dim, rot_dim = _get(m, "dim", int, where), int(m.get("rot_dim") or 0)
        c = LatentConfig(heads=_get(m, "heads", int, where), dim=dim, rot_dim=rot_dim,
                         vdim=int(m["vdim"]) if m.get("vdim") is not None else dim,
                         kv_rank=_get(m, "kv_rank", int, where),
                         scale=float(m["scale"]) if m.get("scale") is not None else (dim + rot_dim) ** -0.5,
                         rot=RotConfig.from_json(m.get("rot"), where + ".rot", rot_dim))
        _positive(where, heads=c.heads, dim=c.dim, vdim=c.vdim, kv_rank=c.kv_rank)
        if c.rot_dim < 0:
            raise ConfigError(f"config.json `{where}.rot_dim` must not be negative")
        return c


_MIXERS = {"attention": GatedAttentionConfig, "retention": RetentionConfig, "latent_attention": LatentConfig}


@dataclass(frozen=True)
class MlpConfig:
    kind: str  # "dense" | "moe"
    ff: int  # of the dense layer, or of one expert
    experts: int = 0
    top: int = 0

    @staticmethod
    def from_json(m, where):
        kind = str(m.get("kind", "dense"))
        if kind == "dense":
            c = MlpConfig("dense", _get(m, "ff", int, where))
        elif kind == "moe":
            r = m.get("router")
            c = MlpConfig("moe", _get(m.get("expert"), "ff", int, where + ".expert"),
                          experts=_get(r, "experts", int, where + ".router"), top=_get(r, "top", int, where + ".router"))
            if not 1 <= c.top <= c.experts:
                raise ConfigError(f"config.json `{where}.router`: top = {c.top} must lie in 1..experts = {c.experts}")
        else:
            raise ConfigError(f"config.json `{where}.kind` = `{kind}`; this engine knows: dense, moe")
        _positive(where, ff=c.ff)
        return c


@dataclass(frozen=True)
class SutosunLayer:
    type: str
    mixer: object
    mlp: Optional[MlpConfig]
    weights_of: Optional[int]  # the layer whose tensors this one runs with (None: its own)


@dataclass(frozen=True)
class SutosunConfig:
    vocab: int
    width: int
    eps: float
    logit_softcap: Optional[float]
    layers: tuple

    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer i runs with: i itself, or where its `weights_of` leads."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config.json `layers[{i}].weights_of` leads back to itself")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    @staticmethod
    def from_json(cfg: dict) -> "SutosunConfig":
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
            of = entry.get("weights_of")
            if of is not None and not (isinstance(of, int) and 0 <= of < len(layers) and of != i):
                raise ConfigError(f"config.json `{where}.weights_of` = {of!r} must name another layer")
            out.append(SutosunLayer(kind, _MIXERS[kind].from_json(entry["mixer"], where + ".mixer"),
                                    MlpConfig.from_json(mlp, where + ".mlp") if mlp else None, of))
        cap = cfg.get("logit_softcap")
        c = SutosunConfig(vocab=_get(cfg, "vocab", int, ""), width=_get(cfg, "width", int, ""),
                          eps=_get(cfg.get("norm"), "eps", float, "norm"),
                          logit_softcap=float(cap) if cap else None, layers=tuple(out))
        if c.vocab < 1 or c.width < 1:
            raise ConfigError("config.json `vocab` and `width` must be positive")
        if c.logit_softcap is not None and c.logit_softcap <= 0:
            raise ConfigError("config.json `logit_softcap` must be positive")
        for i, layer in enumerate(c.layers):
            j = c.weights_layer(i)
            if c.layers[j].type != layer.type:
                raise ConfigError(f"config.json `layers[{i}]` is `{layer.type}` but runs with the tensors of "
                                  f"layers[{j}], a `{c.layers[j].type}`")
        return c
