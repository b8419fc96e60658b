"""The Pudinex decoder as a `ModelSpec`.

Every layer has one RMS norm (in `norm.groups` parts) whose output both of its sublayers read: x += mixer(h) + ff(h)
(`parallel_residual` blocks). Mixers: `attention` (the `attention` part with a norm per head on queries, keys and
values, rotary pairs (i, i + n/2) on part of a head with YaRN-scaled frequencies, a smooth cap on the scores and a
sink in the softmax's denominator) and `hgrn2` (the `hgrn2` part: linear attention whose forget gate also decides what
is written). Feed-forwards: `glu_capped` (a gated unit with capped inputs), or `routed_scored` experts (scores over all
router outputs, a correction that only the choice sees, experts that return their input, a shared expert). The
embedding rows are scaled; the model's norm is the layers' kind.
Tensor names: `embed`, `head`, `final.norm` and per layer i `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`.
"""
from __future__ import annotations

from ..config.pudinex_config import MAX_POSITIONS, PudinexConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, default_schedule

GLU_ALPHA = 1.702  # the dense feed-forward's gate is g sigmoid(1.702 g)
YARN_MAGNITUDE = 0.1  # cos and sin are multiplied by 0.1 ln(factor) + 1


def _mixer_spec(layer, E: int, eps: float, p: str) -> PartSpec:
    m = layer.mixer
    if layer.type == "attention":
        position = None
        if m.rot_dims:
            scaling = None
            if m.yarn is not None:
                y = m.yarn
                scaling = {"kind": "yarn", "factor": y.factor, "original": y.original, "fast": y.fast, "slow": y.slow,
                           "magnitude": YARN_MAGNITUDE}
            position = PartSpec("rope", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                         "pairs": "half", "scaling": scaling})
        return PartSpec("attention",
                        {"width": E, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim,
                         "v_head_dim": m.vdim, "window": None, "scale": m.scale, "position": position, "qk_norm": True,
                         "v_norm": True, "eps": eps, "softcap": m.softcap, "sink": True},
                        {"q": p + "q", "k": p + "k", "v": p + "v", "q_norm": p + "q.norm", "k_norm": p + "k.norm",
                         "o": p + "o"})
    if layer.type == "hgrn2":
        return PartSpec("hgrn2", {"width": E, "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "eps": eps},
                        {"q": p + "q", "f": p + "f", "f_bias": p + "f.b", "lower": p + "lower", "v": p + "v",
                         "norm": p + "norm", "o": p + "o"})
    raise ValueError(layer.type)


def _mlp_spec(mlp, E: int, p: str) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("glu_capped", {"width": E, "inner": mlp.ff, "limit": mlp.limit, "alpha": GLU_ALPHA},
                        {"gate": p + "gate", "up": p + "up", "down": p + "down"})
    names = {"router": p + "router", "correction": p + "correction", "shared_gate": p + "shared.gate",
             "shared_up": p + "shared.up", "shared_down": p + "shared.down"}
    for e in range(mlp.experts):
        names[f"gate{e}"] = f"{p}e{e}.gate"
        names[f"up{e}"] = f"{p}e{e}.up"
        names[f"down{e}"] = f"{p}e{e}.down"
    return PartSpec("routed_scored", {"width": E, "inner": mlp.ff, "experts": mlp.experts, "identity": mlp.identity,
                                      "top": mlp.top, "shared": mlp.shared, "correction": True}, names)


def pudinex_spec(cfg: PudinexConfig) -> ModelSpec:
    E, eps = cfg.width, cfg.eps

    def norm(name):
        return PartSpec("rmsnorm", {"width": E, "eps": eps, "groups": cfg.norm_groups}, {"weight": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        layers.append(LayerSpec(block=PartSpec("parallel_residual"), mixer=_mixer_spec(layer, E, eps, p + "mix."),
                                mixer_norm=norm(p + "norm1"),
                                feed_forward=_mlp_spec(layer.mlp, E, p + "mlp.") if layer.mlp is not None else None))
    return ModelSpec(
        architecture="Pudinex", vocab_size=cfg.vocab, width=E, max_positions=MAX_POSITIONS,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "width": E, "scale": cfg.embedding_scale},
                           {"weight": "embed"}),
        layers=layers, schedule=default_schedule(len(layers)), final_norm=norm("final.norm"),
        head=PartSpec("head", {"vocab": cfg.vocab, "width": E}, {"weight": "head"}))


@register_architecture("Pudinex")
def build_pudinex(config_json: dict) -> ModelSpec:
    return pudinex_spec(PudinexConfig.from_json(config_json))
