"""The Sutosun decoder as a `ModelSpec`.

The stream starts as the RMS-normed embedding row (weight `embed.norm`). Layers are `pre_norm` blocks:
x += mixer(norm1(x)), then x += ff(norm2(x)). Mixers: `attention` (the `attention` part without rotation: biases, an RMS
norm over the whole q and the whole k projection, a query temperature that grows with the position, a stored sink score
per head in the softmax's denominator, one output gate per head), `retention` (the `retention` part: linear attention
with a fixed decay per head) and `latent_attention` (the `latent_attention` part without output gate: keys and values
from a cached latent, one rotated key part shared by the heads, rotation in pairs (i, i + n/2) with YaRN-scaled
frequencies, a stored sink score per head). Feed-forwards: `glu` with the tanh form of gelu, or `routed` experts with
gated silu units, a router bias and the softmax over the chosen logits as weights. A layer entry with `weights_of`: j
runs layer j's parts with a cache and state of its own. The logits pass a smooth cap c tanh(. / c).
Tensor names: `embed`, `embed.norm`, `head`, `final.norm` and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`,
`l<i>.mlp.*`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sutosun_config import MAX_POSITIONS, SutosunConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, Run

YARN_MAGNITUDE = 0.1  # cos and sin are multiplied by 0.1 ln(factor) + 1


def _rope(rot, size: int):
    """The rotary part over the first `rot.dims` of `size` dimensions, pairs (i, i + dims/2), or None."""
    if rot is None:
        return None
    scaling = None
    if rot.yarn is not None:
        y = rot.yarn
        scaling = {"kind": "yarn", "factor": y.factor, "original": y.original, "fast": y.fast, "slow": y.slow,
                   "magnitude": YARN_MAGNITUDE}
    return PartSpec("rope", {"head_dim": size, "rotary_dim": rot.dims, "theta": rot.base, "pairs": "half",
                             "scaling": scaling})


def _mixer_spec(layer, E: int, eps: float, p: str) -> PartSpec:
    m = layer.mixer
    if layer.type == "attention":
        q_temp = {"coef": m.q_temp_coef, "every": m.q_temp_every} if m.q_temp_coef is not None else None
        return PartSpec("attention",
                        {"width": E, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim,
                         "v_head_dim": m.vdim, "window": None, "scale": m.scale, "position": None, "qk_norm": "whole",
                         "eps": eps, "sink": "learned", "gate": "head", "q_temp": q_temp},
                        {"q": p + "q", "k": p + "k", "v": p + "v", "q_bias": p + "q.b", "k_bias": p + "k.b",
                         "v_bias": p + "v.b", "q_norm": p + "q.norm", "k_norm": p + "k.norm", "sink": p + "sink",
                         "g": p + "g", "o": p + "o"})
    if layer.type == "retention":
        return PartSpec("retention", {"width": E, "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay),
                                      "eps": eps, "position": _rope(m.rot, m.dim)},
                        {"q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "o": p + "o"})
    if layer.type == "latent_attention":
        return PartSpec("latent_attention",
                        {"width": E, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                         "kv_rank": m.kv_rank, "window": None, "scale": m.scale, "eps": eps,
                         "position": _rope(m.rot, m.rot_dim), "gate": False, "sink": True},
                        {"q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv",
                         "sink": p + "sink", "o": p + "o"})
    raise ValueError(layer.type)


def _mlp_spec(mlp, E: int, p: str) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("glu", {"width": E, "inner": mlp.ff, "act": "gelu_tanh"},
                        {"gate": p + "gate", "up": p + "up", "down": p + "down"})
    names = {"router": p + "router", "router_bias": p + "router.b"}
    for e in range(mlp.experts):
        names[f"gate{e}"] = f"{p}e{e}.gate"
        names[f"up{e}"] = f"{p}e{e}.up"
        names[f"down{e}"] = f"{p}e{e}.down"
    return PartSpec("routed", {"width": E, "inner": mlp.ff, "experts": mlp.experts, "top": mlp.top, "act": "swiglu",
                               "router_bias": True}, names)


def sutosun_spec(cfg: SutosunConfig) -> ModelSpec:
    E, eps = cfg.width, cfg.eps

    def norm(name):
        return PartSpec("rmsnorm", {"width": E, "eps": eps}, {"weight": name})

    layers, at = [], {}  # the layers that have tensors of their own, and where each sits in that list
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        at[i] = len(layers)
        layers.append(LayerSpec(block=PartSpec("pre_norm"), mixer=_mixer_spec(layer, E, eps, p + "mix."),
                                mixer_norm=norm(p + "norm1"),
                                feed_forward=_mlp_spec(layer.mlp, E, p + "mlp.") if layer.mlp is not None else None,
                                ffn_norm=norm(p + "norm2") if layer.mlp is not None else None))
    # every entry of the file is one run with a cache and state of its own
    schedule = [Run(layer=at[cfg.weights_layer(i)], cache=i, owns=True) for i in range(len(cfg.layers))]
    return ModelSpec(
        architecture="Sutosun", vocab_size=cfg.vocab, width=E, max_positions=MAX_POSITIONS,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "width": E, "norm_eps": eps},
                           {"weight": "embed", "norm": "embed.norm"}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("head", {"vocab": cfg.vocab, "width": E, "softcap": cfg.logit_softcap}, {"weight": "head"}))


@register_architecture("Sutosun")
def build_sutosun(config_json: dict) -> ModelSpec:
    return sutosun_spec(SutosunConfig.from_json(config_json))
