"""Small Pudinex configurations with weights that exercise every mechanism, for the engine and for the plain
implementation alike (the same values, bfloat16-rounded, as a folder and as 64-bit arrays)."""
from __future__ import annotations

import copy

import numpy as np
import torch

import plain_pudinex
from bananex_util import bf16_round, plain_weights, random_tokens, write_model  # noqa: F401  (shared helpers)

YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}


def attn(heads=4, kv_heads=2, dim=16, vdim=24, dims=8, base=10000.0, scaling=YARN, scale=None, softcap=8.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else dim ** -0.5}
    if softcap is not None:
        m["softcap"] = softcap
    if dims:
        m["rot"] = {"base": base, "dims": dims}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    return {"type": "attention", "mixer": m}


def hg(heads=3, dim=12, vdim=20):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def dense(ff=72, limit=0.6):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff=24, experts=5, identity=2, top=2, shared=40):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(layers, mlps, width=60, vocab=199, groups=3, eps=1e-5, emb_scale=2.0):
    out = []
    for l, m in zip(layers, mlps):
        l = copy.deepcopy(l)
        l["mlp"] = copy.deepcopy(m)
        out.append(l)
    cfg = {"architecture": "Pudinex", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
           "layers": out}
    if emb_scale is not None:
        cfg["embedding"] = {"scale": emb_scale}
    return cfg


# sizes that differ in every respect: the order of the layers, 1 to 4 norm parts, key heads shared or not, one head,
# values wider and narrower than keys and as wide, rotation of all, part or none of a head with and without scaled
# frequencies, a score cap that bites, a loose one and none, layers without a feed-forward, routed layers with and
# without experts that return their input, with and without a shared expert, one expert of one, all outputs chosen
CONFIGS = {
    "mix": config([hg(), attn(), hg(heads=2, dim=16, vdim=8), attn(heads=6, kv_heads=2, dim=12, vdim=10, dims=12,
                                                                  scaling=None, softcap=None)],
                  [dense(), moe(), moe(ff=16, experts=4, identity=0, top=4, shared=0), dense(40, limit=2.5)]),
    "plain": config([attn(heads=3, kv_heads=3, dims=0, vdim=16), hg(heads=1, dim=40, vdim=8), hg(heads=5, dim=4, vdim=36)],
                    [None, moe(ff=32, experts=3, identity=1, top=1, shared=0), dense(56, limit=1.2)], width=48,
                    vocab=131, groups=1, emb_scale=None),
    "one": config([attn(heads=1, kv_heads=1, dim=32, vdim=16, dims=32, softcap=50.0, scale=0.4), hg(heads=2, dim=20, vdim=8)],
                  [moe(ff=8, experts=1, identity=0, top=1, shared=24), None], width=40, vocab=97, groups=4,
                  emb_scale=0.5),
    # (attention shapes of a kind the tensor-core kernels take in bfloat16: values as wide as keys of 64, twice as wide)
    "wide": config([attn(heads=4, kv_heads=2, dim=64, vdim=64, dims=32, base=250000.0,
                         scaling={"factor": 16.0, "original": 32, "fast": 8.0, "slow": 1.0}, softcap=20.0),
                    hg(heads=2, dim=128, vdim=96), attn(heads=2, kv_heads=1, dim=64, vdim=128, dims=16, softcap=5.0),
                    hg(heads=3, dim=48, vdim=72)],
                   [moe(ff=40, experts=16, identity=3, top=3, shared=72), dense(136, limit=0.9),
                    moe(ff=24, experts=2, identity=6, top=4, shared=0), moe(ff=32, experts=9, identity=1, top=2, shared=16)],
                   width=96, vocab=257, groups=2, eps=1e-6, emb_scale=3.5),
    "two": config([hg(heads=2, dim=8, vdim=8), attn(dims=4, scaling={"factor": 2.0, "original": 16, "fast": 4.0,
                                                                      "slow": 0.5})],
                  [dense(48, limit=10.0), dense(48, limit=0.3)], width=56, vocab=89, groups=2, emb_scale=1.0),
}


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> bfloat16 tensor. Matrices N(0, 1/fan_in) so activations stay of order one; norm gains 1 + N(0, 0.2);
    lower bounds of the forget gate spread over (0, 0.9) and its biases spread, so that heads remember for a few and for
    many tokens; router rows large so that few choices are close calls; corrections of the size of a score."""
    from cuca_b200.config.registry import build_spec
    from cuca_b200.models.model import Model

    needs = Model(build_spec(cfg), runtime=None).tensor_needs()
    rng = np.random.default_rng(seed)
    out = {}
    for name, need in sorted(needs.items()):
        shape = tuple(need.shape)
        if name.endswith(".lower"):
            v = rng.uniform(0.0, 0.9, shape)
        elif name.endswith(".f.b"):
            v = rng.normal(1.0, 1.5, shape)
        elif name.endswith(".correction"):
            v = rng.normal(0.0, 0.5 / shape[0], shape)
        elif need.init == "ones":
            v = 1.0 + rng.normal(0.0, 0.2, shape)
        elif name.endswith(".router"):
            v = rng.normal(0.0, 3.0, shape) / np.sqrt(shape[-1])
        elif name == "embed":
            v = rng.normal(0.0, 1.0, shape)
        else:
            v = rng.normal(0.0, 1.0, shape) / np.sqrt(shape[-1])
        out[name] = torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16)
    return out


class Oracle:
    """Whole-sequence logits of the plain implementation, cached per request (the interface `replay_util.compare`
    takes)."""

    def __init__(self, cfg: dict, weights: dict):
        self.cfg, self.w = cfg, plain_weights(weights)
        self._cache = {}

    def logits(self, rid: str, tokens: list) -> np.ndarray:
        if rid not in self._cache:
            self._cache[rid] = plain_pudinex.forward(self.cfg, self.w, tokens)
        return self._cache[rid]

    def tolerance(self, dtype: str, requests: dict) -> float:
        """What a replay may differ by, relative to a row's largest logit. 32-bit: a fixed small number. bfloat16:
        three times what rounding alone does to these very requests (the plain implementation run once more with
        everything that enters a contraction, and the cached keys and values, rounded to bfloat16), at least 3e-2."""
        if dtype == "float32":
            return 1e-4
        errs = []
        for rid, tokens in requests.items():
            key = ("rounded", rid)
            if key not in self._cache:
                plain_pudinex.ROUND = bf16_round
                try:
                    self._cache[key] = plain_pudinex.forward(self.cfg, self.w, tokens)
                finally:
                    plain_pudinex.ROUND = None
            exact = self.logits(rid, tokens)
            errs.append(np.abs(self._cache[key] - exact).max(axis=1) / np.abs(exact).max(axis=1))
        # the median row: a routed layer takes another expert here and there once its input is rounded, and such a
        # row's error says nothing about rounding
        return max(3e-2, 3.0 * float(np.median(np.concatenate(errs))) * 2.0)


def compare(steps, got, requests, oracle, dtype, allow=0.10, tol32=None):
    """`replay_util.compare` for a model with routed layers: in bfloat16 a token whose choice scores nearly tie at the
    cut may go to another expert than in the plain implementation (and what it then leaves in the layers' states and
    keys moves the tokens after it a little), so up to `allow` of the wanted places may be off by more than the
    tolerance while the median place stays well inside it (never in 32-bit, and never by a non-finite value)."""
    import replay_util as ru
    tol = oracle.tolerance(dtype, requests)
    if dtype == "float32":
        return ru.compare(steps, got, requests, oracle, tol32 or tol)
    pos = {rid: 0 for rid in requests}
    errs = []
    for s in steps:
        row = 0
        for e in s["entries"]:
            ref = oracle.logits(e["id"], requests[e["id"]])
            for w in e.get("want", []):
                r, g = ref[pos[e["id"]] + w], got[s["step"]][row]
                assert np.isfinite(g).all(), (s["step"], e["id"])
                errs.append((float(np.abs(g - r).max()) / float(np.abs(r).max()), s["step"], e["id"], pos[e["id"]] + w))
                row += 1
            pos[e["id"]] += len(e["tokens"])
    over = [x for x in errs if x[0] > tol]
    assert len(over) <= max(1, allow * len(errs)), f"{len(over)} of {len(errs)} places over {tol:.2e}; first: {over[:3]}"
    assert float(np.median([x[0] for x in errs])) < 0.5 * tol
    return max(x[0] for x in errs)
