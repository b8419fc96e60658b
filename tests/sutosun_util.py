"""Small Sutosun configurations with weights that exercise every mechanism, for the engine and for the plain
implementation alike (the same values, bfloat16-rounded, as a folder and as 64-bit arrays)."""
from __future__ import annotations

import copy

import numpy as np
import torch

import plain_sutosun
from bananex_util import bf16_round, plain_weights, random_tokens, write_model  # noqa: F401  (shared helpers)

YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}


def attn(heads=4, kv_heads=2, dim=16, vdim=24, scale=None, coef=0.4, every=7):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else dim ** -0.5}
    if coef is not None:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m}


def ret(heads=3, dim=12, vdim=20, decay=None, dims=8, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim,
         "decay": list(decay) if decay is not None else [1.0 - 2.0 ** -(2 + 2 * a) for a in range(heads)]}
    if dims:
        m["rot"] = {"base": base, "dims": dims}
    return {"type": "retention", "mixer": m}


def lat(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=None, base=10000.0, scaling=YARN, rotated=True):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if rotated and rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    return {"type": "latent_attention", "mixer": m}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(ff=24, experts=5, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, mlps, width=60, vocab=199, eps=1e-5, softcap=12.0, weights_of=None):
    """`weights_of`: {entry: the entry whose tensors it runs with}; such an entry repeats the other's sizes."""
    out = []
    for i, (l, m) in enumerate(zip(layers, mlps)):
        j = (weights_of or {}).get(i)
        if j is not None:
            l, m = layers[j], mlps[j]
        l = copy.deepcopy(l)
        l["mlp"] = copy.deepcopy(m)
        if j is not None:
            l["weights_of"] = j
        out.append(l)
    cfg = {"architecture": "Sutosun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": out}
    if softcap is not None:
        cfg["logit_softcap"] = softcap
    return cfg


# sizes that differ in every respect: the order of the layers, key heads shared or not, one head, values wider and
# narrower than keys and as wide, a query temperature that starts early, late or not at all, rotation of all, part or
# none of a head with and without scaled frequencies, decays from fast to none, layers without a feed-forward, layers
# that run with an earlier and with a later layer's tensors, one expert of one, all experts chosen, no cap on the logits
CONFIGS = {
    "mix": config([lat(), attn(), ret(), attn(), lat(heads=2, dim=8, rot_dim=4, vdim=12, kv_rank=24, scaling=None), ret()],
                  [dense(), moe(), moe(ff=16, experts=4, top=4), None, dense(40), None], weights_of={3: 1, 5: 2}),
    "plain": config([attn(heads=3, kv_heads=3, vdim=16, coef=None), ret(heads=1, dim=40, vdim=8, decay=[1.0], dims=0),
                     lat(heads=5, dim=4, rot_dim=0, vdim=36, kv_rank=8)],
                    [None, moe(ff=32, experts=3, top=1), dense(56)], width=48, vocab=131, softcap=None),
    "one": config([ret(heads=2, dim=20, vdim=8, decay=[0.5, 0.96875], dims=20, base=500.0),
                   attn(heads=1, kv_heads=1, dim=32, vdim=16, scale=0.4, coef=1.5, every=1),
                   lat(heads=1, dim=24, rot_dim=16, vdim=8, kv_rank=16, scale=0.3, rotated=False)],
                  [moe(ff=8, experts=1, top=1), None, dense(24)], width=40, vocab=97, softcap=3.0, eps=1e-6),
    # (shapes of a kind the tensor-core kernels take in bfloat16: keys of 64 and 128 with values as wide, a latent of
    # 64 + 16; the first entry runs with the tensors of a later one)
    "wide": config([attn(heads=4, kv_heads=2, dim=64, vdim=64, coef=0.25, every=100), ret(heads=2, dim=128, vdim=96, dims=64),
                    attn(heads=4, kv_heads=2, dim=64, vdim=64, coef=0.25, every=100),
                    lat(heads=4, dim=32, rot_dim=16, vdim=48, kv_rank=64, base=250000.0,
                        scaling={"factor": 16.0, "original": 32, "fast": 8.0, "slow": 1.0}),
                    attn(heads=2, kv_heads=1, dim=128, vdim=128, coef=None)],
                   [moe(ff=40, experts=12, top=3), dense(136), moe(ff=40, experts=12, top=3),
                    moe(ff=32, experts=9, top=2), None],
                   width=96, vocab=257, weights_of={0: 2}),
    "two": config([ret(heads=2, dim=8, vdim=8, dims=4), lat(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16,
                                                           scaling={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5})],
                  [dense(48), dense(48)], width=56, vocab=89, softcap=30.0),
}


def draw(name: str, need, rng) -> np.ndarray:
    """One tensor's values. Matrices N(0, 1/fan_in) so activations stay of order one; norm gains 1 + N(0, 0.2); sink
    scores and biases of a score's size; router rows large so that few choices are close calls."""
    shape = tuple(need.shape)
    if name.endswith(".sink"):
        return rng.normal(0.0, 1.5, shape)
    if name.endswith(".router.b"):
        return rng.normal(0.0, 1.0, shape)
    if name.endswith(".b"):
        return rng.normal(0.0, 0.5, shape)
    if need.init == "ones":
        return 1.0 + rng.normal(0.0, 0.2, shape)
    if name.endswith(".router"):
        return rng.normal(0.0, 3.0, shape) / np.sqrt(shape[-1])
    if name == "embed":
        return rng.normal(0.0, 1.0, shape)
    return rng.normal(0.0, 1.0, shape) / np.sqrt(shape[-1])


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> bfloat16 tensor for every tensor the model asks for."""
    from cuca_b200.config.registry import build_spec
    from cuca_b200.models.model import Model

    needs = Model(build_spec(cfg), runtime=None).tensor_needs()
    rng = np.random.default_rng(seed)
    return {name: torch.from_numpy(np.asarray(draw(name, need, rng), dtype=np.float32)).to(torch.bfloat16)
            for name, need in sorted(needs.items())}


class Oracle:
    """Whole-sequence logits of the plain implementation, cached per request (the interface `replay_util.compare`
    takes)."""

    def __init__(self, cfg: dict, weights: dict):
        self.cfg, self.w = cfg, plain_weights(weights)
        self._cache = {}

    def logits(self, rid: str, tokens: list) -> np.ndarray:
        if rid not in self._cache:
            self._cache[rid] = plain_sutosun.forward(self.cfg, self.w, tokens)
        return self._cache[rid]

    def rounded(self, rid: str, tokens: list) -> np.ndarray:
        """The plain implementation's logits with everything that enters a contraction, and what the caches hold,
        rounded to bfloat16."""
        key = ("rounded", rid)
        if key not in self._cache:
            plain_sutosun.ROUND = bf16_round
            try:
                self._cache[key] = plain_sutosun.forward(self.cfg, self.w, tokens)
            finally:
                plain_sutosun.ROUND = None
        return self._cache[key]

    def tolerance(self, dtype: str, requests: dict) -> float:
        """What a replay may differ by, relative to a row's largest logit. 32-bit: a fixed small number. bfloat16:
        three times what rounding alone does to these very requests (the plain implementation run once more with
        everything that enters a contraction, and what the caches hold, rounded to bfloat16), at least 3e-2."""
        if dtype == "float32":
            return 1e-4
        errs = []
        for rid, tokens in requests.items():
            exact = self.logits(rid, tokens)
            errs.append(np.abs(self.rounded(rid, tokens) - exact).max(axis=1) / np.abs(exact).max(axis=1))
        # the median row: a routed layer takes another expert here and there once its input is rounded, and such a
        # row's error says nothing about rounding
        return max(3e-2, 3.0 * float(np.median(np.concatenate(errs))) * 2.0)


def compare(steps, got, requests, oracle, dtype, allow=0.10, tol32=None):
    """`replay_util.compare` for a model with routed layers. 32-bit: every wanted place within the tolerance of the
    plain implementation. bfloat16: a token whose router logits nearly tie at the cut may go to another expert once its
    input is rounded, and what it then leaves in the states and keys moves the tokens after it; the plain
    implementation with rounded inputs takes the same turn. So a place is measured against the exact logits and against
    the rounded ones and the smaller distance counts; up to `allow` of the places may still be over the tolerance (a
    tie that falls the other way) while the median place stays well inside it, and never by a non-finite value."""
    import replay_util as ru
    tol = oracle.tolerance(dtype, requests)
    if dtype == "float32":
        return ru.compare(steps, got, requests, oracle, tol32 or tol)
    pos = {rid: 0 for rid in requests}
    errs = []
    for s in steps:
        row = 0
        for e in s["entries"]:
            rid = e["id"]
            ref, near = oracle.logits(rid, requests[rid]), oracle.rounded(rid, requests[rid])
            for w in e.get("want", []):
                p, g = pos[rid] + w, got[s["step"]][row]
                assert np.isfinite(g).all(), (s["step"], rid)
                scale = float(np.abs(ref[p]).max())
                errs.append((min(float(np.abs(g - ref[p]).max()), float(np.abs(g - near[p]).max())) / scale, s["step"], rid, p))
                row += 1
            pos[rid] += len(e["tokens"])
    over = [x for x in errs if x[0] > tol]
    assert len(over) <= max(1, allow * len(errs)), f"{len(over)} of {len(errs)} places over {tol:.2e}; first: {over[:3]}"
    assert float(np.median([x[0] for x in errs])) < 0.5 * tol
    return max(x[0] for x in errs)
