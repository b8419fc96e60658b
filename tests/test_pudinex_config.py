"""Pudinex without a GPU: the configuration reader and its refusals, caches per layer, tensor names, a folder of
random weights, the rotation tables, and properties of the plain implementation itself."""
import copy
import math

import numpy as np
import pytest

import plain_pudinex as pp
import pudinex_util as pu
from cuca_b200.config.model_config import ConfigError
from cuca_b200.config.pudinex_config import PudinexConfig
from cuca_b200.config.registry import architectures, build_spec
from cuca_b200.models.model import Model
from cuca_b200.weights.loader import WeightsError, check_tensors


def test_registered_and_read():
    assert "Pudinex" in architectures()
    cfg = PudinexConfig.from_json(pu.CONFIGS["mix"])
    assert cfg.norm_groups == 3 and cfg.embedding_scale == 2.0 and len(cfg.layers) == 4
    assert [l.type for l in cfg.layers] == ["hgrn2", "attention", "hgrn2", "attention"]
    a = cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.rot_dims, a.softcap) == (4, 2, 16, 24, 8, 8.0)
    assert a.yarn.factor == 4.0 and a.yarn.original == 64
    b = cfg.layers[3].mixer
    assert b.yarn is None and b.softcap is None and b.rot_dims == 12
    assert cfg.layers[0].mlp.kind == "dense" and cfg.layers[0].mlp.limit == 0.6
    m = cfg.layers[1].mlp
    assert (m.kind, m.experts, m.identity, m.top, m.shared, m.ff) == ("moe", 5, 2, 2, 40, 24)
    assert cfg.layers[2].mlp.identity == 0 and cfg.layers[2].mlp.shared == 0
    plain = PudinexConfig.from_json(pu.CONFIGS["plain"])
    assert plain.norm_groups == 1 and plain.embedding_scale == 1.0 and plain.layers[0].mlp is None
    assert plain.layers[0].mixer.rot_dims == 0
    # absent keys: as many key heads as heads, values as wide as keys
    bare = copy.deepcopy(pu.CONFIGS["mix"])
    del bare["layers"][1]["mixer"]["kv_heads"], bare["layers"][1]["mixer"]["vdim"]
    c = PudinexConfig.from_json(bare).layers[1].mixer
    assert c.kv_heads == 4 and c.vdim == 16


@pytest.mark.parametrize("path, value", [
    (("layers", 0, "type"), "conv_only"), (("layers", 1, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "dim"), 0),
    (("layers", 1, "mixer", "rot", "dims"), 7), (("layers", 1, "mixer", "rot", "dims"), 18),
    (("layers", 1, "mixer", "softcap"), -1.0), (("layers", 1, "mixer", "rot", "scaling", "factor"), 0.0),
    (("layers", 1, "mlp", "router", "top"), 8), (("layers", 1, "mlp", "kind"), "sparse"),
    (("layers", 0, "mlp", "limit"), 0.0), (("norm", "groups"), 7), (("norm",), None), (("layers", 0, "mixer"), None),
    (("layers", 1, "mlp", "expert"), None)])
def test_refusals_name_the_key(path, value):
    cfg = copy.deepcopy(pu.CONFIGS["mix"])
    node = cfg
    for k in path[:-1]:
        node = node[k]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        PudinexConfig.from_json(cfg)
    assert str(path[-1]) in str(e.value) or str(path[-2]) in str(e.value)


def test_a_cache_per_layer():
    for name, cfg in pu.CONFIGS.items():
        spec = build_spec(cfg)
        runs = spec.runs()
        assert [r.layer for r in runs] == list(range(len(cfg["layers"]))) and all(r.owns for r in runs)
        needs = Model(spec, runtime=None).cache_needs()
        for r in runs:
            layer = cfg["layers"][r.layer]
            m, n = layer["mixer"], needs[r.cache]
            if layer["type"] == "attention":
                assert n.state is None and n.kv.n_kv_heads == m["kv_heads"] and n.kv.head_dim == m["dim"]
                assert (n.kv.v_head_dim or n.kv.head_dim) == m["vdim"] and n.kv.window is None
            else:
                assert n.kv is None and n.state["memory"].shape == (m["heads"], m["vdim"], m["dim"])


def test_tensor_names_and_shapes():
    cfg = pu.CONFIGS["mix"]
    model = Model(build_spec(cfg), runtime=None)
    needs = model.tensor_needs()
    for name in ("embed", "head", "final.norm", "l0.norm1", "l0.mix.q", "l0.mix.f", "l0.mix.f.b", "l0.mix.lower",
                 "l0.mix.v", "l0.mix.norm", "l0.mix.o", "l0.mlp.gate", "l1.mix.q.norm", "l1.mix.k.norm", "l1.mix.k",
                 "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e4.gate", "l1.mlp.shared.down", "l2.mlp.e3.up"):
        assert name in needs, name
    assert "l1.mlp.e5.up" not in needs and "l2.mlp.shared.gate" not in needs and "l0.norm2" not in needs
    assert needs["l1.mlp.router"].shape == (7, 60) and needs["l1.mlp.correction"].shape == (7,)
    assert needs["l0.mix.lower"].shape == (36,) and needs["l0.mix.norm"].shape == (20,)
    assert needs["l1.mix.q.norm"].shape == (16,) and needs["l1.mix.v"].shape == (48, 60)
    assert needs["l1.mlp.shared.gate"].shape == (40, 60)
    shapes = {n: tuple(t.shape) for n, t in needs.items()}
    check_tensors(needs, shapes)
    shapes["l1.mlp.router"] = (5, 60)  # the router has an output for every expert, also for those without weights
    with pytest.raises(WeightsError) as e:
        check_tensors(needs, shapes)
    assert [w[0] for w in e.value.wrong_shape] == ["l1.mlp.router"]


def test_a_folder_of_random_weights(tmp_path):
    from cuca_b200.weights.loader import FolderSource, write_model_folder
    cfg = pu.CONFIGS["two"]
    model = Model(build_spec(cfg), runtime=None)
    write_model_folder(tmp_path, cfg, model.tensor_needs(), seed=3, norm_std=0.2)
    model.check_weights(FolderSource(tmp_path))


@pytest.mark.parametrize("rot", [{"base": 10000.0, "dims": 8, "scaling": pu.YARN},
                                 {"base": 250000.0, "dims": 32, "scaling": {"factor": 16.0, "original": 32, "fast": 8.0, "slow": 1.0}},
                                 {"base": 100.0, "dims": 6, "scaling": {"factor": 2.0, "original": 4096, "fast": 64.0, "slow": 0.25}},
                                 {"base": 10000.0, "dims": 4}])
def test_rotation_tables_are_the_plain_frequencies(rot):
    """The engine's cos and sin tables against angles made from the plain implementation's frequencies."""
    from cuca_b200.parts.base import PartSpec
    from cuca_b200.parts.rope import RotaryEncoding
    sc = dict(rot["scaling"], kind="yarn") if rot.get("scaling") else None
    part = RotaryEncoding(PartSpec("rope", {"head_dim": 40, "rotary_dim": rot["dims"], "theta": rot["base"],
                                            "scaling": sc}), None)
    cos, sin = part.host_tables(300)
    f, mag = pp.yarn_frequencies(rot)
    ang = np.arange(300)[:, None] * f[None, :]
    assert np.abs(cos.numpy() - np.cos(ang) * mag).max() < 1e-6 and np.abs(sin.numpy() - np.sin(ang) * mag).max() < 1e-6
    if sc:
        plain = np.array([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)])
        assert np.isclose(f[0], plain[0]) or rot["dims"] == 6  # the fastest pair turns as it would unscaled
        assert mag == pytest.approx(0.1 * math.log(sc["factor"]) + 1.0)
        assert (f <= plain + 1e-15).all() and (f >= plain / sc["factor"] - 1e-15).all()


# ------------------------------------------------------------------------------------------ the plain implementation
def _w(cfg, seed):
    return pu.plain_weights(pu.make_weights(cfg, seed))


@pytest.mark.parametrize("name", list(pu.CONFIGS))
def test_plain_is_causal_and_carries_the_first_token(name):
    cfg = pu.CONFIGS[name]
    w = _w(cfg, 1)
    toks = pu.random_tokens(30, cfg["vocab"], 2)
    a = pp.forward(cfg, w, toks)
    b = pp.forward(cfg, w, toks[:20] + pu.random_tokens(10, cfg["vocab"], 3))
    assert np.array_equal(a[:20], b[:20]) and not np.allclose(a[20:], b[20:])
    c = pp.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert not np.allclose(a[-1], c[-1])


def test_plain_norm_parts_are_normed_apart():
    x = np.random.default_rng(0).normal(size=(3, 12)) * np.array([1.0] * 4 + [100.0] * 4 + [0.01] * 4)
    y = pp.group_norm(x, np.ones(12), 3, 0.0)
    for part in range(3):
        assert np.allclose(np.mean(y[:, 4 * part:4 * part + 4] ** 2, axis=1), 1.0)
    assert not np.allclose(np.mean(pp.group_norm(x, np.ones(12), 1, 0.0)[:, :4] ** 2, axis=1), 1.0)


def test_plain_sink_and_cap():
    """One token: the softmax has two terms, the key's exp(s) and the sink's exp(0), so the output is the normed value
    times exp(s) / (1 + exp(s)); a huge score is capped to `softcap`."""
    E, d, dv = 6, 4, 3
    rs = np.random.default_rng(1)
    w = {"q": rs.normal(size=(d, E)), "k": rs.normal(size=(d, E)), "v": rs.normal(size=(dv, E)),
         "q.norm": np.full(d, 30.0), "k.norm": np.full(d, 30.0), "o": np.eye(dv)}
    h = rs.normal(size=(1, E))
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": dv, "scale": 1.0, "softcap": 2.0}
    q, k = pp.rms(w["q"] @ h[0], 1e-6) * 30.0, pp.rms(w["k"] @ h[0], 1e-6) * 30.0
    v = pp.rms(w["v"] @ h[0], 1e-6)
    s = 2.0 * np.tanh((q @ k) / 2.0)
    assert abs(q @ k) > 20 and abs(s) <= 2.0
    out = pp.sink_attention(h, w, "", m, 1e-6)
    assert np.allclose(out[0], v * np.exp(s) / (1.0 + np.exp(s)))
    m["softcap"] = None
    out = pp.sink_attention(h, w, "", m, 1e-6)
    assert np.allclose(out[0], v * (1.0 / (1.0 + np.exp(-(q @ k)))))


def test_plain_forget_gate_stays_above_its_lower_bound_and_first_token():
    m = {"heads": 1, "dim": 3, "vdim": 2}
    E = 4
    rs = np.random.default_rng(2)
    w = {"q": rs.normal(size=(3, E)), "f": rs.normal(size=(3, E)), "f.b": np.array([-50.0, 0.0, 50.0]),
         "lower": np.array([0.25, 0.5, 0.75]), "v": rs.normal(size=(2, E)), "norm": np.ones(2), "o": np.eye(2)}
    h = rs.normal(size=(1, E)) * 0.1
    f = w["lower"] + (1 - w["lower"]) * pp.sigmoid(w["f"] @ h[0] + w["f.b"])
    assert np.isclose(f[0], 0.25) and np.isclose(f[2], 1.0) and 0.5 < f[1] < 1.0
    q, v = pp.silu(w["q"] @ h[0]), w["v"] @ h[0]
    o = np.outer(1.0 - f, v).T @ q  # the state after the first token is (1 - f) v^T
    assert np.allclose(pp.hgrn2(h, w, "", m, 1e-6)[0], o / np.sqrt(np.mean(o * o) + 1e-6))


def test_plain_experts_chosen_by_corrected_scores_and_weighted_by_plain_ones():
    mlp = pu.moe(ff=4, experts=3, identity=2, top=2, shared=5)
    rs = np.random.default_rng(3)
    E = 6
    w = {"router": rs.normal(size=(5, E)), "correction": np.array([0.0, 0.0, 5.0, 0.0, 5.0])}
    for e in list(range(3)) + ["shared"]:
        p = f"e{e}." if e != "shared" else "shared."
        n = 5 if e == "shared" else 4
        w[p + "gate"], w[p + "up"], w[p + "down"] = rs.normal(size=(n, E)), rs.normal(size=(n, E)), rs.normal(size=(E, n))
    f = rs.normal(size=(4, E))
    got = pp.routed_ff(f, w, "", mlp)
    z = f @ w["router"].T
    s = np.exp(z) / np.exp(z).sum(1, keepdims=True)
    for t in range(4):
        g2, g4 = s[t, 2] / (s[t, 2] + s[t, 4]), s[t, 4] / (s[t, 2] + s[t, 4])  # the correction decides, the score weighs
        want = g2 * pp.silu_glu(f[t:t + 1], w, "e2.")[0] + g4 * f[t] + pp.silu_glu(f[t:t + 1], w, "shared.")[0]
        assert np.allclose(got[t], want)


def test_plain_capped_unit():
    E = 3
    w = {"gate": np.eye(E), "up": np.eye(E), "down": np.eye(E)}
    f = np.array([[5.0, -5.0, 0.5]])
    g, u = np.array([2.0, -5.0, 0.5]), np.array([2.0, -2.0, 0.5])  # the gate is capped from above only
    assert np.allclose(pp.capped_glu(f, w, "", 2.0)[0], g * pp.sigmoid(1.702 * g) * (u + 1.0))
