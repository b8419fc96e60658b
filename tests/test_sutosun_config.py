"""Sutosun without a GPU: the configuration reader and its refusals, the run order with layers that borrow another
layer's tensors, caches per run, tensor names, a folder of random weights, the rotation tables, and properties of the
plain implementation itself."""
import copy
import math

import numpy as np
import pytest

import plain_sutosun as ps
import sutosun_util as su
from cuca_b200.config.model_config import ConfigError
from cuca_b200.config.registry import architectures, build_spec
from cuca_b200.config.sutosun_config import SutosunConfig
from cuca_b200.models.model import Model
from cuca_b200.weights.loader import WeightsError, check_tensors


def test_registered_and_read():
    assert "Sutosun" in architectures()
    cfg = SutosunConfig.from_json(su.CONFIGS["mix"])
    assert cfg.logit_softcap == 12.0 and cfg.eps == 1e-5 and len(cfg.layers) == 6
    assert [l.type for l in cfg.layers] == ["latent_attention", "attention", "retention", "attention",
                                            "latent_attention", "retention"]
    a = cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.q_temp_coef, a.q_temp_every) == (4, 2, 16, 24, 0.4, 7)
    r = cfg.layers[2].mixer
    assert (r.heads, r.dim, r.vdim, r.rot.dims, r.rot.yarn) == (3, 12, 20, 8, None) and r.decay == (0.75, 0.9375, 0.984375)
    l = cfg.layers[0].mixer
    assert (l.heads, l.dim, l.rot_dim, l.vdim, l.kv_rank, l.rot.dims) == (3, 16, 8, 24, 40, 8)
    assert l.rot.yarn.factor == 4.0 and l.rot.yarn.original == 64 and cfg.layers[4].mixer.rot.yarn is None
    assert [x.weights_of for x in cfg.layers] == [None, None, None, 1, None, 2]
    assert [cfg.weights_layer(i) for i in range(6)] == [0, 1, 2, 1, 4, 2]
    m = cfg.layers[1].mlp
    assert (m.kind, m.experts, m.top, m.ff) == ("moe", 5, 2, 24) and cfg.layers[0].mlp.kind == "dense"
    plain = SutosunConfig.from_json(su.CONFIGS["plain"])
    assert plain.logit_softcap is None and plain.layers[0].mlp is None and plain.layers[0].mixer.q_temp_coef is None
    assert plain.layers[1].mixer.rot is None and plain.layers[2].mixer.rot is None
    # absent keys: as many key heads as heads, values as wide as keys
    bare = copy.deepcopy(su.CONFIGS["mix"])
    del bare["layers"][1]["mixer"]["kv_heads"], bare["layers"][1]["mixer"]["vdim"]
    bare["layers"][3] = copy.deepcopy(bare["layers"][1]) | {"weights_of": 1}
    c = SutosunConfig.from_json(bare).layers[1].mixer
    assert c.kv_heads == 4 and c.vdim == 16


@pytest.mark.parametrize("path, value", [
    (("layers", 0, "type"), "conv_only"), (("layers", 1, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "dim"), 0),
    (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "rot", "dims"), 10),
    (("layers", 2, "mixer", "rot", "dims"), 14), (("layers", 2, "mixer", "decay"), [0.5, 0.9]),
    (("layers", 2, "mixer", "decay"), None), (("layers", 1, "mixer", "q_temp", "every"), 0),
    (("layers", 0, "mixer", "rot", "scaling", "factor"), 0.0), (("layers", 1, "mlp", "router", "top"), 6),
    (("layers", 1, "mlp", "kind"), "sparse"), (("norm",), None), (("layers", 0, "mixer"), None),
    (("layers", 1, "mlp", "expert"), None), (("layers", 3, "weights_of"), 3), (("layers", 3, "weights_of"), 9),
    (("layers", 3, "weights_of"), 0), (("logit_softcap",), -2.0)])
def test_refusals_name_the_key(path, value):
    cfg = copy.deepcopy(su.CONFIGS["mix"])
    node = cfg
    for k in path[:-1]:
        node = node[k]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        SutosunConfig.from_json(cfg)
    assert str(path[-1]) in str(e.value) or str(path[-2]) in str(e.value)


def test_every_entry_is_a_run_with_a_cache_of_its_own():
    """An entry that borrows tensors runs the lender's parts; caches and states are per entry."""
    for name, cfg in su.CONFIGS.items():
        spec = build_spec(cfg)
        runs = spec.runs()
        assert [r.cache for r in runs] == list(range(len(cfg["layers"]))) and all(r.owns for r in runs)
        own = [i for i, l in enumerate(cfg["layers"]) if l.get("weights_of") is None]
        assert len(spec.layers) == len(own)
        for i, r in enumerate(runs):
            lender = cfg["layers"][i].get("weights_of")
            assert r.layer == own.index(i if lender is None else lender)
        needs = Model(spec, runtime=None).cache_needs()
        for i, layer in enumerate(cfg["layers"]):
            m, n = layer["mixer"], needs[i]
            if layer["type"] == "attention":
                assert n.state is None and n.kv.n_kv_heads == m["kv_heads"] and n.kv.head_dim == m["dim"]
                assert (n.kv.v_head_dim or n.kv.head_dim) == m["vdim"] and n.kv.window is None
            elif layer["type"] == "latent_attention":
                assert n.state is None and n.kv.n_kv_heads == 1 and n.kv.head_dim == m["kv_rank"] + m["rot_dim"]
                assert n.kv.v_head_dim == 0
            else:
                assert n.kv is None and n.state["memory"].shape == (m["heads"], m["vdim"], m["dim"])
    wide = build_spec(su.CONFIGS["wide"])  # the first entry borrows from a later one
    assert [r.layer for r in wide.runs()] == [1, 0, 1, 2, 3]


def test_tensor_names_and_shapes():
    cfg = su.CONFIGS["mix"]
    model = Model(build_spec(cfg), runtime=None)
    needs = model.tensor_needs()
    for name in ("embed", "embed.norm", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.dkv",
                 "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.sink", "l0.mix.o", "l0.mlp.gate", "l0.mlp.up",
                 "l0.mlp.down", "l1.mix.q", "l1.mix.q.b", "l1.mix.k.b", "l1.mix.v.b", "l1.mix.q.norm", "l1.mix.k.norm",
                 "l1.mix.sink", "l1.mix.g", "l1.mlp.router", "l1.mlp.router.b", "l1.mlp.e4.gate", "l2.mix.q", "l2.mix.k",
                 "l2.mix.v", "l2.mix.g", "l2.mix.o", "l2.mlp.e3.down", "l4.mix.sink"):
        assert name in needs, name
    # entries that borrow have no tensors; a latent layer has no gate; a layer without a feed-forward no second norm
    assert not [n for n in needs if n.startswith(("l3.", "l5."))]
    assert "l0.mix.g" not in needs and "l1.mlp.e5.up" not in needs
    assert needs["l1.mix.q.norm"].shape == (64,) and needs["l1.mix.k.norm"].shape == (32,)
    assert needs["l1.mix.g"].shape == (4, 60) and needs["l1.mix.sink"].shape == (4,)
    assert needs["l1.mix.v"].shape == (48, 60) and needs["l1.mix.v.b"].shape == (48,) and needs["l1.mix.o"].shape == (60, 96)
    assert needs["l0.mix.q"].shape == (72, 60) and needs["l0.mix.dkv"].shape == (48, 60) and needs["l0.mix.uk"].shape == (48, 40)
    assert needs["l0.mix.uv"].shape == (72, 40) and needs["l0.mix.dkv.norm"].shape == (40,)
    assert needs["l2.mix.q"].shape == (36, 60) and needs["l2.mix.g"].shape == (60, 60)
    assert needs["l1.mlp.router"].shape == (5, 60) and needs["l1.mlp.router.b"].shape == (5,)
    plain = Model(build_spec(su.CONFIGS["plain"]), runtime=None).tensor_needs()
    assert "l0.norm2" not in plain and "l0.norm1" in plain
    shapes = {n: tuple(t.shape) for n, t in needs.items()}
    check_tensors(needs, shapes)
    shapes["l1.mix.g"] = (96, 60)  # one gate per head, not per value
    with pytest.raises(WeightsError) as e:
        check_tensors(needs, shapes)
    assert [w[0] for w in e.value.wrong_shape] == ["l1.mix.g"]


def test_a_folder_of_random_weights(tmp_path):
    from cuca_b200.weights.loader import FolderSource, write_model_folder
    cfg = su.CONFIGS["two"]
    model = Model(build_spec(cfg), runtime=None)
    write_model_folder(tmp_path, cfg, model.tensor_needs(), seed=3, norm_std=0.2)
    model.check_weights(FolderSource(tmp_path))


@pytest.mark.parametrize("rot", [{"base": 10000.0, "dims": 8, "scaling": su.YARN},
                                 {"base": 250000.0, "dims": 32, "scaling": {"factor": 16.0, "original": 32, "fast": 8.0, "slow": 1.0}},
                                 {"base": 100.0, "dims": 6, "scaling": {"factor": 2.0, "original": 4096, "fast": 64.0, "slow": 0.25}},
                                 {"base": 500.0, "dims": 20}])
def test_rotation_tables_are_the_plain_frequencies(rot):
    """The engine's cos and sin tables, as the model builder asks for them, against angles made from the plain
    implementation's frequencies."""
    from cuca_b200.config.sutosun_config import RotConfig
    from cuca_b200.models.sutosun import _rope
    from cuca_b200.parts.rope import RotaryEncoding
    part = RotaryEncoding(_rope(RotConfig.from_json(rot, "rot", 40), 40), None)
    assert part.pairs == "half" and part.rotary_dim == rot["dims"]
    cos, sin = part.host_tables(300)
    f, mag = ps.frequencies(rot)
    ang = np.arange(300)[:, None] * f[None, :]
    assert np.abs(cos.numpy() - np.cos(ang) * mag).max() < 1e-6 and np.abs(sin.numpy() - np.sin(ang) * mag).max() < 1e-6
    if rot.get("scaling"):
        plain = np.array([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)])
        assert mag == pytest.approx(0.1 * math.log(rot["scaling"]["factor"]) + 1.0)
        assert (f <= plain + 1e-15).all() and (f >= plain / rot["scaling"]["factor"] - 1e-15).all()
    else:
        assert mag == 1.0


# ------------------------------------------------------------------------------------------ the plain implementation
def _w(cfg, seed):
    return su.plain_weights(su.make_weights(cfg, seed))


@pytest.mark.parametrize("name", list(su.CONFIGS))
def test_plain_is_causal_and_carries_the_first_token(name):
    cfg = su.CONFIGS[name]
    w = _w(cfg, 1)
    toks = su.random_tokens(30, cfg["vocab"], 2)
    a = ps.forward(cfg, w, toks)
    b = ps.forward(cfg, w, toks[:20] + su.random_tokens(10, cfg["vocab"], 3))
    assert np.array_equal(a[:20], b[:20]) and not np.allclose(a[20:], b[20:])
    c = ps.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert not np.allclose(a[-1], c[-1])
    cap = cfg.get("logit_softcap")
    if cap:
        assert np.abs(a).max() < cap


def test_plain_layers_that_borrow_run_the_lenders_weights():
    """Two entries with the same tensors are the same function of the stream: with the lender's tensors written under
    a name of their own, the borrowing entry as an ordinary layer gives the same logits."""
    cfg = su.CONFIGS["mix"]
    w = _w(cfg, 4)
    toks = su.random_tokens(17, cfg["vocab"], 5)
    own = copy.deepcopy(cfg)
    for i, layer in enumerate(own["layers"]):
        j = layer.pop("weights_of", None)
        if j is not None:
            for name in [n for n in w if n.startswith(f"l{j}.")]:
                w[f"l{i}." + name.split(".", 1)[1]] = w[name]
    assert np.array_equal(ps.forward(cfg, w, toks), ps.forward(own, w, toks))


def test_plain_sink_with_one_key():
    """One token: the softmax has two terms, the key's exp(s) and the sink's exp(sink), so a head's output is its
    value times exp(s) / (exp(s) + exp(sink)), times the head's gate."""
    E, d, dv = 6, 4, 3
    rs = np.random.default_rng(1)
    w = {"q": rs.normal(size=(2 * d, E)), "k": rs.normal(size=(d, E)), "v": rs.normal(size=(dv, E)),
         "q.b": rs.normal(size=2 * d), "k.b": rs.normal(size=d), "v.b": rs.normal(size=dv),
         "q.norm": rs.normal(1, 0.2, 2 * d), "k.norm": rs.normal(1, 0.2, d), "sink": np.array([0.7, -1.1]),
         "g": rs.normal(size=(2, E)), "o": np.eye(2 * dv)}
    h = rs.normal(size=(1, E))
    m = {"heads": 2, "kv_heads": 1, "dim": d, "vdim": dv, "scale": 0.6, "q_temp": {"coef": 0.5, "every": 1}}
    q = ps.rms(w["q"] @ h[0] + w["q.b"], 1e-6) * w["q.norm"] * (1 + 0.5 * math.log(2))  # position 0: floor(1 / 1) + 1
    k = ps.rms(w["k"] @ h[0] + w["k.b"], 1e-6) * w["k.norm"]
    v = w["v"] @ h[0] + w["v.b"]
    out = ps.gated_attention(h, w, "", m, 1e-6)[0]
    for a in range(2):
        s = (q[a * d:(a + 1) * d] @ k) * 0.6
        gate = ps.sigmoid(w["g"][a] @ h[0])
        assert np.allclose(out[a * dv:(a + 1) * dv], v * np.exp(s) / (np.exp(s) + np.exp(w["sink"][a])) * gate)


def test_plain_query_temperature_steps():
    """The factor on the query is 1 below position every - 1 and grows by steps: 1 + coef ln(2) from every - 1 on."""
    E, d = 5, 4
    rs = np.random.default_rng(2)
    w = {"q": rs.normal(size=(d, E)), "k": rs.normal(size=(d, E)), "v": np.eye(d, E), "q.b": np.zeros(d),
         "k.b": np.zeros(d), "v.b": np.zeros(d), "q.norm": np.ones(d), "k.norm": np.ones(d), "sink": np.array([-50.0]),
         "g": np.zeros((1, E)), "o": np.eye(d)}
    h = rs.normal(size=(9, E))
    base = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": d, "scale": 1.0}
    cold = ps.gated_attention(h, w, "", base, 1e-6)
    warm = ps.gated_attention(h, w, "", dict(base, q_temp={"coef": 2.0, "every": 4}), 1e-6)
    assert np.allclose(cold[:3], warm[:3]) and not np.allclose(cold[3], warm[3])
    scaled = ps.gated_attention(h, w, "", dict(base, scale=1.0 + 2.0 * math.log(2)), 1e-6)
    assert np.allclose(warm[3:7], scaled[3:7]) and not np.allclose(warm[7], scaled[7])


def test_plain_retention_is_a_decaying_sum():
    """Without rotation o_t = sum_j decay^(t - j) (q_t . k_j) v_j / sqrt(dim), then the head's root mean square."""
    E, d, dv, T = 5, 4, 3, 7
    rs = np.random.default_rng(3)
    w = {"q": rs.normal(size=(d, E)), "k": rs.normal(size=(d, E)), "v": rs.normal(size=(dv, E)),
         "g": rs.normal(size=(dv, E)), "o": np.eye(dv)}
    h = rs.normal(size=(T, E))
    m = {"heads": 1, "dim": d, "vdim": dv, "decay": [0.8]}
    q, k, v = h @ w["q"].T, h @ w["k"].T / 2.0, h @ w["v"].T
    got = ps.retention(h, w, "", m, 1e-6)
    for t in range(T):
        o = sum(0.8 ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1))
        assert np.allclose(got[t], o / np.sqrt(np.mean(o * o) + 1e-6) * ps.silu(w["g"] @ h[t]))
    # a rotation of the whole head by the same angle on both sides leaves q . k of one position as it is
    m["rot"] = {"base": 100.0, "dims": 4}
    assert np.allclose(ps.retention(h, w, "", m, 1e-6)[0], got[0]) and not np.allclose(ps.retention(h, w, "", m, 1e-6)[3], got[3])


def test_plain_latent_keys_are_made_from_the_latent():
    """A head's key and value come from the normed latent alone; the turned part is shared by the heads."""
    E, T = 6, 5
    rs = np.random.default_rng(4)
    m = {"heads": 2, "dim": 3, "rot_dim": 2, "vdim": 4, "kv_rank": 5, "scale": 0.5, "rot": {"base": 50.0, "dims": 2}}
    w = {"q": rs.normal(size=(10, E)), "dkv": rs.normal(size=(7, E)), "dkv.norm": rs.normal(1, 0.2, 5),
         "uk": rs.normal(size=(6, 5)), "uv": rs.normal(size=(8, 5)), "sink": np.array([0.3, -0.4]), "o": np.eye(8)}
    h = rs.normal(size=(T, E))
    got = ps.latent_attention(h, w, "", m, 1e-6)
    down = h @ w["dkv"].T
    c = ps.rms(down[:, :5], 1e-6) * w["dkv.norm"]
    q = (h @ w["q"].T).reshape(T, 2, 5)
    turn = lambda v, p: np.array([v[0] * math.cos(p) - v[1] * math.sin(p), v[1] * math.cos(p) + v[0] * math.sin(p)])  # noqa: E731
    t = T - 1
    for a in range(2):
        s = np.array([(q[t, a, :3] @ (w["uk"][3 * a:3 * a + 3] @ c[j]) + turn(q[t, a, 3:], t) @ turn(down[j, 5:], j)) * 0.5
                      for j in range(T)])
        pr = np.exp(s) / (np.exp(s).sum() + np.exp(w["sink"][a]))
        assert np.allclose(got[t, 4 * a:4 * a + 4], sum(pr[j] * (w["uv"][4 * a:4 * a + 4] @ c[j]) for j in range(T)))


def test_plain_experts_are_chosen_by_logit_with_the_bias_and_weighted_over_the_chosen():
    mlp = su.moe(ff=4, experts=4, top=2)
    rs = np.random.default_rng(5)
    E = 6
    w = {"router": rs.normal(size=(4, E)) * 0.01, "router.b": np.array([0.0, 3.0, -2.0, 2.0])}
    for e in range(4):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = rs.normal(size=(4, E)), rs.normal(size=(4, E)), rs.normal(size=(E, 4))
    f = rs.normal(size=(3, E))
    got = ps.routed_ff(f, w, "", mlp)
    z = f @ w["router"].T + w["router.b"]
    for t in range(3):  # the bias decides: experts 1 and 3
        g1 = 1.0 / (1.0 + math.exp(z[t, 3] - z[t, 1]))
        want = g1 * ps.gated_unit(f[t:t + 1], w, "e1.", ps.silu)[0] + (1 - g1) * ps.gated_unit(f[t:t + 1], w, "e3.", ps.silu)[0]
        assert np.allclose(got[t], want)
    assert ps.chosen_experts(np.array([1.0, 2.0, 2.0, 0.0]), 2)[0] == [1, 2]  # a tie goes to the lower number
    assert ps.chosen_experts(np.array([1.0, 2.0, 2.0, 0.0]), 1)[0] == [1]


def test_plain_gelu_unit():
    E = 3
    w = {"gate": np.eye(E), "up": 2 * np.eye(E), "down": np.eye(E)}
    f = np.array([[3.0, -3.0, 0.5]])
    g = 0.5 * f[0] * (1 + np.tanh(math.sqrt(2 / math.pi) * (f[0] + 0.044715 * f[0] ** 3)))
    assert np.allclose(ps.gated_unit(f, w, "", ps.gelu_tanh)[0], g * 2 * f[0])
    assert abs(ps.gelu_tanh(np.array([3.0]))[0] - 2.9964) < 1e-3 and abs(ps.gelu_tanh(np.array([-3.0]))[0] + 0.0036) < 1e-3
