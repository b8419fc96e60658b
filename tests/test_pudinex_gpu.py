"""Pudinex on the GPU against the plain implementation (`plain_pudinex.py`): every mechanism alone, whole and cut,
then whole models through the replayer in the four work splits, pages and slots used again, long decoding, and greedy
generation through the entry point and its scheduler."""
import numpy as np
import pytest
import torch

import plain_pudinex as pp
import pudinex_util as pu
import replay_util as ru
from test_bananex_gpu import CUTS, _load, _run_cut, _step

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt32():
    from cuca_b200.runtime import Runtime
    return Runtime("cuda:0", torch.float32)


def _f32(a, dev):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=dev)


def _mixer(layer, rt, E, eps):
    import cuca_b200.models.model  # noqa: F401  (registers the parts)
    from cuca_b200.config.pudinex_config import PudinexConfig
    from cuca_b200.models.pudinex import _mixer_spec
    from cuca_b200.parts.base import MIXERS
    cfg = PudinexConfig.from_json(pu.config([layer], [None], width=E, eps=eps, groups=1))
    spec = _mixer_spec(cfg.layers[0], E, eps, "l0.mix.")
    return MIXERS.get(spec.kind)(spec, rt)


def _weights_for(part, seed):
    rs = np.random.default_rng(seed)
    ws = {}
    for name, need in part.tensors().items():
        shape = tuple(need.shape)
        if name.endswith(".lower"):
            v = rs.uniform(0.0, 0.9, shape)
        elif name.endswith(".f.b"):
            v = rs.normal(1.0, 1.5, shape)
        elif name.endswith(".correction"):
            v = rs.normal(0.0, 0.5 / shape[0], shape)
        elif need.init == "ones":
            v = 1 + rs.normal(0, 0.3, shape)
        else:
            v = rs.normal(0, 1, shape) / np.sqrt(shape[-1])
        ws[name] = np.asarray(v, dtype=np.float32).astype(np.float64)
    return ws


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("E, groups", [(60, 3), (52, 1), (64, 2), (2052, 4), (33, 33), (8192, 2), (35, 5)])
def test_norm_in_parts(rt32, E, groups):
    """Every part has its own root mean square; rows gathered; a stream that a contraction left slices on."""
    from cuca_b200.kernels import ops
    dev, eps, rows = rt32.device, 1e-5, 9
    rs = np.random.default_rng(E)
    x = rs.normal(0, 2, (rows, E)) * np.repeat(rs.uniform(0.01, 30, groups), E // groups)
    w = 1 + rs.normal(0, 0.3, E)
    want = pp.group_norm(x, w, groups, eps)
    out = torch.empty(rows, E, device=dev)
    ops.rmsnorm(_f32(x, dev), _f32(w, dev), out, eps, groups=groups)
    assert np.abs(out.cpu().numpy() - want).max() < 1e-5 * np.abs(want).max()
    gather = torch.tensor([5, 0, 5, 8], dtype=torch.int32, device=dev)
    g = torch.empty(4, E, dtype=torch.bfloat16, device=dev)
    ops.rmsnorm(_f32(x, dev), _f32(w, dev), g, eps, gather, groups=groups)
    assert np.abs(g.float().cpu().numpy() - want[[5, 0, 5, 8]]).max() < 1e-2 * np.abs(want).max()
    # slices left unadded: x = base + sum of the slices, added in the same pass
    slices = rs.normal(0, 1, (3, rows, E))
    base = x - slices.sum(0)
    xd = _f32(base, dev)
    ops.add_partials_rmsnorm(xd, ops.PartialSums(_f32(slices, dev), 3), _f32(w, dev), out, eps, groups=groups)
    assert np.abs(out.cpu().numpy() - want).max() < 2e-5 * np.abs(want).max()
    assert np.abs(xd.cpu().numpy() - x).max() < 1e-5 * np.abs(x).max()


def test_embedding_rows_are_scaled(rt32):
    from cuca_b200.kernels import ops
    dev = rt32.device
    for E, dt in ((40, torch.bfloat16), (37, torch.bfloat16), (44, torch.float32)):
        table = torch.randn(11, E, device=dev).to(dt)
        toks = torch.tensor([3, 0, 10, 3], dtype=torch.int32, device=dev)
        out = torch.empty(4, E, device=dev)
        ops.embed(table, toks, out, rt32.err, 2.5)
        assert torch.equal(out, table.float()[toks.long()] * 2.5)
    assert int(rt32.err.item()) == 0


@pytest.mark.parametrize("limit", [0.3, 1.0, 7.0])
def test_capped_unit_alone(rt32, limit):
    from cuca_b200.parts.base import PartSpec
    from cuca_b200.parts.mlp import CappedGLU
    dev, E, F = rt32.device, 44, 70
    part = CappedGLU(PartSpec("glu_capped", {"width": E, "inner": F, "limit": limit},
                              {"gate": "gate", "up": "up", "down": "down"}), rt32)
    rs = np.random.default_rng(1)
    ws = {"gate": rs.normal(0, 1, (F, E)) / np.sqrt(E), "up": rs.normal(0, 1, (F, E)) / np.sqrt(E),
          "down": rs.normal(0, 1, (E, F)) / np.sqrt(F)}
    _load(part, ws, dev)
    f = rs.normal(0, 2.0, (13, E))  # gate and up values well beyond the smaller caps, on both sides
    assert (np.abs(f @ ws["up"].T) > limit).any() or limit > 5
    want = pp.capped_glu(f, ws, "", limit)
    x = torch.zeros(13, E, device=dev)
    part.forward(_f32(f, dev), x, None)
    assert np.abs(x.cpu().numpy() - want).max() < 2e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("limit", [0.4, 6.0])
@pytest.mark.parametrize("T", [1, 9, 64, 65, 200, 700])
def test_capped_unit_as_the_contraction_epilogue(limit, T):
    """In the serving precision the unit is computed inside the gate/up contraction, from its 32-bit sums, whichever
    tiling the number of tokens selects; sizes that are no multiple of a tile."""
    from cuca_b200.parts.base import PartSpec
    from cuca_b200.parts.mlp import CappedGLU
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", torch.bfloat16)
    dev, E, F = rt.device, 72, 200
    part = CappedGLU(PartSpec("glu_capped", {"width": E, "inner": F, "limit": limit},
                              {"gate": "gate", "up": "up", "down": "down"}), rt)
    rs = np.random.default_rng(T)
    ws = {k: pu.bf16_round(v) for k, v in (("gate", rs.normal(0, 1, (F, E)) / np.sqrt(E)),
                                           ("up", rs.normal(0, 1, (F, E)) / np.sqrt(E)),
                                           ("down", rs.normal(0, 1, (E, F)) / np.sqrt(F)))}
    part.load(lambda name: torch.tensor(ws[name], dtype=torch.bfloat16, device=dev))
    f = pu.bf16_round(rs.normal(0, 2.0, (T, E)))
    want = pp.capped_glu(f, ws, "", limit)
    stream = rt.stream(torch.zeros(T, E, device=dev))
    part.forward(torch.tensor(f, dtype=torch.bfloat16, device=dev), stream, None)
    assert np.abs(stream.data.cpu().numpy() - want).max() < 2e-2 * max(1.0, np.abs(want).max())
    assert int(rt.err.item()) == 0


@pytest.mark.parametrize("layer", [pu.hg(), pu.hg(heads=1, dim=40, vdim=8), pu.hg(heads=2, dim=128, vdim=96),
                                   pu.hg(heads=5, dim=4, vdim=36), pu.hg(heads=1, dim=7, vdim=150),
                                   pu.hg(heads=2, dim=200, vdim=5)])
def test_forget_gate_attention_alone_whole_and_cut(rt32, layer):
    """Three requests in slots 1, 3, 0, whole, one token at a time and in cuts down to two tokens; the state carries
    across every cut; slots start from what an earlier run left and are cleared."""
    from cuca_b200.cache.device import CacheView
    dev, E, eps = rt32.device, 44, 1e-5
    part = _mixer(layer, rt32, E, eps)
    ws = _weights_for(part, 5)
    _load(part, ws, dev)
    rs = np.random.default_rng(6)
    xs = [rs.normal(0, 1.5, (n, E)) for n in (41, 3, 17)]
    want = [pp.hgrn2(x, ws, "l0.mix.", layer["mixer"], eps) for x in xs]
    state = {k: torch.full((4, *v.shape), 7.0, device=dev) for k, v in part.cache_needs().state.items()}
    for cuts in ([CUTS[0]] * 3, [CUTS[1], CUTS[2], CUTS[1]], [CUTS[2], CUTS[1], CUTS[2]]):
        for t in state.values():
            t.zero_()  # what the engine does when a slot gets a new request

        def fwd(h, step):
            out = torch.zeros(h.shape[0], E, device=dev)
            part.forward(h, out, step, CacheView(None, None, None, 16, -1, state, step.slots))
            return out
        got = _run_cut(dev, fwd, xs, cuts, [1, 3, 0], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < 3e-5 * max(1.0, np.abs(b).max())


def test_forget_gate_attention_remembers_a_far_token(rt32):
    """A channel whose gate stays at 1 (a lower bound of 1) keeps what the first token wrote... and writes nothing:
    so a channel with lower bound near 1 and a large bias. One channel is opened for the first token only (its gate
    reads input column 0, set on that token alone); four hundred tokens later the read-out still holds its value."""
    from cuca_b200.cache.device import CacheView
    dev, E, eps, n = rt32.device, 24, 1e-5, 400
    layer = pu.hg(heads=1, dim=8, vdim=6)
    part = _mixer(layer, rt32, E, eps)
    ws = _weights_for(part, 15)
    ws["l0.mix.f"][0] = 0.0
    ws["l0.mix.f"][0, 0] = -40.0  # channel 0: f = 0 where column 0 is 1 (the token is written whole) ...
    ws["l0.mix.f.b"][0] = 20.0    # ... and f = 1 elsewhere (kept for ever)
    ws["l0.mix.lower"][0] = 0.0
    ws["l0.mix.q"][0] = 0.0
    ws["l0.mix.q"][0, 1] = 30.0   # q channel 0 is large where column 1 is set
    _load(part, ws, dev)
    rs = np.random.default_rng(16)
    x = rs.normal(0, 1.0, (n, E))
    x[:, 0:2] = 0.0
    x[0, 0] = 1.0
    x[n - 5:, 1] = 1.0
    want = pp.hgrn2(x, ws, "l0.mix.", layer["mixer"], eps)
    x2 = x.copy()
    x2[0, 2:] = rs.normal(0, 1.0, E - 2)
    other = pp.hgrn2(x2, ws, "l0.mix.", layer["mixer"], eps)
    assert np.abs(want[-1] - other[-1]).max() > 0.3 * np.abs(want[-1]).max()  # the first token decides the last rows
    for cuts in ([1000], [n - 6] + [1] * 10, [3, 2, 200, 2, 1000]):
        state = {"memory": torch.zeros(4, 1, 6, 8, device=dev)}

        def fwd(h, step):
            out = torch.zeros(h.shape[0], E, device=dev)
            part.forward(h, out, step, CacheView(None, None, None, 16, -1, state, step.slots))
            return out
        got = _run_cut(dev, fwd, [x], [cuts], [2], E)[0]
        assert np.abs(got - want).max() < 1e-4 * np.abs(want).max(), cuts


ATTENTIONS = [pu.attn(), pu.attn(heads=3, kv_heads=3, dims=0, vdim=16, softcap=None),
              pu.attn(heads=1, kv_heads=1, dim=32, vdim=16, dims=32, softcap=50.0, scale=0.4),
              pu.attn(heads=6, kv_heads=2, dim=12, vdim=10, dims=6, scale=1.2, base=250000.0, scaling=None, softcap=1.5),
              pu.attn(heads=2, kv_heads=1, dim=8, vdim=300, dims=2),
              pu.attn(heads=2, kv_heads=2, dim=136, vdim=40, dims=64, scaling={"factor": 32.0, "original": 16,
                                                                                "fast": 2.0, "slow": 0.5})]


@pytest.mark.parametrize("layer", ATTENTIONS)
def test_sink_attention_alone_whole_and_cut(rt32, layer):
    """Pages of 8 positions handed out in a scrambled order; head norms, rotation of a part of a head with scaled
    frequencies, the cap and the sink; whole, one by one and in cuts."""
    from cuca_b200.cache.device import CacheView
    dev, E, eps, bs = rt32.device, 36, 1e-5, 8
    part = _mixer(layer, rt32, E, eps)
    assert part.general and part.sink and part.qk_norm and part.v_norm
    m = layer["mixer"]
    ws = _weights_for(part, 7)
    _load(part, ws, dev)
    part.prepare(128)
    rs = np.random.default_rng(8)
    xs = [rs.normal(0, 1.5, (n, E)) for n in (75, 20)]
    want = [pp.sink_attention(x, ws, "l0.mix.", m, eps) for x in xs]
    order = rs.permutation(16).tolist()
    for cuts in ([CUTS[0]] * 2, [CUTS[1], CUTS[2]], [CUTS[2], CUTS[1]]):
        kpool = torch.full((16, m["kv_heads"], bs, m["dim"]), float("nan"), device=dev)
        vpool = torch.full((16, m["kv_heads"], bs, m["vdim"]), float("nan"), device=dev)
        tables = torch.full((4, 16), -1, dtype=torch.int32, device=dev)
        tables[2, :10] = torch.tensor(order[:10], dtype=torch.int32)
        tables[0, :3] = torch.tensor(order[10:13], dtype=torch.int32)

        def fwd(h, step):
            out = torch.zeros(h.shape[0], E, device=dev)
            part.forward(h, out, step, CacheView(kpool, vpool, tables, bs, 0, None, step.slots))
            return out
        got = _run_cut(dev, fwd, xs, cuts, [2, 0], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < 2e-5 * max(1.0, np.abs(b).max())
    assert int(rt32.err.item()) == 0


def _planted(dtype, dim, vdim, softcap, n, far, askers, sign=1.0, scale=0.25):
    """An attention layer with a planted key: one unrotated dimension of q reads input column 0 and of k input column
    1; only position `far` has column 1 set, the rows `askers` have column 0 set (with `sign`). After the head norms
    that dimension holds about sqrt(dim) on both sides (its norm weights are 1), so the planted score is about
    sign * scale * dim and stands far above (or below) the others."""
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", dtype)
    E, eps = 40, 1e-5
    layer = pu.attn(heads=2, kv_heads=1, dim=dim, vdim=vdim, dims=8, scale=scale, softcap=softcap)
    part = _mixer(layer, rt, E, eps)
    ws = {k: pu.bf16_round(v) for k, v in _weights_for(part, 13).items()}
    for head in range(2):
        ws["l0.mix.q"][head * dim + dim - 1] = 0.0
        ws["l0.mix.q"][head * dim + dim - 1, 0] = 8.0 * sign
    ws["l0.mix.k"][dim - 1] = 0.0
    ws["l0.mix.k"][dim - 1, 1] = 8.0
    ws["l0.mix.q.norm"][dim - 1] = ws["l0.mix.k.norm"][dim - 1] = 1.0
    needs = part.tensors()
    part.load(lambda name: torch.tensor(ws[name], dtype=torch.float32 if needs[name].keep_fp32 else dtype, device=rt.device))
    part.prepare(max(128, n + 8))
    rs = np.random.default_rng(14)
    x = rs.normal(0, 1.0, (n, E))
    x[:, 0:2] = 0.0
    x[far, 1] = 1.0
    x[askers, 0] = 1.0
    return rt, part, layer["mixer"], ws, pu.bf16_round(x), E, eps


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, vdim", [(16, 24), (64, 64), (32, 96), (128, 128), (128, 40)])
@pytest.mark.parametrize("softcap", [None, 12.0])
def test_one_far_key_that_matters(dtype, dim, vdim, softcap):
    """Position 3 among five hundred keys, over many pages in a scrambled order: the last rows put nearly all their
    weight on it. Whole, decoded one by one and in portions."""
    from cuca_b200.cache.device import CacheView
    n, far, bs = 500, 3, 8
    rt, part, m, ws, x, E, eps = _planted(dtype, dim, vdim, softcap, n, far, slice(n - 12, n))
    dev = rt.device
    want = pp.sink_attention(x, ws, "l0.mix.", m, eps)
    x2 = x.copy()
    x2[far, 2:] += 1.0
    other = pp.sink_attention(x2, ws, "l0.mix.", m, eps)
    assert np.abs(want[-1] - other[-1]).max() > 0.2 * np.abs(want[-1]).max()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    rs = np.random.default_rng(3)
    for cuts in ([1000], [n - 14] + [1] * 20, [5, 2, 300, 2, 1000]):
        kpool = torch.zeros((70, 1, bs, dim), dtype=dtype, device=dev)
        vpool = torch.zeros((70, 1, bs, part.v_pool_dim), dtype=dtype, device=dev)  # (padded in bfloat16)
        tables = torch.full((4, 64), -1, dtype=torch.int32, device=dev)
        tables[1, :63] = torch.tensor(rs.permutation(70)[:63].tolist(), dtype=torch.int32)

        def fwd(h, step):
            stream = rt.stream(torch.zeros(h.shape[0], E, device=dev))
            part.forward(h.to(dtype), stream, step, CacheView(kpool, vpool, tables, bs, 0, None, step.slots))
            return stream.data
        got = _run_cut(dev, fwd, [x], [cuts], [1], E)[0]
        assert np.abs(got - want).max() < tol * np.abs(want).max(), cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, vdim", [(16, 24), (64, 64), (128, 128)])
def test_the_sink_takes_the_weight_when_no_key_fits(dtype, dim, vdim):
    """Rows whose every score is far below zero: with all keys at about -16 against the sink's 0 the output nearly
    vanishes, where a softmax without the sink would still return a mean of the values (of norm one per head)."""
    from cuca_b200.cache.device import CacheView
    n, bs = 40, 8
    # every position is a planted key, and the askers ask with the opposite sign: all their scores are about -16
    rt, part, m, ws, x, E, eps = _planted(dtype, dim, vdim, None, n, slice(0, n), slice(20, n), sign=-1.0, scale=16.0 / dim)
    dev = rt.device
    x[:, 2:] *= 0.05  # the other dimensions hardly count, so that every score of an asker is low
    x = pu.bf16_round(x)
    want = pp.sink_attention(x, ws, "l0.mix.", m, eps)
    o = ws["l0.mix.o"]
    no_sink_scale = np.abs(pp.sink_attention(x[:5], ws, "l0.mix.", m, eps)).max()
    assert np.abs(want[25:]).max() < 1e-3 * no_sink_scale and np.abs(o).max() > 0
    for cuts in ([1000], [22] + [1] * 30):
        kpool = torch.zeros((8, 1, bs, dim), dtype=dtype, device=dev)
        vpool = torch.zeros((8, 1, bs, part.v_pool_dim), dtype=dtype, device=dev)
        tables = torch.full((4, 8), -1, dtype=torch.int32, device=dev)
        tables[3, :6] = torch.tensor([4, 1, 7, 0, 2, 5], dtype=torch.int32)

        def fwd(h, step):
            stream = rt.stream(torch.zeros(h.shape[0], E, device=dev))
            part.forward(h.to(dtype), stream, step, CacheView(kpool, vpool, tables, bs, 0, None, step.slots))
            return stream.data
        got = _run_cut(dev, fwd, [x], [cuts], [3], E)[0]
        assert np.abs(got[25:]).max() < 2e-3 * no_sink_scale
        assert np.abs(got - want).max() < (2e-5 if dtype == torch.float32 else 3e-2) * np.abs(want).max()


def _routed(mlp, E, rt):
    from cuca_b200.config.pudinex_config import MlpConfig
    from cuca_b200.models.pudinex import _mlp_spec
    from cuca_b200.parts.mlp import ScoredExperts
    return ScoredExperts(_mlp_spec(MlpConfig.from_json(mlp, "mlp"), E, "l0.mlp."), rt)


MOES = [(pu.moe(), 48), (pu.moe(ff=8, experts=1, identity=0, top=1, shared=24), 40),
        (pu.moe(ff=16, experts=4, identity=0, top=4, shared=0), 36), (pu.moe(ff=40, experts=37, identity=5, top=3, shared=72), 64),
        (pu.moe(ff=9, experts=100, identity=30, top=32, shared=10), 50), (pu.moe(ff=24, experts=2, identity=6, top=4, shared=0), 44),
        (pu.moe(ff=12, experts=0, identity=3, top=2, shared=20), 32)]


@pytest.mark.parametrize("mlp, E", MOES)
def test_scored_experts_alone(rt32, mlp, E):
    """Few tokens read only the chosen experts, many tokens run all experts with the unchosen ones weighted 0; both
    against the plain implementation, added to a stream and stored into an unwritten one. The corrections are as
    large as the scores, so they decide many choices, and must not enter the weights."""
    from cuca_b200.runtime import ResidualStream
    dev = rt32.device
    part = _routed(mlp, E, rt32)
    rs = np.random.default_rng(E)
    ws = {name: rs.normal(0, 1, need.shape) / np.sqrt(need.shape[-1]) for name, need in part.tensors().items()}
    ws["l0.mlp.router"] *= 3.0
    n_out = ws["l0.mlp.router"].shape[0]
    ws["l0.mlp.correction"] = rs.normal(0, 1.0 / n_out, n_out)
    _load(part, ws, dev)
    for T in (1, 5, part.SPARSE_MAX_TOKENS, part.SPARSE_MAX_TOKENS + 1, 150):
        f = rs.normal(0, 1.5, (T, E))
        want = pp.routed_ff(f, ws, "l0.mlp.", mlp)
        plain = dict(ws)
        plain["l0.mlp.correction"] = np.zeros(n_out)
        if T == 150 and mlp["router"]["top"] < n_out and mlp["router"]["experts"]:  # (experts that all return their input
            # give the same sum whichever are chosen)
            assert not np.allclose(want, pp.routed_ff(f, plain, "l0.mlp.", mlp))  # the corrections do decide
        base = rs.normal(0, 1, (T, E))
        x = _f32(base, dev)
        part.forward(_f32(f, dev), x, None)
        assert np.abs(x.cpu().numpy() - (base + want)).max() < 3e-5 * max(1.0, np.abs(want).max())
        y = ResidualStream.unwritten(rt32, T, E)
        part.forward(_f32(f, dev), y, None)
        assert np.abs(y.data.cpu().numpy() - want).max() < 3e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("mlp, E", [(pu.moe(), 48), (pu.moe(ff=64, experts=33, identity=4, top=5, shared=32), 64)])
def test_scored_experts_in_bfloat16(mlp, E):
    """Both forms in the serving precision, on the tokens whose choice is clear (the last chosen choice score well
    above the first unchosen one): there rounding cannot change the choice."""
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", torch.bfloat16)
    dev = rt.device
    part = _routed(mlp, E, rt)
    rs = np.random.default_rng(E)
    ws = {name: pu.bf16_round(rs.normal(0, 1, need.shape) / np.sqrt(need.shape[-1])) for name, need in part.tensors().items()}
    ws["l0.mlp.router"] = pu.bf16_round(ws["l0.mlp.router"] * 4.0)
    n_out = ws["l0.mlp.router"].shape[0]
    ws["l0.mlp.correction"] = pu.bf16_round(rs.normal(0, 0.5 / n_out, n_out))
    needs = part.tensors()
    part.load(lambda n: torch.tensor(ws[n], dtype=torch.float32 if needs[n].keep_fp32 else torch.bfloat16, device=dev))
    top = mlp["router"]["top"]
    for T in (7, part.SPARSE_MAX_TOKENS, 200):
        f = pu.bf16_round(rs.normal(0, 1.5, (T, E)))
        want = pp.routed_ff(f, ws, "l0.mlp.", mlp)
        z = f @ ws["l0.mlp.router"].T
        s = np.exp(z - z.max(1, keepdims=True))
        c = np.sort(s / s.sum(1, keepdims=True) + ws["l0.mlp.correction"], axis=1)[:, ::-1]
        clear = c[:, top - 1] - c[:, top] > 0.05 / n_out  # (the router's inputs are exact in bfloat16 and its sums 32-bit)
        assert clear.sum() >= T // 4
        stream = rt.stream(torch.zeros(T, E, device=dev))  # few rows may leave slices pending on it
        part.forward(torch.tensor(f, dtype=torch.bfloat16, device=dev), stream, None)
        got = stream.data.cpu().numpy()
        assert np.abs(got - want)[clear].max() < 3e-2 * np.abs(want).max()


def test_scoring_of_rows_that_hold_anything(rt32):
    """A captured step's padding rows hold whatever was in memory: the chosen outputs must be outputs all the same,
    and distinct ones, since their numbers index the experts' weights."""
    from cuca_b200.kernels import ops
    dev = rt32.device
    z = torch.randn(6, 8, device=dev)
    z[1] = float("nan")
    z[2, 3:] = float("nan")
    z[3] = float("inf")
    z[4] = float("-inf")
    z[5] = 0.0
    corr = torch.zeros(8, device=dev)
    for top in (1, 2, 8):
        idx = torch.full((6, top), -7, dtype=torch.int32, device=dev)
        wts = torch.empty(6, top, device=dev)
        ident = torch.empty(6, device=dev)
        ops.moe_route_scored(z, corr, 6, top, idx, wts, None, ident)
        got = idx.cpu().numpy()
        assert ((got >= 0) & (got < 8)).all()
        assert all(len(set(row)) == top for row in got.tolist())
        assert got[5].tolist() == list(range(top))  # ties go to the lower number
        assert np.isfinite(wts[0].cpu().numpy()).all() and np.isfinite(wts[5].cpu().numpy()).all()
        assert abs(float(wts[5].sum()) - 1.0) < 1e-5


# ------------------------------------------------------------------------------------------ whole models
LENGTHS = {"mix": [1, 2, 5, 16, 33, 64, 97, 130], "plain": [3, 17, 48, 100], "one": [1, 18, 35, 77],
           "wide": [1, 15, 33, 34, 65, 140], "two": [2, 40, 90]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(pu.CONFIGS.items()):
        weights = pu.make_weights(cfg, seed=20 + i)
        out[name] = (pu.write_model(tmp_path_factory.mktemp(f"pudinex_{name}"), cfg, weights), cfg,
                     pu.Oracle(cfg, weights))
    return out


def _requests(name, cfg):
    return {f"r{n}": pu.random_tokens(n, cfg["vocab"], seed=300 + n) for n in LENGTHS[name]}


def test_the_stream_after_every_layer(models):
    from cuca_b200.engine.core import EngineCore
    from cuca_b200.engine.step import StepEntry
    for name in ("mix", "plain", "one", "wide"):
        folder, cfg, oracle = models[name]
        core = EngineCore.from_folder(folder, dtype="float32", kv_tokens=128, context_length=128, window_pools="full")
        seen = []
        core.model.layer_hook = lambda n, stream: seen.append(stream.data.cpu().numpy().copy())
        toks = pu.random_tokens(29, cfg["vocab"], 4)
        blocks, slot = core.pools.new_seq(), core.slots.alloc()
        core.cache.clear_slot(slot)
        core.pools.reserve(blocks, len(toks))
        core.stepper.step([StepEntry(blocks, slot, toks, [0])])
        want = []
        pp.forward(cfg, oracle.w, toks, want)
        assert len(seen) == len(want) == len(cfg["layers"])
        for a, b in zip(seen, want):
            assert np.abs(a - b).max() < 1e-4 * np.abs(b).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(pu.CONFIGS))
def test_whole_and_decoded_one_by_one(models, name, dtype):
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    for steps in (ru.trace_whole(reqs), ru.trace_tail_one_by_one(reqs, tail=48)):
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8)
        pu.compare(steps, got, reqs, oracle, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(pu.CONFIGS))
def test_portions_down_to_two_tokens(models, name, dtype):
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    for sizes in ((5, 2, 17, 3, 2, 32, 7, 2, 64, 11), (2, 2, 3, 1, 1, 8, 9, 40)):
        steps = ru.trace_portions(reqs, sizes=sizes)
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
        pu.compare(steps, got, reqs, oracle, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(pu.CONFIGS))
def test_mixed_batches_reuse_pages_and_slots(models, name, dtype):
    """Eight and more requests through four (and three) slots and a pool sized for the peak: every slot and most
    pages serve several requests, whose state must start from zero."""
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    reqs.update({f"s{n}": pu.random_tokens(n, cfg["vocab"], seed=900 + n) for n in (4, 9, 23, 31, 58)})
    for live, pools in ((4, "full"), (3, "sized")):
        steps = ru.trace_mixed(reqs, max_live=live, seed=7 + live)
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8, window_pools=pools)
        pu.compare(steps, got, reqs, oracle, dtype)


def test_32_bit_hardly_depends_on_cuts_or_company(models):
    """In 32-bit a position's logits whole, in portions, decoded and beside other requests differ by rounding alone
    (the routed layers sum a token's experts in another order over few tokens than over many, the scan's column sums
    are shuffled over as many threads as the launch's size suggests)."""
    folder, cfg, _ = models["mix"]
    reqs = {"a": pu.random_tokens(70, cfg["vocab"], 1), "b": pu.random_tokens(33, cfg["vocab"], 2)}
    whole = ru.trace_whole(reqs)
    ref = ru.run_in_process(folder, "float32", whole, ru.peak_tokens(whole))
    want = {rid: ref[i] for i, rid in enumerate(reqs)}
    for steps in (ru.trace_portions(reqs, sizes=(3, 2, 9, 1, 1, 30)), ru.trace_mixed(reqs, max_live=2, seed=3)):
        got = ru.run_in_process(folder, "float32", steps, ru.peak_tokens(steps))
        pos = {rid: 0 for rid in reqs}
        for s in steps:
            row = 0
            for e in s["entries"]:
                for w in e["want"]:
                    r = want[e["id"]][pos[e["id"]] + w]
                    assert np.abs(got[s["step"]][row] - r).max() < 2e-5 * np.abs(r).max(), (s["step"], e["id"])
                    row += 1
                pos[e["id"]] += len(e["tokens"])


def test_long_decoding(models):
    folder, cfg, oracle = models["wide"]
    reqs = {"long": pu.random_tokens(230, cfg["vocab"], 5)}
    steps = ru.trace_tail_one_by_one(reqs, tail=200)
    for dtype in ("float32", "bfloat16"):
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8, window_pools="sized")
        pu.compare(steps, got, reqs, oracle, dtype)


def test_long_prompts(models):
    folder, cfg, oracle = models["mix"]
    reqs = {"p": pu.random_tokens(610, cfg["vocab"], 8), "q": pu.random_tokens(300, cfg["vocab"], 9)}
    for steps in (ru.trace_whole(reqs), ru.trace_portions(reqs, sizes=(7, 300, 2, 280, 1, 64))):
        for dtype in ("bfloat16", "float32"):
            got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
            pu.compare(steps, got, reqs, oracle, dtype)


def test_trace_run_as_a_program(models):
    folder, cfg, oracle = models["one"]
    reqs = _requests("one", cfg)
    steps = ru.trace_mixed(reqs, max_live=4, seed=1)
    got = ru.run_subprocess(folder, "float32", steps, ru.peak_tokens(steps))
    pu.compare(steps, got, reqs, oracle, "float32")


# ------------------------------------------------------------------------------------------ the entry point
def _plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(pp.forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["mix", "plain"])
def test_greedy_generation_through_the_entry_point(models, name):
    """`LocalModel.generate`: the scheduler admits, cuts prompts into portions, decodes through captured graphs and
    gives slots to later requests; the tokens are the plain implementation's greedy ones."""
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    folder, cfg, oracle = models[name]
    prompts = [pu.random_tokens(n, cfg["vocab"], seed=40 + n) for n in (3, 50, 21, 9, 70)]
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="float32", context_length=256,
                                             batching=BatchingConfig(max_sequences=2, prefill_chunk=16)))
    outs = model.generate(prompts, max_tokens=12, temperature=0.0)
    for prompt, out in zip(prompts, outs):
        assert out.tokens == _plain_greedy(cfg, oracle.w, prompt, 12)


def test_command_line_sampling_and_the_prefix_cache_refusal(models):
    import subprocess
    import sys
    from pathlib import Path

    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    from cuca_b200.cache.pages import StatefulCacheError
    folder, cfg, oracle = models["two"]
    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([sys.executable, "-m", "cuca_b200", "--model-dir", str(folder), "--prompt", "5 9 20 31",
                        "--max-tokens", "6", "--temperature", "0", "--dtype", "float32"],
                       capture_output=True, text=True, cwd=root, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == _plain_greedy(cfg, oracle.w, [5, 9, 20, 31], 6)
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=128))
    prompt = pu.random_tokens(20, cfg["vocab"], 77)
    a = model.generate(prompt, max_tokens=16, temperature=1.0, top_k=20, seed=5).tokens
    b = model.generate(prompt, max_tokens=16, temperature=1.0, top_k=20, seed=5).tokens
    c = model.generate(prompt, max_tokens=16, temperature=1.0, top_k=20, seed=6).tokens
    assert a == b and a != c and all(0 <= t < cfg["vocab"] for t in a)
    with pytest.raises(StatefulCacheError):
        LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=128,
                                         batching=BatchingConfig(prefix_cache=True)))


def test_bfloat16_generation_through_captured_graphs(models):
    """The serving precision end to end: prompts in portions, decode steps replayed as CUDA graphs. Where two logits
    nearly tie bfloat16 may take the other branch, so every token it takes must be a near-maximum of the plain
    implementation's logits at its place."""
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    folder, cfg, oracle = models["two"]
    prompts = [pu.random_tokens(n, cfg["vocab"], seed=60 + n) for n in (5, 70, 33)]
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=256,
                                             batching=BatchingConfig(max_sequences=4, prefill_chunk=32)))
    assert model.backend.use_graphs
    outs = model.generate(prompts, max_tokens=40, temperature=0.0)
    assert model.backend.graph_steps > 0
    for prompt, out in zip(prompts, outs):
        ref = pp.forward(cfg, oracle.w, prompt + out.tokens)
        for i, tok in enumerate(out.tokens):
            row = ref[len(prompt) - 1 + i]
            assert float(row.max() - row[tok]) < 0.05 * float(np.abs(row).max()), (i, tok, int(row.argmax()))
