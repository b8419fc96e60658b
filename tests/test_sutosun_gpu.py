"""Sutosun on the GPU against the plain implementation (`plain_sutosun.py`): every mechanism alone, whole and cut,
then whole models through the replayer in the four work splits, pages and slots used again, long decoding, and greedy
generation through the entry point and its scheduler."""
import numpy as np
import pytest
import torch

import plain_sutosun as ps
import replay_util as ru
import sutosun_util as su
from test_bananex_gpu import CUTS, _load, _run_cut

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt32():
    from cuca_b200.runtime import Runtime
    return Runtime("cuda:0", torch.float32)


def _f32(a, dev):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=dev)


def _mixer(layer, rt, E, eps):
    import cuca_b200.models.model  # noqa: F401  (registers the parts)
    from cuca_b200.config.sutosun_config import SutosunConfig
    from cuca_b200.models.sutosun import _mixer_spec
    from cuca_b200.parts.base import MIXERS
    cfg = SutosunConfig.from_json(su.config([layer], [None], width=E, eps=eps))
    spec = _mixer_spec(cfg.layers[0], E, eps, "l0.mix.")
    return MIXERS.get(spec.kind)(spec, rt)


def _weights_for(part, seed, rounded=False):
    rs = np.random.default_rng(seed)
    ws = {name: np.asarray(su.draw(name, need, rs), dtype=np.float32).astype(np.float64)
          for name, need in part.tensors().items()}
    return {k: su.bf16_round(v) for k, v in ws.items()} if rounded else ws


def _load_as(part, ws, rt):
    needs = part.tensors()
    part.load(lambda n: torch.tensor(ws[n], dtype=torch.float32 if needs[n].keep_fp32 else rt.dtype, device=rt.device))


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("E, dt", [(40, torch.bfloat16), (37, torch.bfloat16), (44, torch.float32), (2048, torch.bfloat16)])
def test_embedding_rows_are_normed(rt32, E, dt):
    from cuca_b200.kernels import ops
    dev, eps = rt32.device, 1e-5
    rs = np.random.default_rng(E)
    table = torch.tensor(rs.normal(0, 3, (11, E)), dtype=torch.float32, device=dev).to(dt)
    w = 1 + rs.normal(0, 0.3, E)
    toks = torch.tensor([3, 0, 10, 3], dtype=torch.int32, device=dev)
    out = torch.empty(4, E, device=dev)
    ops.embed_norm(table, toks, out, _f32(w, dev), eps, rt32.err)
    want = ps.rms(table.double().cpu().numpy()[[3, 0, 10, 3]], eps) * w
    assert np.abs(out.cpu().numpy() - want).max() < 1e-5 * np.abs(want).max()
    assert int(rt32.err.item()) == 0


def test_logits_are_capped(rt32):
    from cuca_b200.kernels import ops
    x = torch.tensor([[-200.0, -7.0, 0.0, 0.3], [5.0, 40.0, 1e4, -1e-3]], device=rt32.device)
    want = 7.5 * np.tanh(x.double().cpu().numpy() / 7.5)
    ops.softcap_(x, 7.5)
    assert np.abs(x.cpu().numpy() - want).max() < 1e-5 and float(x.abs().max()) <= 7.5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 9, 65, 300])
def test_gelu_unit_alone(dtype, T):
    from cuca_b200.parts.base import PartSpec
    from cuca_b200.parts.mlp import GatedUnit
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", dtype)
    dev, E, F = rt.device, 72, 200
    part = GatedUnit(PartSpec("glu", {"width": E, "inner": F, "act": "gelu_tanh"},
                              {"gate": "gate", "up": "up", "down": "down"}), rt)
    rs = np.random.default_rng(T)
    ws = {k: su.bf16_round(v) for k, v in (("gate", rs.normal(0, 1, (F, E)) / np.sqrt(E)),
                                           ("up", rs.normal(0, 1, (F, E)) / np.sqrt(E)),
                                           ("down", rs.normal(0, 1, (E, F)) / np.sqrt(F)))}
    part.load(lambda name: torch.tensor(ws[name], dtype=dtype, device=dev))
    f = su.bf16_round(rs.normal(0, 2.0, (T, E)))  # gate values on both sides of the activation's bend
    want = ps.gated_unit(f, ws, "", ps.gelu_tanh)
    stream = rt.stream(torch.zeros(T, E, device=dev))
    part.forward(torch.tensor(f, dtype=dtype, device=dev), stream, None)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(stream.data.cpu().numpy() - want).max() < tol * max(1.0, np.abs(want).max())
    assert int(rt.err.item()) == 0


RETENTIONS = [su.ret(), su.ret(heads=1, dim=40, vdim=8, decay=[1.0], dims=0), su.ret(heads=2, dim=128, vdim=96, dims=64),
              su.ret(heads=5, dim=4, vdim=36, dims=4, base=30.0), su.ret(heads=1, dim=7, vdim=150, dims=6, decay=[0.25]),
              su.ret(heads=2, dim=200, vdim=5, dims=2, decay=[0.999, 0.5])]


@pytest.mark.parametrize("layer", RETENTIONS)
def test_retention_alone_whole_and_cut(rt32, layer):
    """Three requests in slots 1, 3, 0, whole, one token at a time and in cuts down to two tokens; the state carries
    across every cut and the rotation follows the position, not the place in the step."""
    from cuca_b200.cache.device import CacheView
    dev, E, eps = rt32.device, 44, 1e-5
    part = _mixer(layer, rt32, E, eps)
    ws = _weights_for(part, 5)
    _load(part, ws, dev)
    part.prepare(64)
    rs = np.random.default_rng(6)
    xs = [rs.normal(0, 1.5, (n, E)) for n in (41, 3, 17)]
    want = [ps.retention(x, ws, "l0.mix.", layer["mixer"], eps) for x in xs]
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
    assert int(rt32.err.item()) == 0


def test_retention_remembers_a_far_token_in_the_slow_head_only(rt32):
    """Two heads, decays 1 and 1/2. Only the first token writes (its key channel reads an input column that is set on
    it alone); four hundred tokens later the head that never decays still returns its value, and the fast head has
    lost it: a lost or mixed-up state, or a decay given to the wrong head, shows."""
    from cuca_b200.cache.device import CacheView
    dev, E, eps, n = rt32.device, 24, 1e-5, 400
    layer = su.ret(heads=2, dim=8, vdim=6, decay=[1.0, 0.5], dims=0)
    part = _mixer(layer, rt32, E, eps)
    ws = _weights_for(part, 15)
    ws["l0.mix.k"][:] = 0.0
    ws["l0.mix.k"][0, 0] = ws["l0.mix.k"][8, 0] = 10.0  # channel 0 of both heads: written where column 0 is set
    ws["l0.mix.q"][0] = ws["l0.mix.q"][8] = 0.0
    ws["l0.mix.q"][0, 1] = ws["l0.mix.q"][8, 1] = 5.0  # ... and read where column 1 is set
    _load(part, ws, dev)
    part.prepare(512)
    rs = np.random.default_rng(16)
    x = rs.normal(0, 1.0, (n, E))
    x[:, 0:2] = 0.0
    x[0, 0] = 1.0
    x[n - 5:, 1] = 1.0
    want = ps.retention(x, ws, "l0.mix.", layer["mixer"], eps)
    x2 = x.copy()
    x2[0, 2:] = rs.normal(0, 1.0, E - 2)
    other = ps.retention(x2, ws, "l0.mix.", layer["mixer"], eps)
    assert np.abs(want[-1] - other[-1]).max() > 0.3 * np.abs(want[-1]).max()  # the first token decides the last rows
    for cuts in ([1000], [n - 6] + [1] * 10, [3, 2, 200, 2, 1000]):
        state = {"memory": torch.zeros(4, 2, 6, 8, device=dev)}

        def fwd(h, step):
            out = torch.zeros(h.shape[0], E, device=dev)
            part.forward(h, out, step, CacheView(None, None, None, 16, -1, state, step.slots))
            return out
        got = _run_cut(dev, fwd, [x], [cuts], [2], E)[0]
        assert np.abs(got - want).max() < 1e-4 * np.abs(want).max(), cuts
        mem = state["memory"][2].cpu().numpy()
        assert np.abs(mem[0]).max() > 1.0 and np.abs(mem[1]).max() < 1e-30  # 2^-399 of what the first token wrote


ATTENTIONS = [su.attn(), su.attn(heads=3, kv_heads=3, vdim=16, coef=None),
              su.attn(heads=1, kv_heads=1, dim=32, vdim=16, scale=0.4, coef=1.5, every=1),
              su.attn(heads=6, kv_heads=2, dim=12, vdim=10, scale=1.2, coef=0.2, every=3),
              su.attn(heads=2, kv_heads=1, dim=8, vdim=300, every=40), su.attn(heads=2, kv_heads=2, dim=136, vdim=40, every=64)]


@pytest.mark.parametrize("layer", ATTENTIONS)
def test_gated_attention_alone_whole_and_cut(rt32, layer):
    """Pages of 8 positions handed out in a scrambled order; biases, the norm over the whole projection, the query
    temperature stepping up inside portions and between single tokens, stored sink scores and a gate per head; whole,
    one by one and in cuts."""
    from cuca_b200.cache.device import CacheView
    dev, E, eps, bs = rt32.device, 36, 1e-5, 8
    part = _mixer(layer, rt32, E, eps)
    assert part.general and part.sink and part.sink_learned and part.norm_whole and part.head_gate
    m = layer["mixer"]
    ws = _weights_for(part, 7)
    _load(part, ws, dev)
    part.prepare(128)
    rs = np.random.default_rng(8)
    xs = [rs.normal(0, 1.5, (n, E)) for n in (75, 20)]
    want = [ps.gated_attention(x, ws, "l0.mix.", m, eps) for x in xs]
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


def _planted(dtype, dim, vdim, n, far, askers, sign=1.0, target=16.0, sink=None, every=50):
    """An attention layer with a planted key: the last dimension of every q head reads input column 0 and of the k
    head input column 1 (no bias there, norm weights 1); only position `far` has column 1 set, the rows `askers` have
    column 0 set (with `sign`). `scale` is chosen so that the planted score is about sign * target at temperature 1,
    far above (or below) the others."""
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", dtype)
    E, eps, H = 40, 1e-5, 2
    # after the norms over the whole projections the planted entries hold about 8 / sqrt(1 + 64 / size) each
    qn = 8.0 / np.sqrt(1.0 + 63.0 / (H * dim))
    kn = 8.0 / np.sqrt(1.0 + 63.0 / dim)
    layer = su.attn(heads=H, kv_heads=1, dim=dim, vdim=vdim, scale=target / (qn * kn), coef=0.4, every=every)
    part = _mixer(layer, rt, E, eps)
    ws = _weights_for(part, 13, rounded=True)
    for head in range(H):
        at = head * dim + dim - 1
        ws["l0.mix.q"][at] = 0.0
        ws["l0.mix.q"][at, 0] = 8.0 * sign
        ws["l0.mix.q.b"][at] = 0.0
        ws["l0.mix.q.norm"][at] = 1.0
    ws["l0.mix.k"][dim - 1] = 0.0
    ws["l0.mix.k"][dim - 1, 1] = 8.0
    ws["l0.mix.k.b"][dim - 1] = 0.0
    ws["l0.mix.k.norm"][dim - 1] = 1.0
    if sink is not None:
        ws["l0.mix.sink"][:] = sink
    _load_as(part, ws, rt)
    part.prepare(max(128, n + 8))
    rs = np.random.default_rng(14)
    x = rs.normal(0, 1.0, (n, E))
    x[:, 0:2] = 0.0
    x[far, 1] = 1.0
    x[askers, 0] = 1.0
    return rt, part, layer["mixer"], ws, su.bf16_round(x), E, eps


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, vdim", [(16, 24), (64, 64), (32, 96), (128, 128), (96, 96), (128, 40)])
def test_one_far_key_that_matters(dtype, dim, vdim):
    """Position 3 among five hundred keys, over many pages in a scrambled order: the last rows put nearly all their
    weight on it. Whole, decoded one by one and in portions; through the plain kernel and the tensor-core ones."""
    from cuca_b200.cache.device import CacheView
    n, far, bs = 500, 3, 8
    rt, part, m, ws, x, E, eps = _planted(dtype, dim, vdim, n, far, slice(n - 12, n))
    dev = rt.device
    want = ps.gated_attention(x, ws, "l0.mix.", m, eps)
    x2 = x.copy()
    x2[far, 2:] += 1.0
    other = ps.gated_attention(x2, ws, "l0.mix.", m, eps)
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
    assert int(rt.err.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, vdim", [(16, 24), (64, 64), (128, 128)])
def test_the_query_temperature_shows_on_a_planted_key(dtype, dim, vdim):
    """A planted score of about 6 against a sink of 6: the planted key and the sink share the weight evenly while the
    temperature is 1, and from position `every` - 1 on the key wins by the temperature's factor in the exponent; a
    temperature that starts a token early or late, or is left out, moves those rows."""
    from cuca_b200.cache.device import CacheView
    n, bs, every = 120, 8, 50
    rt, part, m, ws, x, E, eps = _planted(dtype, dim, vdim, n, 2, slice(40, n), target=6.0, sink=6.0, every=every)
    dev = rt.device
    want = ps.gated_attention(x, ws, "l0.mix.", m, eps)
    for wrong in ({"coef": 0.4, "every": every + 1}, {"coef": 0.4, "every": every - 1}, None):
        off = ps.gated_attention(x, ws, "l0.mix.", dict(m, q_temp=wrong) if wrong else {k: v for k, v in m.items() if k != "q_temp"}, eps)
        assert np.abs(off - want).max() > 0.05 * np.abs(want).max()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for cuts in ([1000], [47, 1, 1, 1, 1, 1, 45, 1, 1, 1, 1, 1, 1000], [48, 2, 49, 2, 1000]):
        kpool = torch.zeros((16, 1, bs, dim), dtype=dtype, device=dev)
        vpool = torch.zeros((16, 1, bs, part.v_pool_dim), dtype=dtype, device=dev)
        tables = torch.full((4, 16), -1, dtype=torch.int32, device=dev)
        tables[0, :15] = torch.tensor([4, 1, 7, 0, 2, 5, 9, 15, 3, 8, 10, 14, 6, 11, 12], dtype=torch.int32)

        def fwd(h, step):
            stream = rt.stream(torch.zeros(h.shape[0], E, device=dev))
            part.forward(h.to(dtype), stream, step, CacheView(kpool, vpool, tables, bs, 0, None, step.slots))
            return stream.data
        got = _run_cut(dev, fwd, [x], [cuts], [0], E)[0]
        assert np.abs(got - want).max() < tol * np.abs(want).max(), cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, vdim", [(16, 24), (64, 64), (128, 128)])
def test_the_sink_takes_the_weight_when_it_is_large(dtype, dim, vdim):
    """Stored sink scores of 14 for head 0 and -14 for head 1 against keys that all score near 0: head 0 returns next
    to nothing, head 1 the mean of its values; swapped, dropped or scaled sink scores show."""
    from cuca_b200.cache.device import CacheView
    n, bs = 40, 8
    rt, part, m, ws, x, E, eps = _planted(dtype, dim, vdim, n, 0, slice(0, 0), target=1e-3)
    dev = rt.device
    ws["l0.mix.sink"][:] = [14.0, -14.0]
    ws["l0.mix.g"][:] = 0.0  # both gates one half
    _load_as(part, ws, rt)
    want = ps.gated_attention(x, ws, "l0.mix.", m, eps)
    w_o = ws["l0.mix.o"]
    head0 = want - ps.gated_attention(x, dict(ws, **{"l0.mix.o": np.concatenate([np.zeros_like(w_o[:, :vdim]), w_o[:, vdim:]], 1)}),
                                      "l0.mix.", m, eps)
    assert np.abs(head0).max() < 1e-3 * np.abs(want).max()
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
        assert np.abs(got - want).max() < (2e-5 if dtype == torch.float32 else 3e-2) * np.abs(want).max()


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("splits, cluster", [(1, True), (2, True), (3, True), (4, False), (8, True), (16, False)])
def test_stored_sink_scores_in_every_merge_of_the_split_key_decode(monkeypatch, dim, splits, cluster):
    """Single tokens over 1,100 keys with the keys dealt to 1 to 16 chunks, merged inside one block, through a
    cluster's shared memory or by the last block to arrive: the sink's term goes in once wherever the row's sum is
    closed. A sink of the planted score's size takes half the weight, so a sink counted per chunk, or not at all, shows."""
    from cuca_b200.cache.device import CacheView
    from cuca_b200.kernels import ops
    monkeypatch.setenv("CUCA_DECODE_SPLITS", str(splits))
    monkeypatch.setattr(ops, "CLUSTER_MERGE", cluster)
    n, far, bs, dtype = 1100, 700, 16, torch.bfloat16
    rt, part, m, ws, x, E, eps = _planted(dtype, dim, dim, n, far, slice(n - 6, n), target=9.0, sink=9.0, every=5000)
    dev = rt.device
    want = ps.gated_attention(x, ws, "l0.mix.", m, eps)
    lost = ps.gated_attention(x, dict(ws, **{"l0.mix.sink": ws["l0.mix.sink"] - 30.0}), "l0.mix.", m, eps)
    assert np.abs(want[-1] - lost[-1]).max() > 0.2 * np.abs(want[-1]).max()
    rs = np.random.default_rng(splits)
    kpool = torch.zeros((80, 1, bs, dim), dtype=dtype, device=dev)
    vpool = torch.zeros((80, 1, bs, dim), dtype=dtype, device=dev)
    tables = torch.full((4, 72), -1, dtype=torch.int32, device=dev)
    tables[1, :70] = torch.tensor(rs.permutation(80)[:70].tolist(), dtype=torch.int32)

    def fwd(h, step):
        stream = rt.stream(torch.zeros(h.shape[0], E, device=dev))
        part.forward(h.to(dtype), stream, step, CacheView(kpool, vpool, tables, bs, 0, None, step.slots))
        return stream.data
    got = _run_cut(dev, fwd, [x], [[n - 8] + [1] * 8], [1], E)[0]
    assert np.abs(got - want)[n - 8:].max() < 3e-2 * np.abs(want).max()
    assert int(rt.err.item()) == 0


LATENTS = [su.lat(), su.lat(heads=5, dim=4, rot_dim=0, vdim=36, kv_rank=8), su.lat(heads=1, dim=24, rot_dim=16, vdim=8, kv_rank=16, scale=0.3, rotated=False),
           su.lat(heads=4, dim=32, rot_dim=16, vdim=48, kv_rank=64, base=250000.0,
                  scaling={"factor": 16.0, "original": 32, "fast": 8.0, "slow": 1.0}),
           su.lat(heads=18, dim=8, rot_dim=4, vdim=8, kv_rank=32, scaling=None), su.lat(heads=2, dim=40, rot_dim=24, vdim=20, kv_rank=96)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layer", LATENTS)
def test_latent_attention_alone_whole_and_cut(dtype, layer):
    """Pages of 8 positions in a scrambled order; rotation in pairs (i, i + n/2) with scaled frequencies, the stored
    sink scores, no output gate; whole, one by one and in cuts; the plain kernel and the tensor-core one."""
    from cuca_b200.cache.device import CacheView
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", dtype)
    dev, E, eps, bs = rt.device, 36, 1e-5, 8
    part = _mixer(layer, rt, E, eps)
    assert part.sink and not part.gated
    m = layer["mixer"]
    ws = _weights_for(part, 9, rounded=True)
    _load_as(part, ws, rt)
    part.prepare(128)
    rs = np.random.default_rng(10)
    xs = [su.bf16_round(rs.normal(0, 1.5, (n, E))) for n in (75, 20)]
    want = [ps.latent_attention(x, ws, "l0.mix.", m, eps) for x in xs]
    if m.get("rot"):  # the pairing matters: adjacent pairs give another answer
        assert part.half_pairs
    order = rs.permutation(16).tolist()
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    for cuts in ([CUTS[0]] * 2, [CUTS[1], CUTS[2]], [CUTS[2], CUTS[1]]):
        pool = torch.full((16, 1, bs, m["kv_rank"] + m["rot_dim"]), float("nan"), dtype=dtype, device=dev)
        tables = torch.full((4, 16), -1, dtype=torch.int32, device=dev)
        tables[2, :10] = torch.tensor(order[:10], dtype=torch.int32)
        tables[0, :3] = torch.tensor(order[10:13], dtype=torch.int32)

        def fwd(h, step):
            stream = rt.stream(torch.zeros(h.shape[0], E, device=dev))
            part.forward(h.to(dtype), stream, step, CacheView(pool, None, tables, bs, 0, None, step.slots))
            return stream.data
        got = _run_cut(dev, fwd, xs, cuts, [2, 0], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < tol * max(1.0, np.abs(b).max())
    assert int(rt.err.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank, rot_dim", [(40, 8), (64, 16), (96, 32)])
def test_latent_attention_finds_a_far_key_by_its_turned_part(dtype, rank, rot_dim):
    """The shared key part of position 5 is large along one pair, the last rows ask along the same pair: after the
    rotation by both positions the score depends on their distance, as the plain implementation has it; the rows put
    most of their weight on that one key among three hundred."""
    from cuca_b200.cache.device import CacheView
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", dtype)
    dev, E, eps, bs, n, far = rt.device, 40, 1e-5, 8, 300, 5
    layer = su.lat(heads=2, dim=16, rot_dim=rot_dim, vdim=24, kv_rank=rank, scale=0.5, base=10000.0, scaling=su.YARN)
    part = _mixer(layer, rt, E, eps)
    m = layer["mixer"]
    ws = _weights_for(part, 21, rounded=True)
    pair = rot_dim // 2 - 1  # the slowest pair: it hardly turns over three hundred positions
    for row in (rank + pair, rank + pair + rot_dim // 2):
        ws["l0.mix.dkv"][row] = 0.0
    ws["l0.mix.dkv"][rank + pair, 1] = 6.0
    for head in range(2):
        at = head * (16 + rot_dim) + 16
        ws["l0.mix.q"][at + pair] = 0.0
        ws["l0.mix.q"][at + pair + rot_dim // 2] = 0.0
        ws["l0.mix.q"][at + pair, 0] = 6.0
    ws["l0.mix.sink"][:] = 0.0
    _load_as(part, ws, rt)
    part.prepare(n + 8)
    rs = np.random.default_rng(22)
    x = rs.normal(0, 1.0, (n, E))
    x[:, 0:2] = 0.0
    x[far, 1] = 1.0
    x[n - 10:, 0] = 1.0
    x = su.bf16_round(x)
    want = ps.latent_attention(x, ws, "l0.mix.", m, eps)
    x2 = x.copy()
    x2[far, 2:] += 1.0
    assert np.abs(want[-1] - ps.latent_attention(x2, ws, "l0.mix.", m, eps)[-1]).max() > 0.2 * np.abs(want[-1]).max()
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    for cuts in ([1000], [n - 12] + [1] * 20, [5, 2, 200, 2, 1000]):
        pool = torch.zeros((40, 1, bs, rank + rot_dim), dtype=dtype, device=dev)
        tables = torch.full((4, 40), -1, dtype=torch.int32, device=dev)
        tables[1, :39] = torch.tensor(rs.permutation(40)[:39].tolist(), dtype=torch.int32)

        def fwd(h, step):
            stream = rt.stream(torch.zeros(h.shape[0], E, device=dev))
            part.forward(h.to(dtype), stream, step, CacheView(pool, None, tables, bs, 0, None, step.slots))
            return stream.data
        got = _run_cut(dev, fwd, [x], [cuts], [1], E)[0]
        assert np.abs(got - want).max() < tol * np.abs(want).max(), cuts


def _routed(mlp, E, rt):
    from cuca_b200.config.sutosun_config import MlpConfig
    from cuca_b200.models.sutosun import _mlp_spec
    from cuca_b200.parts.mlp import RoutedExperts
    return RoutedExperts(_mlp_spec(MlpConfig.from_json(mlp, "mlp"), E, "l0.mlp."), rt)


MOES = [(su.moe(), 48), (su.moe(ff=8, experts=1, top=1), 40), (su.moe(ff=16, experts=4, top=4), 36),
        (su.moe(ff=40, experts=37, top=3), 64), (su.moe(ff=9, experts=100, top=32), 50)]


@pytest.mark.parametrize("mlp, E", MOES)
def test_routed_gated_experts_alone(rt32, mlp, E):
    """Few tokens read only the chosen experts, many tokens run all experts with the unchosen ones weighted 0; both
    against the plain implementation, added to a stream and stored into an unwritten one. The router's biases are as
    large as its logits, so they decide many choices and enter the weights."""
    from cuca_b200.runtime import ResidualStream
    dev = rt32.device
    part = _routed(mlp, E, rt32)
    rs = np.random.default_rng(E)
    ws = {name: np.asarray(su.draw(name, need, rs)) for name, need in part.tensors().items()}
    _load(part, ws, dev)
    for T in (1, 5, part.SPARSE_MAX_TOKENS, part.SPARSE_MAX_TOKENS + 1, 150):
        f = rs.normal(0, 1.5, (T, E))
        want = ps.routed_ff(f, ws, "l0.mlp.", mlp)
        if T == 150 and mlp["router"]["experts"] > 1:
            flat = dict(ws)
            flat["l0.mlp.router.b"] = np.zeros_like(ws["l0.mlp.router.b"])
            assert not np.allclose(want, ps.routed_ff(f, flat, "l0.mlp.", mlp))
        base = rs.normal(0, 1, (T, E))
        x = _f32(base, dev)
        part.forward(_f32(f, dev), x, None)
        assert np.abs(x.cpu().numpy() - (base + want)).max() < 3e-5 * max(1.0, np.abs(want).max())
        y = ResidualStream.unwritten(rt32, T, E)
        part.forward(_f32(f, dev), y, None)
        assert np.abs(y.data.cpu().numpy() - want).max() < 3e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("mlp, E", [(su.moe(), 48), (su.moe(ff=64, experts=33, top=5), 64)])
def test_routed_gated_experts_in_bfloat16(mlp, E):
    """Both forms in the serving precision, on the tokens whose choice is clear (the last chosen logit well above the
    first unchosen one): there rounding cannot change the choice."""
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", torch.bfloat16)
    dev = rt.device
    part = _routed(mlp, E, rt)
    rs = np.random.default_rng(E)
    ws = {name: su.bf16_round(np.asarray(su.draw(name, need, rs))) for name, need in part.tensors().items()}
    _load_as(part, ws, rt)
    top = mlp["router"]["top"]
    for T in (7, part.SPARSE_MAX_TOKENS, 200):
        f = su.bf16_round(rs.normal(0, 1.5, (T, E)))
        want = ps.routed_ff(f, ws, "l0.mlp.", mlp)
        z = np.sort(f @ ws["l0.mlp.router"].T + ws["l0.mlp.router.b"], axis=1)[:, ::-1]
        clear = z[:, top - 1] - z[:, top] > 0.05
        assert clear.sum() >= T // 4
        stream = rt.stream(torch.zeros(T, E, device=dev))  # few rows may leave slices pending on it
        part.forward(torch.tensor(f, dtype=torch.bfloat16, device=dev), stream, None)
        got = stream.data.cpu().numpy()
        assert np.abs(got - want)[clear].max() < 3e-2 * np.abs(want).max()


# ------------------------------------------------------------------------------------------ whole models
LENGTHS = {"mix": [1, 2, 5, 16, 33, 64, 97, 130], "plain": [3, 17, 48, 100], "one": [1, 18, 35, 77],
           "wide": [1, 15, 33, 34, 65, 140], "two": [2, 40, 90]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(su.CONFIGS.items()):
        weights = su.make_weights(cfg, seed=20 + i)
        out[name] = (su.write_model(tmp_path_factory.mktemp(f"sutosun_{name}"), cfg, weights), cfg,
                     su.Oracle(cfg, weights))
    return out


def _requests(name, cfg):
    return {f"r{n}": su.random_tokens(n, cfg["vocab"], seed=300 + n) for n in LENGTHS[name]}


def test_the_stream_after_every_layer(models):
    from cuca_b200.engine.core import EngineCore
    from cuca_b200.engine.step import StepEntry
    for name in ("mix", "plain", "one", "wide"):
        folder, cfg, oracle = models[name]
        core = EngineCore.from_folder(folder, dtype="float32", kv_tokens=128, context_length=128, window_pools="full")
        seen = []
        core.model.layer_hook = lambda n, stream: seen.append(stream.data.cpu().numpy().copy())
        toks = su.random_tokens(29, cfg["vocab"], 4)
        blocks, slot = core.pools.new_seq(), core.slots.alloc()
        core.cache.clear_slot(slot)
        core.pools.reserve(blocks, len(toks))
        core.stepper.step([StepEntry(blocks, slot, toks, [0])])
        want = []
        ps.forward(cfg, oracle.w, toks, want)
        assert len(seen) == len(want) == len(cfg["layers"])
        for a, b in zip(seen, want):
            assert np.abs(a - b).max() < 1e-4 * np.abs(b).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(su.CONFIGS))
def test_whole_and_decoded_one_by_one(models, name, dtype):
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    for steps in (ru.trace_whole(reqs), ru.trace_tail_one_by_one(reqs, tail=48)):
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8)
        su.compare(steps, got, reqs, oracle, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(su.CONFIGS))
def test_portions_down_to_two_tokens(models, name, dtype):
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    for sizes in ((5, 2, 17, 3, 2, 32, 7, 2, 64, 11), (2, 2, 3, 1, 1, 8, 9, 40)):
        steps = ru.trace_portions(reqs, sizes=sizes)
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
        su.compare(steps, got, reqs, oracle, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(su.CONFIGS))
def test_mixed_batches_reuse_pages_and_slots(models, name, dtype):
    """Eight and more requests through four (and three) slots and a pool sized for the peak: every slot and most
    pages serve several requests, whose state must start from zero."""
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    reqs.update({f"s{n}": su.random_tokens(n, cfg["vocab"], seed=900 + n) for n in (4, 9, 23, 31, 58)})
    for live, pools in ((4, "full"), (3, "sized")):
        steps = ru.trace_mixed(reqs, max_live=live, seed=7 + live)
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8, window_pools=pools)
        su.compare(steps, got, reqs, oracle, dtype)


def test_32_bit_hardly_depends_on_cuts_or_company(models):
    """In 32-bit a position's logits whole, in portions, decoded and beside other requests differ by rounding alone
    (the routed layers sum a token's experts in another order over few tokens than over many, the scan's column sums
    are shuffled over as many threads as the launch's size suggests)."""
    folder, cfg, _ = models["mix"]
    reqs = {"a": su.random_tokens(70, cfg["vocab"], 1), "b": su.random_tokens(33, cfg["vocab"], 2)}
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
    """Two hundred tokens decoded one by one: the query temperature steps up twice on the way, the retention state and
    the pages grow token by token."""
    folder, cfg, oracle = models["wide"]
    reqs = {"long": su.random_tokens(230, cfg["vocab"], 5)}
    steps = ru.trace_tail_one_by_one(reqs, tail=200)
    for dtype in ("float32", "bfloat16"):
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8, window_pools="sized")
        su.compare(steps, got, reqs, oracle, dtype)


def test_long_prompts(models):
    folder, cfg, oracle = models["mix"]
    reqs = {"p": su.random_tokens(610, cfg["vocab"], 8), "q": su.random_tokens(300, cfg["vocab"], 9)}
    for steps in (ru.trace_whole(reqs), ru.trace_portions(reqs, sizes=(7, 300, 2, 280, 1, 64))):
        for dtype in ("bfloat16", "float32"):
            got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
            su.compare(steps, got, reqs, oracle, dtype)


def test_trace_run_as_a_program(models):
    folder, cfg, oracle = models["one"]
    reqs = _requests("one", cfg)
    steps = ru.trace_mixed(reqs, max_live=4, seed=1)
    got = ru.run_subprocess(folder, "float32", steps, ru.peak_tokens(steps))
    su.compare(steps, got, reqs, oracle, "float32")


# ------------------------------------------------------------------------------------------ the entry point
def _plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(ps.forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["mix", "plain"])
def test_greedy_generation_through_the_entry_point(models, name):
    """`LocalModel.generate`: the scheduler admits, cuts prompts into portions, decodes through captured graphs and
    gives slots to later requests; the tokens are the plain implementation's greedy ones."""
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    folder, cfg, oracle = models[name]
    prompts = [su.random_tokens(n, cfg["vocab"], seed=40 + n) for n in (3, 50, 21, 9, 70)]
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
    prompt = su.random_tokens(20, cfg["vocab"], 77)
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
    prompts = [su.random_tokens(n, cfg["vocab"], seed=60 + n) for n in (5, 70, 33)]
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=256,
                                             batching=BatchingConfig(max_sequences=4, prefill_chunk=32)))
    assert model.backend.use_graphs
    outs = model.generate(prompts, max_tokens=40, temperature=0.0)
    assert model.backend.graph_steps > 0
    for prompt, out in zip(prompts, outs):
        ref = ps.forward(cfg, oracle.w, prompt + out.tokens)
        for i, tok in enumerate(out.tokens):
            row = ref[len(prompt) - 1 + i]
            assert float(row.max() - row[tok]) < 0.05 * float(np.abs(row).max()), (i, tok, int(row.argmax()))
