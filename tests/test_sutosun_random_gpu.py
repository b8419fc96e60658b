"""Seeded random Sutosun configurations (any layer order, sizes off the beaten track, every feature on or off, entries
that run with another entry's tensors) through the replayer: whole, with the last tokens one by one, in portions and
in mixed batches through four slots, against the plain implementation in both dtypes."""
import numpy as np
import pytest

import replay_util as ru
import sutosun_util as su

pytestmark = pytest.mark.gpu


def random_config(seed: int) -> dict:
    rs = np.random.default_rng(2000 + seed)
    pick = lambda xs: xs[int(rs.integers(len(xs)))]  # noqa: E731
    width = pick([24, 36, 40, 52, 64, 72, 96, 100, 128, 200, 256])
    n_layers = int(rs.integers(2, 8))
    layers, mlps, borrow = [], [], {}
    for i in range(n_layers):
        kind = pick(["attention", "retention", "latent_attention"])
        if kind == "attention":
            heads = pick([1, 2, 4, 6, 8, 12])
            kv = pick([k for k in (1, 2, 3, 4, 6, 8, 12) if heads % k == 0])
            dim = pick([8, 16, 24, 32, 48, 64, 80, 96, 128])
            layers.append(su.attn(heads=heads, kv_heads=kv, dim=dim,
                                  vdim=pick([dim // 2, dim, dim, 2 * dim, dim + 8, 16, 48, 64]),
                                  scale=pick([None, 0.3, 2.0 * dim ** -0.5, 1.0 / dim]),
                                  coef=pick([None, 0.1, 0.5, 2.0]), every=pick([1, 3, 16, 64, 100, 1000])))
        elif kind == "retention":
            heads = pick([1, 2, 3, 4, 6, 8])
            dim = pick([4, 8, 16, 24, 32, 64, 96, 128])
            layers.append(su.ret(heads=heads, dim=dim, vdim=pick([8, 16, 20, 32, 48, 64, 128, 160]),
                                 decay=[float(1.0 - 2.0 ** -rs.integers(1, 12)) for _ in range(heads)],
                                 dims=pick([0, 2, dim // 4 * 2, dim // 2 * 2 // 2 * 2, dim]) // 2 * 2,
                                 base=pick([10000.0, 500.0, 1e6])))
        else:
            rot_dim = pick([0, 2, 8, 16, 32, 64])
            factor = pick([2.0, 4.0, 8.0, 32.0])
            scaling = pick([None, {"factor": factor, "original": pick([16, 64, 512, 4096]),
                                   "fast": pick([4.0, 32.0]), "slow": pick([0.5, 1.0, 2.0])}])
            dim = pick([4, 16, 32, 64, 96])
            layers.append(su.lat(heads=pick([1, 2, 3, 4, 8, 16, 20]), dim=dim, rot_dim=rot_dim,
                                 vdim=pick([8, 24, 32, 64, 80]), kv_rank=pick([8, 24, 32, 64, 96, 128, 160]),
                                 scale=pick([None, 0.3, 1.0 / (dim + rot_dim)]), base=pick([10000.0, 500000.0]),
                                 scaling=scaling, rotated=rs.random() < 0.85))
        kind = rs.random()
        if kind < 0.15:
            mlps.append(None)
        elif kind < 0.45:
            mlps.append(su.dense(int(rs.integers(2, 40)) * pick([8, 8, 4, 6])))
        else:
            experts = pick([1, 2, 3, 4, 8, 16, 33])
            mlps.append(su.moe(ff=pick([8, 12, 16, 20, 24, 40, 64, 96]), experts=experts,
                               top=int(rs.integers(1, min(experts, 6) + 1))))
    for i in range(n_layers):  # some entries run with another entry's tensors, an earlier or a later one
        others = [j for j in range(n_layers) if j != i and j not in borrow and i not in borrow.values()]
        if others and rs.random() < 0.25:
            borrow[i] = pick(others)
    return su.config(layers, mlps, width=width, vocab=int(rs.integers(50, 700)), eps=pick([1e-5, 1e-6]),
                     softcap=pick([None, 5.0, 30.0, 50.0]), weights_of=borrow)


@pytest.mark.parametrize("seed", list(range(12)))
def test_random_configuration(tmp_path, seed):
    cfg = random_config(seed)
    weights = su.make_weights(cfg, seed=100 + seed)
    folder = su.write_model(tmp_path / "m", cfg, weights)
    oracle = su.Oracle(cfg, weights)
    reqs = {f"r{n}": su.random_tokens(n, cfg["vocab"], seed=7 * seed + n) for n in (1, 2, 19, 41, 70, 150)}
    for dtype in ("float32", "bfloat16"):
        for steps in (ru.trace_whole(reqs), ru.trace_tail_one_by_one(reqs, tail=40),
                      ru.trace_portions(reqs, sizes=(7, 2, 33, 2, 3, 64, 5)),
                      ru.trace_mixed(reqs, max_live=4, seed=seed)):
            got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
            su.compare(steps, got, reqs, oracle, dtype, tol32=3e-4)
