"""Seeded random Pudinex configurations (any layer order, sizes off the beaten track, every feature on or off) through
the replayer: whole, with the last tokens one by one, in portions and in mixed batches through four slots, against the
plain implementation in both dtypes."""
import numpy as np
import pytest

import pudinex_util as pu
import replay_util as ru

pytestmark = pytest.mark.gpu


def random_config(seed: int) -> dict:
    rs = np.random.default_rng(1000 + seed)
    pick = lambda xs: xs[int(rs.integers(len(xs)))]  # noqa: E731
    groups = pick([1, 2, 3, 4, 8])
    width = groups * pick([8, 12, 16, 20, 32, 40, 64])
    n_layers = int(rs.integers(2, 7))
    layers, mlps = [], []
    for _ in range(n_layers):
        if rs.random() < 0.5:
            layers.append(pu.hg(heads=pick([1, 2, 3, 4, 6, 8]), dim=pick([4, 8, 16, 24, 32, 64, 96, 128]),
                                vdim=pick([8, 16, 20, 32, 48, 64, 128, 160])))
        else:
            heads = pick([1, 2, 4, 6, 8, 12])
            kv = pick([k for k in (1, 2, 3, 4, 6, 8, 12) if heads % k == 0])
            dim = pick([16, 24, 32, 48, 64, 80, 96, 128])
            vdim = pick([dim // 2, dim, 2 * dim, dim + 8, 3 * dim // 4, 16, 48, 64, 128])
            dims = pick([0, 2, dim // 4 * 2, dim // 2, dim])
            factor = pick([2.0, 4.0, 8.0, 32.0])
            scaling = pick([None, {"factor": factor, "original": pick([16, 64, 512, 4096]),
                                   "fast": pick([4.0, 32.0]), "slow": pick([0.5, 1.0, 2.0])}])
            layers.append(pu.attn(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, dims=dims,
                                  base=pick([10000.0, 500.0, 1e6]), scaling=scaling,
                                  scale=pick([None, 0.3, 2.0 * dim ** -0.5, 1.0 / dim]),
                                  softcap=pick([None, 2.0, 8.0, 30.0, 50.0])))
        kind = rs.random()
        if kind < 0.15:
            mlps.append(None)
        elif kind < 0.45:
            mlps.append(pu.dense(int(rs.integers(2, 40)) * 8, limit=pick([0.3, 1.0, 2.5, 7.0])))
        else:
            experts = pick([1, 2, 3, 4, 8, 16, 33])
            identity = pick([0, 0, 1, 2, 4, 7])
            mlps.append(pu.moe(ff=pick([8, 16, 24, 40, 64, 96]), experts=experts, identity=identity,
                               top=int(rs.integers(1, min(experts + identity, 6) + 1)),
                               shared=pick([0, 8, 24, 64, 96])))
    return pu.config(layers, mlps, width=width, vocab=int(rs.integers(50, 700)), groups=groups,
                     eps=pick([1e-5, 1e-6]), emb_scale=pick([None, 0.5, 1.0, 3.0, 8.0]))


@pytest.mark.parametrize("seed", list(range(12)))
def test_random_configuration(tmp_path, seed):
    cfg = random_config(seed)
    weights = pu.make_weights(cfg, seed=100 + seed)
    folder = pu.write_model(tmp_path / "m", cfg, weights)
    oracle = pu.Oracle(cfg, weights)
    reqs = {f"r{n}": pu.random_tokens(n, cfg["vocab"], seed=7 * seed + n) for n in (1, 2, 19, 41, 70, 150)}
    for dtype in ("float32", "bfloat16"):
        for steps in (ru.trace_whole(reqs), ru.trace_tail_one_by_one(reqs, tail=40),
                      ru.trace_portions(reqs, sizes=(7, 2, 33, 2, 3, 64, 5)),
                      ru.trace_mixed(reqs, max_live=4, seed=seed)):
            got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
            pu.compare(steps, got, reqs, oracle, dtype, tol32=3e-4)
