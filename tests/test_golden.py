"""The committed golden fixture (tests/golden/small_graph.npz, made by tests/golden/make_golden.py)
against the oracle (CPU) and against the CUDA library through the C ABI (GPU)."""
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(HERE, "golden", "small_graph.npz"))


def _live(paths, lens):
    return np.arange(paths.shape[1])[None, :] <= lens[:, None]


def test_oracle_reproduces_golden(oracle, gold):
    x, a, w = gold["xadj"], gold["adjncy"], gold["adjwgt"]
    prob, alias, valid = oracle.alias_build(x, w)
    assert np.array_equal(prob.view(np.uint32), gold["prob"].view(np.uint32))
    assert np.array_equal(alias, gold["alias"]) and np.array_equal(valid, gold["valid"])
    assert oracle.alias_reconstruct_maxrel(x, w, prob, alias, valid) < 1e-6
    table = (prob, alias, valid)
    for name, kw in (("deepwalk", dict(app=oracle.DEEPWALK)), ("ppr", dict(app=oracle.PPR, tp=0.15)),
                     ("node2vec", dict(app=oracle.NODE2VEC, p=2.0, q=0.5))):
        p, l = oracle.walk(x, a, w, table, gold["starts"], 21, seed=42, walker_base=5, **kw)
        assert np.array_equal(l, gold["walk_%s_lengths" % name])
        assert np.array_equal(p, gold["walk_%s_paths" % name])
        p, l = oracle.walk(x, a, None, None, gold["starts"], 21, seed=42, walker_base=5, unbiased=True, **kw)
        assert np.array_equal(l, gold["walk_unbiased_%s_lengths" % name])
        assert np.array_equal(p, gold["walk_unbiased_%s_paths" % name])
    d, s = oracle.khop(x, a, None, None, gold["starts"], [5, 3], flags=2, seed=42, instance_base=9)
    assert np.array_equal(d, gold["khop_unbiased_data"]) and np.array_equal(s, gold["khop_unbiased_lengths"])
    for flags in (0, 1):
        d, s = oracle.khop(x, a, w, table, gold["starts"], [5, 3], flags=flags, seed=42, instance_base=9)
        assert np.array_equal(d, gold["khop_flags%d_data" % flags])
        assert np.array_equal(s, gold["khop_flags%d_lengths" % flags])


def test_golden_corner_vertices(gold):
    # the hub, the zero-weight vertex and the isolated vertex behave as specified
    V = len(gold["xadj"]) - 1
    assert list(gold["valid"][-3:]) == [1, 0, 0]
    for name in ("deepwalk", "ppr", "node2vec"):
        assert list(gold["walk_%s_lengths" % name][-2:]) == [0, 0]      # walkers started on V-2, V-1
    assert gold["walk_deepwalk_lengths"][-3] == 20                          # from the hub: full length
    assert (gold["khop_flags0_lengths"][-2:] == 0).all()


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["offline", "online"])
def test_library_reproduces_golden(ctx, gold, mode):
    from skywalker_b200 import (APP_DEEPWALK, APP_NODE2VEC, APP_PPR, MODE_OFFLINE, MODE_ONLINE)
    m = MODE_OFFLINE if mode == "offline" else MODE_ONLINE
    ctx.upload(gold["xadj"], gold["adjncy"], gold["adjwgt"])
    if mode == "offline":
        ctx.alias_build_offline()
        prob, alias, valid = ctx.alias_export()
        assert np.array_equal(prob.view(np.uint32), gold["prob"].view(np.uint32))
        assert np.array_equal(alias, gold["alias"]) and np.array_equal(valid, gold["valid"])
    for name, kw in (("deepwalk", dict(app=APP_DEEPWALK)), ("ppr", dict(app=APP_PPR, tp=0.15)),
                     ("node2vec", dict(app=APP_NODE2VEC, p=2.0, q=0.5))):
        gp, gl = gold["walk_%s_paths" % name], gold["walk_%s_lengths" % name]
        p, l, _, e = ctx.walk(gold["starts"], 21, mode=m, seed=42, walker_base=5, **kw)
        assert np.array_equal(l, gl) and e == int(gl.sum())
        assert np.array_equal(p[_live(p, l)], gp[_live(gp, gl)])
        if mode == "offline" and name != "node2vec":
            ctx.walk_records_build()
            p, l, _, _ = ctx.walk(gold["starts"], 21, mode=m, seed=42, walker_base=5, **kw)
            assert np.array_equal(l, gl) and np.array_equal(p[_live(p, l)], gp[_live(gp, gl)])
            ctx.walk_records_free()
        if mode == "online":    # both ways of obtaining the drawn slot: tables per step (4), direct (8)
            for flags in (4, 8):
                p, l, _, _ = ctx.walk(gold["starts"], 21, mode=m, seed=42, walker_base=5, flags=flags, **kw)
                assert np.array_equal(l, gl) and np.array_equal(p[_live(p, l)], gp[_live(gp, gl)])
        gp, gl = gold["walk_unbiased_%s_paths" % name], gold["walk_unbiased_%s_lengths" % name]
        p, l, _, e = ctx.walk(gold["starts"], 21, mode=m, seed=42, walker_base=5, flags=2, **kw)   # WALK_UNBIASED
        assert np.array_equal(l, gl) and e == int(gl.sum())
        assert np.array_equal(p[_live(p, l)], gp[_live(gp, gl)])
    for flags in (0, 1):
        d, s, _, _ = ctx.sample_khop(gold["starts"], [5, 3], mode=m, flags=flags, seed=42, instance_base=9)
        assert np.array_equal(d, gold["khop_flags%d_data" % flags])
        assert np.array_equal(s, gold["khop_flags%d_lengths" % flags])
    d, s, _, _ = ctx.sample_khop(gold["starts"], [5, 3], mode=m, flags=2, seed=42, instance_base=9)    # KHOP_UNBIASED
    assert np.array_equal(d, gold["khop_unbiased_data"]) and np.array_equal(s, gold["khop_unbiased_lengths"])
