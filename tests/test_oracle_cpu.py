"""CPU tests: the oracle against published vectors, closed-form properties and hand cases."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def test_philox_known_answers(oracle):
    # Random123 kat_vectors for philox4x32-10
    kat = json.load(open(os.path.join(HERE, "golden", "philox4x32_10_kat.json")))
    for case in kat["cases"]:
        got = oracle.philox([int(x, 16) for x in case["ctr"]], [int(x, 16) for x in case["key"]])
        assert [int(x, 16) for x in case["out"]] == [int(g) for g in got]


def _encoded_probs(w, prob, alias):
    n = len(w)
    acc = prob.astype(np.float64).copy()
    for i in range(n):
        if alias[i] != i:
            acc[alias[i]] += 1.0 - float(prob[i])
    return acc / n


@pytest.mark.parametrize("name,w", [
    ("reference_smoke_vector", [0.5] * 35 + [2.0] * 5),   # test/tmp.cu:31-42 of the reference
    ("uniform", [3.0] * 17),
    ("one_dominant", [1e-3] * 30 + [1000.0]),
    ("single", [7.0]),
    ("two", [1.0, 3.0]),
    ("with_zero", [0.0, 1.0, 2.0, 0.0, 5.0]),
    ("wide_range", [2.0 ** -i for i in range(20)]),
])
def test_alias_vertex_reconstructs(oracle, name, w):
    w = np.asarray(w, np.float32)
    prob, alias, ok = oracle.alias_vertex(w)
    assert ok
    assert (alias < len(w)).all() and (prob >= 0).all() and (prob <= 1).all()
    want = w.astype(np.float64) / w.astype(np.float64).sum()
    got = _encoded_probs(w, prob, alias)
    nz = want > 0
    assert np.max(np.abs(got[nz] - want[nz]) / want[nz]) < 1e-6
    assert np.all(got[~nz] == 0)


def test_alias_uniform_is_identity(oracle):
    prob, alias, ok = oracle.alias_vertex(np.full(9, 2.5, np.float32))
    assert ok and (prob == 1.0).all() and (alias == np.arange(9)).all()


def test_alias_invalid_vertices(oracle):
    for w in ([0.0, 0.0], [-1.0, float("nan")], [float("inf")]):
        _, _, ok = oracle.alias_vertex(np.asarray(w, np.float32))
        assert not ok


def test_alias_masses_conserve_exactly(oracle):
    rng = np.random.default_rng(0)
    for n in (1, 2, 3, 31, 32, 33, 100, 1025, 5000):
        w = rng.uniform(1, 10, n).astype(np.float32)
        M, B = oracle.alias_vertex_masses(w)
        assert B == 40
        assert int(M.astype(object).sum()) == n << B


def test_alias_hand_example(oracle):
    # weights 1,1,2,4: mean 2 -> masses .5,.5,1,2 buckets.  Sweep: donor = slot 2 (first large,
    # exactly one bucket) tops up slot 0 (deficit .5) and drops to .5 < 1 -> becomes a bucket
    # topped up by slot 3; slot 3 (now 1.5) tops up slot 1 and ends with exactly one bucket.
    prob, alias, ok = oracle.alias_vertex(np.asarray([1, 1, 2, 4], np.float32))
    assert ok
    assert np.allclose(prob, [0.5, 0.5, 0.5, 1.0], atol=1e-7)
    assert list(alias) == [2, 3, 3, 3]


def test_graph_tables_reconstruct(oracle, rmat12):
    g = rmat12
    prob, alias, valid = oracle.alias_build(g.xadj, g.adjwgt)
    assert oracle.alias_reconstruct_maxrel(g.xadj, g.adjwgt, prob, alias, valid) < 1e-6
    deg = np.diff(g.xadj.astype(np.int64))
    assert (valid == (deg > 0)).all()


def test_generators_shape(oracle, rmat16):
    g = rmat16
    assert g.V == 65536 and 0.85 * (16 << 16) < g.E <= 16 << 16
    src = np.repeat(np.arange(g.V, dtype=np.uint32), np.diff(g.xadj.astype(np.int64)))
    assert (src != g.adjncy).all()                       # no self loops
    key = (src.astype(np.uint64) << np.uint64(32)) | g.adjncy.astype(np.uint64)
    assert (np.diff(key.astype(np.int64)) > 0).all()     # sorted, no duplicates
    assert g.adjwgt.min() >= 1.0 and g.adjwgt.max() < 10.0


def test_powerlaw_generator(oracle, plaw):
    g = plaw
    src = np.repeat(np.arange(g.V, dtype=np.uint32), np.diff(g.xadj.astype(np.int64)))
    fwd = set(zip(src[:2000].tolist(), g.adjncy[:2000].tolist()))
    key = (src.astype(np.uint64) << np.uint64(32)) | g.adjncy.astype(np.uint64)
    rev = (g.adjncy.astype(np.uint64) << np.uint64(32)) | src.astype(np.uint64)
    assert np.array_equal(np.sort(rev), key)             # symmetric
    assert np.diff(g.xadj.astype(np.int64)).max() <= 3000 * 2


def test_walk_rules(oracle, rmat12):
    g = rmat12
    table = oracle.alias_build(g.xadj, g.adjwgt)
    starts = oracle.gen_starts(512, g.V, 42)
    paths, lens = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, 21)
    deg = np.diff(g.xadj.astype(np.int64))
    for w in range(len(starts)):
        L = int(lens[w])
        assert paths[w, 0] == starts[w]
        for s in range(L):
            u, v = int(paths[w, s]), int(paths[w, s + 1])
            assert v in g.adjncy[g.xadj[u]:g.xadj[u + 1]]
        if L < 20:
            assert deg[paths[w, L]] == 0                  # only a dead end stops a DeepWalk
    # same walkers, split in two calls with a walker_base: identical rows
    p2, l2 = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts[256:], 21, walker_base=256)
    assert np.array_equal(p2, paths[256:]) and np.array_equal(l2, lens[256:])
    # online rebuild gives the same walk as the stored table
    p3, l3 = oracle.walk(g.xadj, g.adjncy, g.adjwgt, None, starts, 21, online=True)
    assert np.array_equal(p3, paths) and np.array_equal(l3, lens)


def test_ppr_lengths_are_geometric(oracle, plaw):
    g = plaw
    table = oracle.alias_build(g.xadj, g.adjwgt)
    starts = oracle.gen_starts(20000, g.V, 1)
    _, lens = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, 101, app=oracle.PPR, tp=0.15)
    # no dead ends in an undirected graph: mean length = (1-tp)/tp (truncated at 100)
    assert abs(lens.mean() - 0.85 / 0.15) < 0.15


def test_khop_layout_and_rules(oracle, rmat12):
    g = rmat12
    table = oracle.alias_build(g.xadj, g.adjwgt)
    seeds = oracle.gen_starts(64, g.V, 3)
    cells, lens, offs = oracle.khop_layout([25, 10])
    assert (cells, lens, offs) == (276, 26, [0, 1, 26])   # include/sampler_result.cuh:226-260
    data, sl = oracle.khop(g.xadj, g.adjncy, g.adjwgt, table, seeds, [25, 10])
    deg = np.diff(g.xadj.astype(np.int64))
    for s in range(len(seeds)):
        assert data[s, 0] == seeds[s]
        assert sl[s, 0] == (25 if deg[seeds[s]] else 0)
        for i in range(25):
            v = data[s, 1 + i]
            kids = data[s, 26 + i * 10: 26 + (i + 1) * 10]
            if v == 0xFFFFFFFF or deg[v] == 0:
                assert sl[s, 1 + i] == 0 and (kids == 0xFFFFFFFF).all()
            else:
                assert sl[s, 1 + i] == 10
                assert np.isin(kids, g.adjncy[g.xadj[v]:g.xadj[v + 1]]).all()
    d2, s2 = oracle.khop(g.xadj, g.adjncy, g.adjwgt, None, seeds, [25, 10], online=True)
    assert np.array_equal(d2, data) and np.array_equal(s2, sl)


def test_chi_square_transition_frequencies(oracle):
    from scipy import stats
    w = np.asarray([1, 2, 3, 4, 10, 0.5, 7, 7, 1.5, 9], np.float32)
    n = len(w)
    xadj = np.asarray([0, n] + [n] * n, np.uint32)        # vertex 0 -> vertices 1..n (sinks)
    adj = np.arange(1, n + 1, dtype=np.uint32)
    table = oracle.alias_build(xadj, w)
    starts = np.zeros(200000, np.uint32)
    paths, lens = oracle.walk(xadj, adj, w, table, starts, 2)
    counts = np.bincount(paths[:, 1] - 1, minlength=n)
    wf = w.astype(np.float64)
    chi, pval = stats.chisquare(counts, f_exp=wf / wf.sum() * counts.sum())
    assert pval > 0.01


def test_unbiased_walks_and_samples_ignore_weights(oracle, rmat12):
    g = rmat12
    starts = oracle.gen_starts(4000, g.V, 3)
    paths, lens = oracle.walk(g.xadj, g.adjncy, None, None, starts, 21, seed=8, unbiased=True)
    # every step follows an edge; lengths end only at dead ends
    for w in range(0, 4000, 97):
        for s in range(lens[w]):
            u, v = paths[w, s], paths[w, s + 1]
            assert v in g.adjncy[g.xadj[u]:g.xadj[u + 1]]
        if lens[w] < 20:
            u = paths[w, lens[w]]
            assert g.xadj[u + 1] == g.xadj[u]
    # first-step frequencies from one vertex are uniform over its columns (chi-square, 64 columns)
    deg = np.diff(g.xadj.astype(np.int64))
    v = int(np.argmax(deg >= 64))
    n = 200 * int(deg[v])
    p1, l1 = oracle.walk(g.xadj, g.adjncy, None, None, np.full(n, v, np.uint32), 2, seed=1, unbiased=True)
    nbrs = g.adjncy[g.xadj[v]:g.xadj[v + 1]]
    uniq, mult = np.unique(nbrs, return_counts=True)
    got = np.array([(p1[:, 1] == u).sum() for u in uniq], np.float64)
    exp = mult.astype(np.float64) / mult.sum() * n
    chi2 = ((got - exp) ** 2 / exp).sum()
    assert chi2 < len(uniq) + 6 * np.sqrt(2 * len(uniq))
    # k-hop: uniform draws need no table; TAKE_ALL still copies whole neighbour lists
    seeds = oracle.gen_starts(256, g.V, 5)
    data, sl = oracle.khop(g.xadj, g.adjncy, None, None, seeds, [6, 3], flags=1 | 2, seed=4)
    for s in range(0, 256, 17):
        d = int(deg[seeds[s]])
        assert sl[s, 0] == (min(d, 6) if d else 0)


def test_alias_denormal_and_huge_weights_reconstruct(oracle):
    for w in ([1e-40, 2e-40, 3e-41, 0, 1e-45], [1e-38, 1e-40, 1.0, 3e-39] * 20, [3.0e38, 1.0, 2.9e38, 1e-30] * 10):
        w = np.asarray(w, np.float32)
        xadj = np.asarray([0, len(w)], np.uint32)
        prob, alias, valid = oracle.alias_build(xadj, w)
        assert valid[0] == 1
        got = _encoded_probs(w, prob, alias)
        want = w.astype(np.float64) / w.astype(np.float64).sum()
        # quantisation keeps 2^-39 of the largest weight: weights far below that may round to zero mass
        assert np.allclose(got, want, rtol=1e-6, atol=2.0 ** -38)


def test_khop_distinct_rule(oracle):
    """flags = 4: children of a parent are distinct columns, in trial order; degree <= fan-out copies
    the whole neighbour list; with a fan-out the degree covers, every neighbour appears exactly once."""
    x, a = oracle.gen_rmat(10, 12 << 10, seed=4)
    w = oracle.gen_weights(len(a), 2)
    table = oracle.alias_build(x, w)
    seeds = oracle.gen_starts(400, len(x) - 1, 6)
    data, sl = oracle.khop(x, a, w, table, seeds, [8, 3], flags=4, seed=1)
    data_on, sl_on = oracle.khop(x, a, w, None, seeds, [8, 3], online=True, flags=4, seed=1)
    assert np.array_equal(data, data_on) and np.array_equal(sl, sl_on)
    deg = np.diff(x.astype(np.int64))
    for s in range(len(seeds)):
        d, got = int(deg[seeds[s]]), int(sl[s, 0])
        kids = data[s, 1:9]
        assert (kids[got:] == 0xFFFFFFFF).all()
        if d <= 8:
            assert got == d and np.array_equal(kids[:got], a[x[seeds[s]]:x[seeds[s] + 1]])
        else:
            assert got <= 8 and len(set(kids[:got].tolist())) == got
    # with replacement (flags = 0) repeats do occur somewhere
    rdata, _ = oracle.khop(x, a, w, table, seeds, [8, 3], flags=0, seed=1)
    assert any(len(set(r[1:9].tolist())) < 8 for r in rdata if r[1] != 0xFFFFFFFF)
