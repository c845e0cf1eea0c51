"""The reference's own offline walk kernel (sample_kernel_static, src/offline_walk.cu:75-124 of
wpybtw/Skywalker, driven through its OfflineWalk entry function) and its own offline 2-hop sampler
(sample_kernel, src/offline_sample.cu:72-141, through OfflineSample) and its unbiased walk
(UnbiasedWalkKernelStatic, src/unbiased_walk.cu:104-130, through UnbiasedWalk) beside this library.

The reference has no golden vectors and its random stream (XORWOW seeded by thread id) cannot be
reproduced, so the comparison is statistical: fed with the alias table THIS library builds (exported
as the reference's prob / alias / valid arrays), the reference kernel's transitions must follow the
edge weights (chi-square, p > 0.01), and its walks must have the same length statistics and visit
distribution as this library's walks over the same table.  The harness is built from the reference
tree by oracle/ref_cuda/Makefile; on a machine that has neither the tree nor the built library the
tests are skipped.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import reference_kernel as R
    if not R.available():
        pytest.skip("oracle/_ref/libskw_ref.so was not built (no reference tree on the build machine)")
    return R


def _two_way_star(w):
    """Vertex 0 points at leaves 1..n with weights w; every leaf points back at vertex 0."""
    n = len(w)
    xadj = np.concatenate([[0, n], n + 1 + np.arange(n)]).astype(np.uint32)
    adj = np.concatenate([np.arange(1, n + 1), np.zeros(n)]).astype(np.uint32)
    wgt = np.concatenate([w, np.ones(n)]).astype(np.float32)
    return xadj, adj, wgt


def test_reference_kernel_follows_the_weights_of_our_table(ctx, ref):
    """Chi-square of the reference kernel's transitions out of the hub of a two-way star against the
    edge weights, with the table this library built.  Every walker returns to the hub after each leaf
    (a leaf has one out-edge, which the reference takes without a draw), so a walker of 200 steps makes
    100 draws from the hub's table.  Long walks on purpose: the reference seeds one XORWOW generator per
    thread with the thread id, and the very first outputs of generators seeded 0, 1, 2, ... are
    measurably non-uniform (400,000 single first draws from a 2-slot table failed this test with
    p = 3e-26), a property of that seeding, not of the table."""
    from scipy import stats
    rng = np.random.default_rng(3)
    for n in (2, 7, 33, 300):
        w = rng.uniform(1, 10, n).astype(np.float32)
        xadj, adj, wgt = _two_way_star(w)
        ctx.upload(xadj, adj, wgt)
        ctx.alias_build_offline()
        table = ctx.alias_export()
        N, hop = 4096, 201
        paths, lens, _ = ref.offline_walk(xadj, adj, table, np.zeros(N, np.uint32), hop)
        assert (lens == hop - 1).all()
        assert (paths[:, 0::2] == 0).all()
        leaves = paths[:, 1::2].astype(np.int64).reshape(-1) - 1
        counts = np.bincount(leaves, minlength=n)
        wf = w.astype(np.float64)
        chi, pval = stats.chisquare(counts, f_exp=wf / wf.sum() * len(leaves))
        assert pval > 0.01, (n, pval)
        # the same check on this library's walk kernel over the same table
        ours, olens, _, _ = ctx.walk(np.zeros(N, np.uint32), hop, seed=n)
        oleaves = ours[:, 1::2].astype(np.int64).reshape(-1) - 1
        chi, pval = stats.chisquare(np.bincount(oleaves, minlength=n), f_exp=wf / wf.sum() * len(oleaves))
        assert pval > 0.01, (n, pval)


def test_reference_walks_and_ours_have_the_same_statistics(ctx, oracle, ref, rmat12):
    """Same graph, same table, 200,000 walkers x 20 steps: the two implementations draw from different
    random streams, so rows differ, but the walk-length histogram and the visit counts of the most
    visited vertices must agree (two-sample chi-square, p > 0.01)."""
    from scipy import stats
    g = rmat12
    ctx.upload(g.xadj, g.adjncy, g.adjwgt)
    ctx.alias_build_offline()
    table = ctx.alias_export()
    N, hop = 200000, 21
    starts = oracle.gen_starts(N, g.V, 77)
    ours_p, ours_l, _, _ = ctx.walk(starts, hop, seed=5)
    ref_p, ref_l, sec = ref.offline_walk(g.xadj, g.adjncy, table, starts, hop)
    assert sec > 0
    # every step of the reference walk follows an edge of the graph
    for s in range(3):
        alive = ref_l > s
        src, dst = ref_p[alive, s].astype(np.int64), ref_p[alive, s + 1]
        lo, hi = g.xadj[src], g.xadj[src + 1]
        ok = np.fromiter((d in g.adjncy[a:b] for a, b, d in zip(lo[:2000], hi[:2000], dst[:2000])), bool)
        assert ok.all()
    # walk lengths: a walk ends early only at a vertex without out-edges
    ha = np.bincount(ours_l, minlength=hop)
    hb = np.bincount(ref_l, minlength=hop)
    keep = (ha + hb) >= 20
    _, p_len, _, _ = stats.chi2_contingency(np.vstack([ha[keep], hb[keep]]))
    assert p_len > 0.01, p_len
    # visit counts after 3 steps, 40 most visited vertices (by the pooled count) + the rest
    def visits(paths, lens):
        v = paths[lens >= 3, 3].astype(np.int64)
        return np.bincount(v, minlength=g.V)
    va, vb = visits(ours_p, ours_l), visits(ref_p, ref_l)
    top = np.argsort(-(va + vb))[:40]
    ta = np.append(va[top], va.sum() - va[top].sum())
    tb = np.append(vb[top], vb.sum() - vb[top].sum())
    _, p_vis, _, _ = stats.chi2_contingency(np.vstack([ta, tb]))
    assert p_vis > 0.01, p_vis


def test_reference_sampler_follows_the_weights_of_our_table(ctx, ref):
    """The reference's offline sampler draws f1 = 25 neighbours with replacement from a vertex of more
    than 25 neighbours through the alias table it is handed (src/offline_sample.cu:103-118): from the
    centre of a star, with the table this library built, its hop-1 samples must follow the edge weights
    (chi-square).  One thread block per SM and 400,000 instances of the same seed, so that a thread
    draws for about ten of them: with the reference's default launch (four blocks per SM, one XORWOW
    generator per thread seeded with the thread id) 120,000 instances meant fewer than one per thread, i.e.
    only the first outputs of neighbouring seeds, and failed with p = 2e-17 -- the same property of that
    seeding as in the walk test above."""
    from scipy import stats
    rng = np.random.default_rng(8)
    for n in (33, 300):
        w = rng.uniform(1, 10, n).astype(np.float32)
        xadj = np.asarray([0, n] + [n] * n, np.uint32)         # leaves have no out-edges
        adj = np.arange(1, n + 1, dtype=np.uint32)
        ctx.upload(xadj, adj, w)
        ctx.alias_build_offline()
        table = ctx.alias_export()
        N, f1, f2 = 400000, 25, 2
        data, sl, sec, edges = ref.offline_sample(xadj, adj, table, np.zeros(N, np.uint32), f1, f2, blocks_per_sm=1)
        assert sec > 0 and (data[:, 0] == 0).all()
        assert (sl[:, 0] == f1).all() and (sl[:, 1:] == 0).all() and edges == N * f1
        leaves = data[:, 1:1 + f1].astype(np.int64).reshape(-1) - 1
        assert leaves.min() >= 0 and leaves.max() < n
        wf = w.astype(np.float64)
        chi, pval = stats.chisquare(np.bincount(leaves, minlength=n), f_exp=wf / wf.sum() * len(leaves))
        assert pval > 0.001, (n, pval)


def test_reference_samples_and_ours_have_the_same_statistics(ctx, oracle, ref, rmat12):
    """Same graph, same table, same 100,000 seeds, fan-outs 5 then 3: the reference hands over every
    neighbour of a vertex that has no more than the fan-out and draws with replacement otherwise, which is
    this library's SKW_KHOP_TAKE_ALL rule, so the hop-1 sample counts must be equal cell by cell, every
    sample must be a neighbour of its parent, and the distribution of the sampled vertices must agree
    (two-sample chi-square).  Hop 2 of the reference is incomplete by construction: its kernel fills the
    queue of hop-2 jobs while other thread blocks already drain it, publishes a queue slot before writing
    it (include/frontier.cuh:236-246) and drops what it reads too early; where it did sample, the count
    and the samples must be right."""
    from scipy import stats
    from skywalker_b200 import KHOP_TAKE_ALL
    g = rmat12
    ctx.upload(g.xadj, g.adjncy, g.adjwgt)
    ctx.alias_build_offline()
    table = ctx.alias_export()
    N, f1, f2 = 100000, 5, 3
    seeds = oracle.gen_starts(N, g.V, 55)
    rdata, rsl, sec, redges = ref.offline_sample(g.xadj, g.adjncy, table, seeds, f1, f2)
    odata, osl, _, oedges = ctx.sample_khop(seeds, [f1, f2], flags=KHOP_TAKE_ALL, seed=6)
    assert sec > 0 and (rdata[:, 0] == seeds).all()
    deg = np.diff(g.xadj.astype(np.int64))
    assert np.array_equal(rsl[:, 0], np.minimum(deg[seeds], f1)) and np.array_equal(osl[:, 0], rsl[:, 0])
    # hop 1: every sample is a neighbour of its seed
    for i in range(2000):
        k = rsl[i, 0]
        nb = g.adjncy[g.xadj[seeds[i]]:g.xadj[seeds[i] + 1]]
        assert np.isin(rdata[i, 1:1 + k], nb).all()
    # hop 2: under a hop-1 sample either nothing (a dropped job, or a vertex without neighbours) or
    # min(its degree, f2) samples, each of them its neighbour
    done = expected = 0
    for i in range(2000):
        for j in range(rsl[i, 0]):
            p = int(rdata[i, 1 + j])
            k = int(rsl[i, 1 + j])
            expected += deg[p] > 0
            if k:
                done += 1
                assert k == min(deg[p], f2)
                kids = rdata[i, 1 + f1 + j * f2:1 + f1 + j * f2 + k]
                assert np.isin(kids, g.adjncy[g.xadj[p]:g.xadj[p + 1]]).all()
    assert 0 < done <= expected
    assert redges == int(rsl.sum()) and redges <= oedges
    # sampled vertices of hop 1 where a draw happens (degree above the fan-out): 40 most frequent + the rest
    drawn = deg[seeds] > f1
    ra = np.bincount(rdata[drawn, 1:1 + f1].astype(np.int64).reshape(-1), minlength=g.V)
    oa = np.bincount(odata[drawn, 1:1 + f1].astype(np.int64).reshape(-1), minlength=g.V)
    top = np.argsort(-(ra + oa))[:40]
    ta = np.append(ra[top], ra.sum() - ra[top].sum())
    tb = np.append(oa[top], oa.sum() - oa[top].sum())
    _, p_vis, _, _ = stats.chi2_contingency(np.vstack([ta, tb]))
    assert p_vis > 0.001, p_vis
    print("reference hop 2: %d of %d jobs of the first 2000 seeds sampled; sampled edges %d (ours %d)"
          % (done, expected, redges, oedges))


def test_reference_unbiased_walks_and_ours_have_the_same_statistics(ctx, oracle, ref, rmat12):
    """The reference's unbiased walk with its stop rule (UnbiasedWalkKernelStatic, src/unbiased_walk.cu:104-130)
    beside SKW_WALK_UNBIASED on the same graph and start vertices, tp = 0.15: every step follows an edge, and
    the walk-length histogram and the visit counts after two steps agree (two-sample chi-square)."""
    from scipy import stats
    from skywalker_b200 import APP_PPR, WALK_UNBIASED
    g = rmat12
    ctx.upload(g.xadj, g.adjncy, g.adjwgt)
    N, hop = 300000, 41
    starts = oracle.gen_starts(N, g.V, 91)
    ref_p, ref_l, sec = ref.unbiased_walk(g.xadj, g.adjncy, starts, hop, tp=0.15)
    ours_p, ours_l, _, _ = ctx.walk(starts, hop, app=APP_PPR, tp=0.15, flags=WALK_UNBIASED, seed=4)
    assert sec > 0 and (ref_p[:, 0] == starts).all()
    for s_ in range(2):
        alive = ref_l > s_
        src, dst = ref_p[alive, s_].astype(np.int64)[:2000], ref_p[alive, s_ + 1][:2000]
        assert all(d in g.adjncy[g.xadj[a]:g.xadj[a + 1]] for a, d in zip(src, dst))
    ha, hb = np.bincount(ours_l, minlength=hop), np.bincount(ref_l, minlength=hop)
    keep = (ha + hb) >= 20
    _, p_len, _, _ = stats.chi2_contingency(np.vstack([ha[keep], hb[keep]]))
    assert p_len > 0.001, p_len
    def visits(paths, lens):
        return np.bincount(paths[lens >= 2, 2].astype(np.int64), minlength=g.V)
    va, vb = visits(ours_p, ours_l), visits(ref_p, ref_l)
    top = np.argsort(-(va + vb))[:40]
    ta = np.append(va[top], va.sum() - va[top].sum())
    tb = np.append(vb[top], vb.sum() - vb[top].sum())
    _, p_vis, _, _ = stats.chi2_contingency(np.vstack([ta, tb]))
    assert p_vis > 0.001, p_vis
