"""Properties that hold at any size, checked at benchmark configuration 2's size (R-MAT scale 22, ~65 M edges)
where a bit-for-bit CPU walk of every configuration would be slow: reconstruction of the edge
probabilities, every step is an edge, determinism, invisibility of sharding, agreement of the two
table layouts, PPR length statistics, k-hop children are neighbours of their parent."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from skywalker_b200 import APP_DEEPWALK, APP_PPR, MODE_OFFLINE, MODE_ONLINE


@pytest.fixture(scope="module")
def big(ctx):
    ctx.generate_rmat(22, 16 << 22, graph_seed=1, weight_seed=7)
    ctx.alias_build_offline()
    xadj, adjncy, w = ctx.download()
    return xadj, adjncy, w


def _is_edge(xadj, adjncy, u, v):
    """vectorised membership of (u -> v) in a CSR with sorted adjacency lists"""
    key = (u.astype(np.uint64) << np.uint64(32)) | v.astype(np.uint64)
    src = np.repeat(np.arange(len(xadj) - 1, dtype=np.uint64), np.diff(xadj.astype(np.int64)))
    allk = (src << np.uint64(32)) | adjncy.astype(np.uint64)
    pos = np.searchsorted(allk, key)
    pos = np.minimum(pos, len(allk) - 1)
    return allk[pos] == key


def test_fullsize_table_reconstructs_and_matches_oracle(ctx, oracle, big):
    xadj, adjncy, w = big
    assert len(xadj) - 1 == 1 << 22 and 60e6 < len(adjncy) < 68e6
    prob, alias, valid = ctx.alias_export()
    assert oracle.alias_reconstruct_maxrel(xadj, w, prob, alias, valid) < 1e-6
    # bit-exact against the sequential sweep on a slice that contains every degree class
    deg = np.diff(xadj.astype(np.int64))
    order = np.argsort(deg)[::-1]
    picks = np.concatenate([order[:40], order[1000:1040], order[20000:20100], order[200000:200200],
                            np.arange(5000)])
    for v in picks:
        n = deg[v]
        if n == 0:
            continue
        s = slice(int(xadj[v]), int(xadj[v + 1]))
        p, a, ok = oracle.alias_vertex(w[s])
        assert ok and np.array_equal(a, alias[s]) and np.array_equal(p.view(np.uint32), prob[s].view(np.uint32)), v


def test_fullsize_walks(ctx, oracle, big):
    xadj, adjncy, w = big
    V = len(xadj) - 1
    starts = oracle.gen_starts(40000, V, 42)                 # config 2: 40,000 walkers x 80
    paths, lens, ms, edges = ctx.walk(starts, 81, app=APP_DEEPWALK, seed=42)
    assert edges == int(lens.sum()) and (paths[:, 0] == starts).all()
    cols = np.arange(81)[None, :]
    has_next = cols < lens[:, None]
    u = paths[:, :-1][has_next[:, :-1]]
    v = paths[:, 1:][has_next[:, :-1]]
    assert _is_edge(xadj, adjncy, u, v).all()                # every step is an edge of the graph
    deg = np.diff(xadj.astype(np.int64))
    short = lens < 80
    assert (deg[paths[np.arange(len(lens)), lens][short]] == 0).all()   # only dead ends stop a DeepWalk
    # determinism and sharding invariance
    p2, l2, _, _ = ctx.walk(starts, 81, app=APP_DEEPWALK, seed=42)
    assert np.array_equal(l2, lens) and np.array_equal(p2[cols <= lens[:, None]], paths[cols <= lens[:, None]])
    pa, la, _, _ = ctx.walk(starts[25000:], 81, app=APP_DEEPWALK, seed=42, walker_base=25000)
    live = cols <= la[:, None]
    assert np.array_equal(la, lens[25000:]) and np.array_equal(pa[live], paths[25000:][live])
    # the oracle walks the first walkers bit for bit (tables from the GPU build)
    table = ctx.alias_export()
    op, ol = oracle.walk(xadj, adjncy, w, table, starts[:4000], 81, seed=42)
    live = cols <= ol[:, None]
    assert np.array_equal(ol, lens[:4000]) and np.array_equal(op[live], paths[:4000][live])
    # fused records: identical rows
    ctx.walk_records_build()
    pr, lr, _, er = ctx.walk(starts, 81, app=APP_DEEPWALK, seed=42)
    live = cols <= lens[:, None]
    assert er == edges and np.array_equal(lr, lens) and np.array_equal(pr[live], paths[live])
    ctx.walk_records_free()


def test_fullsize_ppr_statistics(ctx, oracle, big):
    xadj, adjncy, w = big
    V = len(xadj) - 1
    deg = np.diff(xadj.astype(np.int64))
    starts = oracle.gen_starts(1000000, V, 1)
    paths, lens, _, edges = ctx.walk(starts, 101, app=APP_PPR, tp=0.15, seed=3)
    assert edges == int(lens.sum())
    # a walker standing on a vertex with out-edges stops there with probability tp
    alive0 = deg[starts] > 0
    stopped0 = lens[alive0] == 0
    n = int(alive0.sum())
    assert abs(stopped0.mean() - 0.15) < 5 * np.sqrt(0.15 * 0.85 / n)
    assert (lens[~alive0] == 0).all()


def test_fullsize_packed_result_equals_rows(ctx, oracle, big):
    """4 M PPR walkers (four slices of the packed pipeline): the packed result holds exactly the live
    cells of the row matrix, in walker order, with and without walk records."""
    xadj, adjncy, w = big
    V = len(xadj) - 1
    n = 4 << 20
    starts = oracle.gen_starts(n, V, 9)
    paths, lens, _, edges = ctx.walk(starts, 41, app=APP_PPR, tp=0.15, seed=5, walker_base=3)
    live = np.arange(41)[None, :] <= lens[:, None]
    want = paths[live]
    packed, plens, cells, _, pedges = ctx.walk_packed(starts, 41, app=APP_PPR, tp=0.15, seed=5, walker_base=3)
    assert cells == len(want) == edges + n and pedges == edges
    assert np.array_equal(plens, lens) and np.array_equal(packed[:cells], want)
    ctx.walk_records_build()
    packed2, plens2, cells2, _, _ = ctx.walk_packed(starts, 41, app=APP_PPR, tp=0.15, seed=5, walker_base=3)
    ctx.walk_records_free()
    assert cells2 == cells and np.array_equal(plens2, lens) and np.array_equal(packed2[:cells], want)


def test_fullsize_khop(ctx, oracle, big):
    xadj, adjncy, w = big
    V = len(xadj) - 1
    seeds = oracle.gen_starts(65536, V, 9)
    for mode in (MODE_OFFLINE, MODE_ONLINE):
        data, sl, ms, edges = ctx.sample_khop(seeds, [25, 10], mode=mode, seed=5)
        assert edges == int(sl.sum())
        deg = np.diff(xadj.astype(np.int64))
        assert np.array_equal(sl[:, 0], np.where(deg[seeds] > 0, 25, 0))
        hop1 = data[:, 1:26]
        ok1 = hop1 != 0xFFFFFFFF
        assert _is_edge(xadj, adjncy, np.repeat(data[:, 0], 25)[ok1.reshape(-1)], hop1[ok1]).all()
        hop2 = data[:, 26:].reshape(-1, 25, 10)
        ok2 = hop2 != 0xFFFFFFFF
        par = np.broadcast_to(hop1[:, :, None], hop2.shape)
        assert _is_edge(xadj, adjncy, par[ok2], hop2[ok2]).all()
        if mode == MODE_OFFLINE:
            first = (data.copy(), sl.copy())
        else:
            assert np.array_equal(first[0], data) and np.array_equal(first[1], sl)   # online == offline
    ctx.alias_build_offline()   # leave a full table behind for later tests
