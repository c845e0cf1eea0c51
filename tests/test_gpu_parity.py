"""GPU parity tests: every entry point of the C ABI against the CPU oracle, bit for bit.

Run on a B200 with `pytest -m gpu`.  Everything goes through libskywalker_b200.so via ctypes.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from skywalker_b200 import (APP_DEEPWALK, APP_NODE2VEC, APP_PPR, INVALID_VERTEX, KHOP_DISTINCT, KHOP_TAKE_ALL,
                            KHOP_UNBIASED, MODE_OFFLINE, MODE_ONLINE, WALK_UNBIASED)


def _upload(ctx, g):
    ctx.upload(g.xadj, g.adjncy, g.adjwgt)


def _cmp_walks(paths, lens, opaths, olens):
    assert np.array_equal(lens, olens)
    cols = np.arange(paths.shape[1])[None, :]
    live = cols <= lens[:, None]
    assert np.array_equal(paths[live], opaths[live])


def test_graph_roundtrip(ctx, rmat12):
    _upload(ctx, rmat12)
    V, E, md = ctx.graph_info()
    assert (V, E) == (rmat12.V, rmat12.E)
    assert md == int(np.diff(rmat12.xadj.astype(np.int64)).max())
    x, a, w = ctx.download()
    assert np.array_equal(x, rmat12.xadj) and np.array_equal(a, rmat12.adjncy) and np.array_equal(w, rmat12.adjwgt)


def test_rmat_generator_matches_oracle(ctx, oracle):
    for scale, sym in ((12, False), (14, True)):
        ctx.generate_rmat(scale, 16 << scale, symmetric=sym, graph_seed=5, weight_seed=6)
        x, a, w = ctx.download()
        ox, oa = oracle.gen_rmat(scale, 16 << scale, symmetric=sym, seed=5)
        assert np.array_equal(x, ox) and np.array_equal(a, oa)
        assert np.array_equal(w, oracle.gen_weights(len(oa), 6))


def test_rmat_generator_folded_vertex_count(ctx, oracle):
    ctx.generate_rmat(13, 100000, graph_seed=2, weight_seed=3, num_vertices=5000)
    x, a, w = ctx.download()
    ox, oa = oracle.gen_rmat(13, 100000, seed=2, num_vertices=5000)
    assert len(x) == 5001 and np.array_equal(x, ox) and np.array_equal(a, oa)


def test_powerlaw_generator_matches_oracle(ctx, oracle):
    ctx.generate_powerlaw(20000, 300000, 2.1, 4.0, 3000, graph_seed=5, weight_seed=11)
    x, a, w = ctx.download()
    ox, oa = oracle.gen_powerlaw(20000, 300000, 2.1, 4.0, 3000, seed=5)
    assert np.array_equal(x, ox) and np.array_equal(a, oa)
    assert np.array_equal(w, oracle.gen_weights(len(oa), 11))


def test_starts_match_oracle(ctx, oracle, rmat12):
    import torch
    _upload(ctx, rmat12)
    d = torch.zeros(1000, dtype=torch.int32, device="cuda")
    ctx.generate_starts(1000, 42, d, id_base=17)
    ctx.synchronize()
    got = d.cpu().numpy().view(np.uint32)
    assert np.array_equal(got, oracle.gen_starts(1000, rmat12.V, 42, id_base=17))


@pytest.mark.parametrize("gname", ["rmat12", "rmat16", "plaw"])
def test_alias_table_bit_exact(ctx, oracle, request, gname):
    g = request.getfixturevalue(gname)
    _upload(ctx, g)
    ctx.alias_build_offline()
    prob, alias, valid = ctx.alias_export()
    oprob, oalias, ovalid = oracle.alias_build(g.xadj, g.adjwgt)
    assert np.array_equal(valid, ovalid)
    assert np.array_equal(alias, oalias)
    assert np.array_equal(prob.view(np.uint32), oprob.view(np.uint32))
    assert oracle.alias_reconstruct_maxrel(g.xadj, g.adjwgt, prob, alias, valid) < 1e-6


def _star_graph(weights_per_vertex):
    """Vertex i has the given weight list; all edges point to sink vertices."""
    degs = [len(w) for w in weights_per_vertex]
    nsrc = len(degs)
    maxd = max(degs) if degs else 0
    V = nsrc + max(maxd, 1)
    xadj = np.zeros(V + 1, np.uint32)
    xadj[1:nsrc + 1] = np.cumsum(degs)
    xadj[nsrc + 1:] = xadj[nsrc]
    adj = np.concatenate([nsrc + np.arange(d, dtype=np.uint32) for d in degs]) if degs else np.zeros(0, np.uint32)
    w = np.concatenate([np.asarray(x, np.float32) for x in weights_per_vertex])
    return xadj, adj.astype(np.uint32), w


def test_alias_every_degree_class_and_edge_cases(ctx, oracle):
    rng = np.random.default_rng(1)
    lists = []
    for n in list(range(1, 70)) + [127, 128, 129, 200, 511, 512, 513, 1023, 1024, 1025, 4000, 4096, 4097, 8191, 8192, 8193, 16384, 16385, 20000, 70000]:
        lists.append(rng.uniform(1, 10, n).astype(np.float32))
    lists.append(np.asarray([0.5] * 35 + [2.0] * 5, np.float32))       # reference smoke vector
    lists.append(np.full(40, 3.0, np.float32))                         # uniform
    lists.append(np.asarray([1e-3] * 30 + [1000.0], np.float32))       # one dominant
    lists.append(np.zeros(5, np.float32))                              # all zero -> invalid
    lists.append(np.zeros(100, np.float32))                            # all zero, CTA class
    lists.append(np.asarray([0, 1, 2, 0, 5], np.float32))              # zeros inside
    lists.append(np.asarray([np.nan, -1, np.inf, 2, 3], np.float32))   # unusable entries
    lists.append((2.0 ** -np.arange(20)).astype(np.float32))           # wide range
    lists.append(rng.uniform(0, 1, 3000).astype(np.float32) ** 8)      # skewed, many tiny
    lists.append(np.asarray([1e-40, 2e-40, 3e-41, 0, 1e-45], np.float32))           # denormals only
    lists.append(np.full(300, 1e-45, np.float32))                                   # the smallest denormal, warp class
    lists.append(np.asarray([1e-38, 1e-40, 1.0, 3e-39] * 20, np.float32))           # denormals beside normals
    lists.append(np.asarray([3.0e38, 1.0, 2.9e38, 1e-30] * 10, np.float32))         # near the largest float
    xadj, adj, w = _star_graph(lists)
    ctx.upload(xadj, adj, w)
    ctx.alias_build_offline()
    prob, alias, valid = ctx.alias_export()
    oprob, oalias, ovalid = oracle.alias_build(xadj, w)
    assert np.array_equal(valid, ovalid)
    assert np.array_equal(alias, oalias)
    assert np.array_equal(prob.view(np.uint32), oprob.view(np.uint32))


def test_alias_packed_builders_boundaries(ctx, oracle):
    """Lists on both sides of every boundary of the register-resident and packed-list builders
    (8 elements per lane; groups of 1..32 lanes; tiles of 256 and 2048; 4096), as skewed lists with
    zeros, uniform lists (no small at all), lists with one dominant weight and lists of all-equal
    pairs (ties between deficit and excess prefixes)."""
    rng = np.random.default_rng(2)
    lists = []
    for n in (1, 2, 7, 8, 9, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 128, 129, 250, 255, 256, 257, 600, 1024, 1025,
              2047, 2048, 2049, 4095, 4096, 4097):
        w = (rng.uniform(0, 1, n) ** 8).astype(np.float32)
        if n > 3:
            w[rng.integers(0, n, n // 5)] = 0.0
        w[rng.integers(0, n)] = 0.7
        lists.append(w)
        lists.append(np.full(n, 2.5, np.float32))
        d = rng.uniform(1, 2, n).astype(np.float32)
        d[rng.integers(0, n)] = 1.0e6
        lists.append(d)
        lists.append(np.tile(np.asarray([1.0, 3.0], np.float32), n // 2 + 1)[:n])
    xadj, adj, w = _star_graph(lists)
    ctx.upload(xadj, adj, w)
    ctx.alias_build_offline()
    prob, alias, valid = ctx.alias_export()
    oprob, oalias, ovalid = oracle.alias_build(xadj, w)
    assert np.array_equal(valid, ovalid)
    assert np.array_equal(alias, oalias)
    assert np.array_equal(prob.view(np.uint32), oprob.view(np.uint32))


def test_alias_weights_around_the_truncation_threshold(ctx, oracle):
    """A weight loses bits in the quantisation once it is more than 2^16 below the largest weight of its
    list (for up to 4096 weights): lists with one weight 2^15, 2^16, 2^17 and 2^24 times the others, with
    and without the lowest significand bit set, the large weight first, in the middle or everywhere but at
    the sampled positions; zeros; a largest weight that is barely normal; one near the largest float.  In
    every class that walks its list in more than one tile."""
    rng = np.random.default_rng(12)
    lists = []
    for n in (300, 1000, 1500, 4000, 6000, 12000, 20000):
        base = rng.uniform(1, 2, n).astype(np.float32)
        for ratio_log2 in (15, 16, 17, 24):               # smallest weight 2^-r of the largest
            w = base.copy()
            w[0] = 2.0 ** ratio_log2                        # the largest first
            lists.append(w)
            w = base.copy()
            w[n // 3] = np.float32(1.0 + 2.0 ** -23) * 2.0 ** ratio_log2   # lowest significand bit set
            lists.append(w)
            w = (base * 2.0 ** ratio_log2).astype(np.float32)
            w[0] = 1.0                                     # first, middle and last are small, the rest large
            w[n // 2] = 1.5
            w[n - 1] = 1.25
            lists.append(w)
        w = base.copy()
        w[5] = 0.0                                         # zeros do not count as small weights
        w[n - 1] = 0.0
        lists.append(w)
        w = base.copy() * np.float32(1e-38)                # the largest weight barely normal, others denormal
        lists.append(w.astype(np.float32))
        w = base.copy()
        w[n // 2] = 3.0e38                                 # near the largest float
        lists.append(w)
    xadj, adj, w = _star_graph(lists)
    ctx.upload(xadj, adj, w)
    ctx.alias_build_offline()
    prob, alias, valid = ctx.alias_export()
    oprob, oalias, ovalid = oracle.alias_build(xadj, w)
    assert np.array_equal(valid, ovalid)
    assert np.array_equal(alias, oalias)
    assert np.array_equal(prob.view(np.uint32), oprob.view(np.uint32))


def test_alias_build_partial_range(ctx, oracle, rmat12):
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline(0, g.V // 2)
    ctx.alias_build_offline(g.V // 2, g.V)
    prob, alias, valid = ctx.alias_export()
    oprob, oalias, ovalid = oracle.alias_build(g.xadj, g.adjwgt)
    assert np.array_equal(valid, ovalid) and np.array_equal(alias, oalias)
    assert np.array_equal(prob.view(np.uint32), oprob.view(np.uint32))


def test_alias_import_export(ctx, oracle, rmat12):
    g = rmat12
    _upload(ctx, g)
    table = oracle.alias_build(g.xadj, g.adjwgt)
    ctx.alias_import(*table)
    prob, alias, valid = ctx.alias_export()
    assert np.array_equal(prob, table[0]) and np.array_equal(alias, table[1]) and np.array_equal(valid, table[2])


def test_config1_deepwalk_bit_exact(ctx, oracle, rmat16):
    """benchmark configuration 1: 4,096 walkers, length 80, seed 42, tables from the oracle."""
    g = rmat16
    _upload(ctx, g)
    table = oracle.alias_build(g.xadj, g.adjwgt)
    ctx.alias_import(*table)
    starts = oracle.gen_starts(4096, g.V, 42)
    paths, lens, ms, edges = ctx.walk(starts, 81, app=APP_DEEPWALK, seed=42)
    opaths, olens = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, 81, seed=42)
    _cmp_walks(paths, lens, opaths, olens)
    assert edges == int(olens.sum())
    # the same through GPU-built tables
    ctx.alias_build_offline()
    paths2, lens2, _, _ = ctx.walk(starts, 81, app=APP_DEEPWALK, seed=42)
    _cmp_walks(paths2, lens2, opaths, olens)


@pytest.mark.parametrize("app,kw", [(APP_DEEPWALK, {}), (APP_PPR, {"tp": 0.15}), (APP_NODE2VEC, {"p": 2.0, "q": 0.5}),
                                    (APP_NODE2VEC, {"p": 0.25, "q": 4.0})])
@pytest.mark.parametrize("mode,flags", [(MODE_OFFLINE, 0), (MODE_ONLINE, 0), (MODE_ONLINE, 4), (MODE_ONLINE, 8)])
def test_walks_bit_exact(ctx, oracle, plaw, app, kw, mode, flags):
    # online: flags 4 (WALK_BUILD_TABLES) builds the tables of the frontier at every step, 8
    # (WALK_DIRECT_SLOTS) evaluates every drawn slot straight from the weights, 0 lets the library pick
    g = plaw
    _upload(ctx, g)
    table = oracle.alias_build(g.xadj, g.adjwgt)
    if mode == MODE_OFFLINE:
        ctx.alias_build_offline()
    starts = oracle.gen_starts(3000, g.V, 7)
    hop = 41 if app != APP_PPR else 101
    paths, lens, ms, edges = ctx.walk(starts, hop, app=app, mode=mode, seed=99, walker_base=1000, flags=flags, **kw)
    opaths, olens = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, hop, app=app, seed=99, walker_base=1000,
                                online=False, **kw)
    _cmp_walks(paths, lens, opaths, olens)
    assert edges == int(olens.sum())


@pytest.mark.parametrize("app,kw", [(APP_DEEPWALK, {}), (APP_PPR, {"tp": 0.15})])
@pytest.mark.parametrize("gname", ["rmat16", "plaw"])
def test_walk_records_bit_exact(ctx, oracle, request, gname, app, kw):
    """The fused 32-byte record layout gives the same walks as the oracle (and as the 8-byte slots)."""
    g = request.getfixturevalue(gname)
    _upload(ctx, g)
    ctx.alias_build_offline()
    table = oracle.alias_build(g.xadj, g.adjwgt)
    starts = oracle.gen_starts(4096, g.V, 42)
    hop = 81 if app != APP_PPR else 101
    base, blen, _, bedges = ctx.walk(starts, hop, app=app, seed=42, **kw)
    ctx.walk_records_build()
    paths, lens, _, edges = ctx.walk(starts, hop, app=app, seed=42, **kw)
    opaths, olens = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, hop, app=app, seed=42, **kw)
    _cmp_walks(paths, lens, opaths, olens)
    _cmp_walks(base, blen, opaths, olens)
    assert edges == bedges == int(olens.sum())
    ctx.walk_records_free()


def test_walk_records_dead_ends_and_invalid(ctx):
    xadj = np.asarray([0, 1, 1, 2, 3, 3, 5], np.uint32)
    adj = np.asarray([1, 3, 2, 0, 4], np.uint32)     # 5 -> {0 (unusable weights), 4 (isolated)}
    w = np.asarray([0.0, 1.0, 2.0, 1.0, 1.0], np.float32)
    ctx.upload(xadj, adj, w)
    ctx.alias_build_offline()
    ctx.walk_records_build()
    starts = np.asarray([0, 1, 2, 3, 4, 5, 5, 5, 5], np.uint32)
    paths, lens, _, edges = ctx.walk(starts, 6, seed=1)
    assert list(lens[:5]) == [0, 0, 5, 5, 0]
    assert list(paths[2]) == [2, 3, 2, 3, 2, 3]
    assert (lens[5:] == 1).all() and np.isin(paths[5:, 1], [0, 4]).all()
    ctx.walk_records_free()


def test_walk_dead_ends_and_invalid_vertices(ctx, oracle):
    # 0 -> 1 (weight 0: unusable), 2 -> 3 -> 2 cycle, 4 isolated
    xadj = np.asarray([0, 1, 1, 2, 3, 3], np.uint32)
    adj = np.asarray([1, 3, 2], np.uint32)
    w = np.asarray([0.0, 1.0, 2.0], np.float32)
    ctx.upload(xadj, adj, w)
    ctx.alias_build_offline()
    starts = np.asarray([0, 1, 2, 3, 4], np.uint32)
    for mode in (MODE_OFFLINE, MODE_ONLINE):
        paths, lens, _, edges = ctx.walk(starts, 6, mode=mode)
        assert list(lens) == [0, 0, 5, 5, 0]
        assert list(paths[2]) == [2, 3, 2, 3, 2, 3]
        assert edges == 10


def test_walk_empty_and_single_hop(ctx, rmat12):
    _upload(ctx, rmat12)
    ctx.alias_build_offline()
    paths, lens, _, edges = ctx.walk(np.zeros(0, np.uint32), 10)
    assert edges == 0
    paths, lens, _, edges = ctx.walk(np.asarray([5, 6], np.uint32), 1)
    assert list(paths[:, 0]) == [5, 6] and list(lens) == [0, 0]


def test_walk_sharding_is_invisible(ctx, oracle, rmat12):
    """Rows do not depend on how walkers are split between calls (multi-GPU sharding rule)."""
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline()
    starts = oracle.gen_starts(2000, g.V, 3)
    full, flen, _, _ = ctx.walk(starts, 31, app=APP_PPR, tp=0.1, seed=5)
    a, al, _, _ = ctx.walk(starts[:700], 31, app=APP_PPR, tp=0.1, seed=5, walker_base=0)
    b, bl, _, _ = ctx.walk(starts[700:], 31, app=APP_PPR, tp=0.1, seed=5, walker_base=700)
    _cmp_walks(np.vstack([a, b]), np.concatenate([al, bl]), full, flen)


def test_enqueue_only_walks(ctx, oracle, rmat12):
    import torch
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline()
    starts = oracle.gen_starts(2000, g.V, 3)
    ref_p, ref_l, _, ref_e = ctx.walk(starts, 31, app=APP_PPR, tp=0.1, seed=5)
    d_s = torch.from_numpy(starts.view(np.int32)).cuda()
    d_p = torch.zeros(2000 * 31, dtype=torch.int32, device="cuda")
    d_l = torch.zeros(2000, dtype=torch.int32, device="cuda")
    for _ in range(3):
        _, _, ms, e = ctx.walk(d_s, 31, app=APP_PPR, tp=0.1, seed=5, paths=d_p, lengths=d_l, enqueue_only=True)
        assert ms is None and e is None
    assert ctx.take_sampled_edges() == 3 * ref_e
    assert ctx.take_sampled_edges() == 0
    _cmp_walks(d_p.cpu().numpy().view(np.uint32).reshape(2000, 31), d_l.cpu().numpy().view(np.uint32), ref_p, ref_l)
    # a bad start vertex in an enqueued call is reported when the count is taken, and not twice
    from skywalker_b200.api import SkwError
    d_s[0] = g.V + 7
    ctx.walk(d_s, 31, paths=d_p, lengths=d_l, enqueue_only=True)
    with pytest.raises(SkwError):
        ctx.take_sampled_edges()
    d_s[0] = 0
    ctx.walk(d_s, 31, paths=d_p, lengths=d_l, enqueue_only=True)
    assert ctx.take_sampled_edges() > 0


def test_online_walk_with_cached_tables(ctx, oracle, plaw):
    from skywalker_b200 import WALK_CACHE_TABLES
    g = plaw
    _upload(ctx, g)
    starts = oracle.gen_starts(2000, g.V, 7)
    a, al, _, ae = ctx.walk(starts, 41, app=APP_NODE2VEC, mode=MODE_ONLINE, seed=9)
    launches = ctx.kernel_launches
    b, bl, _, be = ctx.walk(starts, 41, app=APP_NODE2VEC, mode=MODE_ONLINE, seed=9, flags=WALK_CACHE_TABLES)
    _cmp_walks(b, bl, a, al)
    assert ae == be
    c, cl, _, _ = ctx.walk(starts, 41, app=APP_NODE2VEC, mode=MODE_ONLINE, seed=10, flags=WALK_CACHE_TABLES)
    d, dl, _, _ = ctx.walk(starts, 41, app=APP_NODE2VEC, mode=MODE_ONLINE, seed=10)
    _cmp_walks(c, cl, d, dl)      # a new call starts a new round: nothing stale is reused wrongly


def test_walk_into_pinned_host_memory(ctx, oracle, rmat12):
    """Pinned result buffers receive only the cells each walk wrote; the rest keeps the caller's bytes."""
    import torch
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline()
    starts = oracle.gen_starts(5000, g.V, 3)
    ref_p, ref_l, _, ref_e = ctx.walk(starts, 101, app=APP_PPR, tp=0.15, seed=5)
    pin_p = torch.full((5000, 101), 0x5A5A5A5A, dtype=torch.int32).pin_memory()
    pin_l = torch.zeros(5000, dtype=torch.int32).pin_memory()
    p, l, _, e = ctx.walk(starts, 101, app=APP_PPR, tp=0.15, seed=5, paths=pin_p.numpy().view(np.uint32),
                          lengths=pin_l.numpy().view(np.uint32))
    assert e == ref_e and np.array_equal(l, ref_l)
    cols = np.arange(101)[None, :]
    live = cols <= l[:, None]
    assert np.array_equal(p[live], ref_p[live])
    assert (p[~live] == 0x5A5A5A5A).all()


def test_interleaved_walker_ids(ctx, oracle, rmat12):
    """Reference-style interleaving over 3 'GPUs' (id = dev + i*3) gives the rows of one big call."""
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline()
    table = oracle.alias_build(g.xadj, g.adjwgt)
    starts = oracle.gen_starts(1500, g.V, 8)
    full, flen, _, _ = ctx.walk(starts, 21, seed=4)
    for dev in range(3):
        sub = np.ascontiguousarray(starts[dev::3])
        p, l, _, _ = ctx.walk(sub, 21, seed=4, walker_base=dev, walker_stride=3)
        _cmp_walks(p, l, full[dev::3], flen[dev::3])
        op, ol = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, sub, 21, seed=4, walker_base=dev, walker_stride=3)
        _cmp_walks(p, l, op, ol)
    seeds = starts[:300]
    d, s_, _, _ = ctx.sample_khop(seeds, [5, 3], seed=9)
    d1, s1, _, _ = ctx.sample_khop(np.ascontiguousarray(seeds[1::2]), [5, 3], seed=9, instance_base=1, instance_stride=2)
    assert np.array_equal(d1, d[1::2]) and np.array_equal(s1, s_[1::2])


@pytest.mark.parametrize("mode", [MODE_OFFLINE, MODE_ONLINE])
@pytest.mark.parametrize("flags", [0, KHOP_TAKE_ALL])
def test_khop_bit_exact(ctx, oracle, rmat16, mode, flags):
    g = rmat16
    _upload(ctx, g)
    table = oracle.alias_build(g.xadj, g.adjwgt)
    if mode == MODE_OFFLINE:
        ctx.alias_build_offline()
    seeds = oracle.gen_starts(2048, g.V, 11)
    data, sl, ms, edges = ctx.sample_khop(seeds, [25, 10], mode=mode, flags=flags, seed=77, instance_base=3)
    odata, osl = oracle.khop(g.xadj, g.adjncy, g.adjwgt, table, seeds, [25, 10], flags=flags, seed=77,
                             instance_base=3)
    assert np.array_equal(sl, osl)
    assert np.array_equal(data, odata)
    assert edges == int(osl.sum())


def test_khop_three_hops_and_layout(ctx, oracle, rmat12):
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline()
    table = oracle.alias_build(g.xadj, g.adjwgt)
    assert ctx.khop_layout([25, 10]) == (276, 26)
    seeds = oracle.gen_starts(100, g.V, 2)
    data, sl, _, _ = ctx.sample_khop(seeds, [3, 4, 2])
    odata, osl = oracle.khop(g.xadj, g.adjncy, g.adjwgt, table, seeds, [3, 4, 2])
    assert np.array_equal(data, odata) and np.array_equal(sl, osl)


def test_chi_square_on_gpu_walks(ctx):
    from scipy import stats
    rng = np.random.default_rng(3)
    for n in (2, 7, 33, 300):
        w = rng.uniform(1, 10, n).astype(np.float32)
        xadj = np.asarray([0, n] + [n] * n, np.uint32)
        adj = np.arange(1, n + 1, dtype=np.uint32)
        ctx.upload(xadj, adj, w)
        ctx.alias_build_offline()
        N = 400000
        paths, lens, _, _ = ctx.walk(np.zeros(N, np.uint32), 2, seed=n)
        counts = np.bincount(paths[:, 1].astype(np.int64) - 1, minlength=n)
        wf = w.astype(np.float64)
        chi, pval = stats.chisquare(counts, f_exp=wf / wf.sum() * N)
        assert pval > 0.01, (n, pval)


def test_errors_are_reported_not_fatal(ctx, rmat12):
    from skywalker_b200.api import SkwError
    _upload(ctx, rmat12)
    with pytest.raises(SkwError):            # offline walk without a table
        ctx.walk(np.zeros(4, np.uint32), 5)
    ctx.alias_build_offline()
    with pytest.raises(SkwError):            # start vertex out of range: device error word, no fault
        ctx.walk(np.asarray([rmat12.V + 5], np.uint32), 5)
    with pytest.raises(SkwError):
        ctx.alias_build_offline(10, 5)
    paths, lens, _, _ = ctx.walk(np.asarray([1], np.uint32), 5)   # context still usable
    assert paths[0, 0] == 1


def test_degenerate_graphs(ctx, oracle):
    # no edges at all
    ctx.upload(np.zeros(6, np.uint32), np.zeros(0, np.uint32), np.zeros(0, np.float32))
    assert ctx.graph_info() == (5, 0, 0)
    ctx.alias_build_offline()
    prob, alias, valid = ctx.alias_export()
    assert len(prob) == 0 and (valid == 0).all()
    for mode in (MODE_OFFLINE, MODE_ONLINE):
        paths, lens, _, edges = ctx.walk(np.arange(5, dtype=np.uint32), 4, mode=mode)
        assert edges == 0 and (lens == 0).all() and list(paths[:, 0]) == [0, 1, 2, 3, 4]
        data, sl, _, e = ctx.sample_khop(np.arange(5, dtype=np.uint32), [3, 2], mode=mode)
        assert e == 0 and (sl == 0).all() and (data[:, 1:] == 0xFFFFFFFF).all()
    # one vertex with a self-contained 2-cycle partner, weights given as None (all ones)
    ctx.upload(np.asarray([0, 1, 2], np.uint32), np.asarray([1, 0], np.uint32), None)
    ctx.alias_build_offline()
    paths, lens, _, edges = ctx.walk(np.asarray([0], np.uint32), 7)
    assert list(paths[0]) == [0, 1, 0, 1, 0, 1, 0] and edges == 6
    # bad arguments come back as errors, not faults
    from skywalker_b200.api import SkwError
    with pytest.raises(SkwError):
        ctx.walk(np.asarray([0], np.uint32), 0)
    with pytest.raises(SkwError):
        ctx.walk(np.asarray([0], np.uint32), 5, app=APP_PPR, tp=1.5)
    with pytest.raises(SkwError):
        ctx.walk(np.asarray([0], np.uint32), 5, app=APP_NODE2VEC, p=0.0)
    with pytest.raises(SkwError):
        ctx.sample_khop(np.asarray([0], np.uint32), [3, 0])
    with pytest.raises(SkwError):
        ctx.upload(np.asarray([1, 2], np.uint32), np.asarray([0, 0], np.uint32), None)   # xadj[0] != 0


def test_offline_table_survives_weight_release(ctx, oracle, rmat12):
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline()
    ctx.free_weights()                                    # src/createTable.cu:175-177
    starts = oracle.gen_starts(500, g.V, 1)
    table = oracle.alias_build(g.xadj, g.adjwgt)
    paths, lens, _, _ = ctx.walk(starts, 21, seed=2)
    op, ol = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, 21, seed=2)
    _cmp_walks(paths, lens, op, ol)
    from skywalker_b200.api import SkwError
    with pytest.raises(SkwError):
        ctx.walk(starts, 21, mode=MODE_ONLINE)            # online needs the weights
    with pytest.raises(SkwError):
        ctx.alias_build_offline()


def test_random_gather_probe(ctx):
    g = ctx.probe_random_gather(1 << 30, 32)
    assert 5.0 < g < 500.0          # giga-accesses/s; ~40 on B200 beyond L2


def test_table_checkpoint(ctx, oracle, rmat12, plaw, tmp_path):
    from skywalker_b200.api import SkwError
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline()
    want = ctx.alias_export()
    path = str(tmp_path / "table.skw")
    ctx.alias_save(path)
    _upload(ctx, g)                       # fresh graph, no table
    with pytest.raises(SkwError):
        ctx.walk(np.zeros(2, np.uint32), 3)
    ctx.alias_load(path)
    got = ctx.alias_export()
    assert all(np.array_equal(a.view(np.uint8), b.view(np.uint8)) for a, b in zip(got, want))
    starts = oracle.gen_starts(300, g.V, 4)
    p1, l1, _, _ = ctx.walk(starts, 11, seed=6)
    op, ol = oracle.walk(g.xadj, g.adjncy, g.adjwgt, oracle.alias_build(g.xadj, g.adjwgt), starts, 11, seed=6)
    _cmp_walks(p1, l1, op, ol)
    _upload(ctx, plaw)                    # a different graph must refuse the file
    with pytest.raises(SkwError):
        ctx.alias_load(path)
    (tmp_path / "bad.skw").write_bytes(b"not a table")
    with pytest.raises(SkwError):
        ctx.alias_load(str(tmp_path / "bad.skw"))


def test_bounded_wait_runs_out_cleanly(ctx, rmat12):
    """A wait on a barrier nobody signals ends by itself with an error record; nothing hangs or faults."""
    lib = ctx._lib
    rc = lib.skw_selftest_bounded_wait(ctx._h)
    assert rc == -4 and b"bounded wait ran out" in lib.skw_last_error(ctx._h)
    _upload(ctx, rmat12)                     # the context keeps working
    ctx.alias_build_offline()
    assert ctx.walk(np.asarray([1, 2], np.uint32), 4)[0][0, 0] == 1


def test_walker_ids_beyond_32_bits(ctx, oracle, rmat12):
    """Global walker ids use both counter words: a base above 2^32 gives the oracle's rows."""
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline()
    table = oracle.alias_build(g.xadj, g.adjwgt)
    starts = oracle.gen_starts(700, g.V, 5)
    base = (1 << 40) + 12345
    p, l, _, _ = ctx.walk(starts, 31, app=APP_PPR, tp=0.05, seed=(1 << 50) + 7, walker_base=base)
    op, ol = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, 31, app=APP_PPR, tp=0.05, seed=(1 << 50) + 7,
                         walker_base=base)
    _cmp_walks(p, l, op, ol)
    low, ll, _, _ = ctx.walk(starts, 31, app=APP_PPR, tp=0.05, seed=(1 << 50) + 7, walker_base=12345)
    assert not np.array_equal(ll, l)          # the high word matters


@pytest.mark.parametrize("fanout", [[7], [2, 3, 2, 2]])
def test_khop_one_and_four_hops(ctx, oracle, rmat12, fanout):
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline()
    table = oracle.alias_build(g.xadj, g.adjwgt)
    seeds = oracle.gen_starts(300, g.V, 8)
    for mode in (MODE_OFFLINE, MODE_ONLINE):
        data, sl, _, e = ctx.sample_khop(seeds, fanout, mode=mode, seed=3, instance_base=1 << 33)
        odata, osl = oracle.khop(g.xadj, g.adjncy, g.adjwgt, table, seeds, fanout, seed=3, instance_base=1 << 33)
        assert np.array_equal(data, odata) and np.array_equal(sl, osl) and e == int(osl.sum())
    from skywalker_b200.api import SkwError
    with pytest.raises(SkwError):
        ctx.sample_khop(seeds, [2, 2, 2, 2, 2])      # more than 4 hops


def test_alias_giant_vertex(ctx, oracle):
    """One vertex with 8.6 M edges: bucket width drops below 40 bits, the scratch class needs more than
    one round of 1023 windows; still bit for bit the sequential sweep."""
    rng = np.random.default_rng(5)
    n = 8_600_000
    w = rng.uniform(1, 10, n).astype(np.float32)
    w[::1000] = 0.0
    xadj = np.asarray([0, n, n], np.uint32)
    adj = np.ones(n, np.uint32)
    ctx.upload(xadj, adj, w)
    ctx.alias_build_offline()
    prob, alias, valid = ctx.alias_export()
    oprob, oalias, ok = oracle.alias_vertex(w)
    assert ok and valid[0] == 1
    assert np.array_equal(alias, oalias)
    assert np.array_equal(prob.view(np.uint32), oprob.view(np.uint32))
    M, B = oracle.alias_vertex_masses(w)
    assert B == 38


@pytest.mark.parametrize("app,kw", [(APP_DEEPWALK, {}), (APP_PPR, {"tp": 0.15}), (APP_NODE2VEC, {"p": 2.0, "q": 0.5})])
def test_unbiased_walks_bit_exact(ctx, oracle, plaw, app, kw):
    # uniform neighbour choice: no table needed, neither weights (the graph goes up without them)
    g = plaw
    ctx.upload(g.xadj, g.adjncy, None)
    starts = oracle.gen_starts(3000, g.V, 7)
    hop = 41 if app != APP_PPR else 101
    paths, lens, ms, edges = ctx.walk(starts, hop, app=app, seed=5, walker_base=17, flags=WALK_UNBIASED, **kw)
    opaths, olens = oracle.walk(g.xadj, g.adjncy, None, None, starts, hop, app=app, seed=5, walker_base=17,
                                unbiased=True, **kw)
    _cmp_walks(paths, lens, opaths, olens)
    assert edges == int(olens.sum())
    # a resident table and walk records change nothing about an unbiased walk
    _upload(ctx, g)
    ctx.alias_build_offline()
    ctx.walk_records_build()
    paths2, lens2, _, _ = ctx.walk(starts, hop, app=app, mode=MODE_ONLINE, seed=5, walker_base=17,
                                   flags=WALK_UNBIASED, **kw)
    assert np.array_equal(lens2, lens) and np.array_equal(paths2, paths)
    # (DeepWalk and PPR then follow the walk records: one access per step.)  Not when a vertex with
    # out-edges has no usable table -- its record would say "no way on", which holds for a biased walk only
    w = g.adjwgt.copy()
    hub = int(np.argmax(np.diff(g.xadj.astype(np.int64))))
    w[g.xadj[hub]:g.xadj[hub + 1]] = 0.0
    ctx.upload(g.xadj, g.adjncy, w)
    ctx.alias_build_offline()
    ctx.walk_records_build()
    paths3, lens3, _, _ = ctx.walk(starts, hop, app=app, seed=5, walker_base=17, flags=WALK_UNBIASED, **kw)
    assert np.array_equal(lens3, lens) and np.array_equal(paths3, paths)


@pytest.mark.parametrize("flags", [0, KHOP_TAKE_ALL])
def test_unbiased_khop_bit_exact(ctx, oracle, rmat16, flags):
    g = rmat16
    ctx.upload(g.xadj, g.adjncy, None)
    seeds = oracle.gen_starts(2048, g.V, 11)
    data, sl, ms, edges = ctx.sample_khop(seeds, [25, 10], flags=flags | KHOP_UNBIASED, seed=77, instance_base=3)
    odata, osl = oracle.khop(g.xadj, g.adjncy, None, None, seeds, [25, 10], flags=flags | 2, seed=77,
                             instance_base=3)
    assert np.array_equal(sl, osl)
    assert np.array_equal(data, odata)
    assert edges == int(osl.sum())


@pytest.mark.parametrize("pinned", [False, True])
def test_packed_host_result_matches_rows(ctx, oracle, plaw, pinned):
    import torch
    from skywalker_b200.api import SkwError
    g = plaw
    _upload(ctx, g)
    ctx.alias_build_offline()
    table = oracle.alias_build(g.xadj, g.adjwgt)
    starts = oracle.gen_starts(5000, g.V, 21)
    opaths, olens = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, 101, app=APP_PPR, tp=0.15, seed=13)
    want = np.concatenate([opaths[w, :olens[w] + 1] for w in range(len(starts))])
    cap = len(want) + 7
    if pinned:
        buf = torch.empty(cap, dtype=torch.int32).pin_memory()
        packed = buf.numpy().view(np.uint32)
    else:
        packed = np.zeros(cap, np.uint32)
    packed[:] = 0xABCDEF01
    out, lens, cells, ms, edges = ctx.walk_packed(starts, 101, app=APP_PPR, tp=0.15, seed=13, packed=packed)
    assert cells == len(want) == edges + len(starts)
    assert np.array_equal(lens, olens)
    assert np.array_equal(out[:cells], want)
    assert (out[cells:] == 0xABCDEF01).all()              # nothing written past the result
    # a buffer that is too small: lengths and the needed size come back, nothing is written, the context lives on
    small = np.full(cells - 1, 0xABCDEF01, np.uint32)
    lens2 = np.zeros(len(starts), np.uint32)
    with pytest.raises(SkwError) as e:
        ctx.walk_packed(starts, 101, app=APP_PPR, tp=0.15, seed=13, packed=small, lengths=lens2)
    assert str(cells) in str(e.value)
    assert np.array_equal(lens2, olens) and (small == 0xABCDEF01).all()
    # no walkers
    _, _, cells0, _, edges0 = ctx.walk_packed(np.zeros(0, np.uint32), 101, app=APP_PPR, tp=0.15, seed=13)
    assert cells0 == 0 and edges0 == 0
    # fixed-length walks fill whole rows
    out3, lens3, cells3, _, _ = ctx.walk_packed(starts[:100], 11, seed=3)
    p3, l3 = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts[:100], 11, seed=3)
    assert np.array_equal(out3[:cells3], np.concatenate([p3[w, :l3[w] + 1] for w in range(100)]))
    # lengths as bytes (skw_walk_packed_u8): the same walks, one byte per length
    packed[:] = 0xABCDEF01
    out8, lens8, cells8, _, edges8 = ctx.walk_packed(starts, 101, app=APP_PPR, tp=0.15, seed=13, packed=packed,
                                                     lengths_u8=True)
    assert lens8.dtype == np.uint8 and np.array_equal(lens8, olens)
    assert cells8 == cells and edges8 == edges and np.array_equal(out8[:cells8], want)
    assert (out8[cells8:] == 0xABCDEF01).all()
    out9, lens9, cells9, _, _ = ctx.walk_packed(starts[:100], 256, seed=3, lengths_u8=True)     # lengths up to 255
    p9, l9 = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts[:100], 256, seed=3)
    assert np.array_equal(lens9, l9) and np.array_equal(out9[:cells9], np.concatenate([p9[w, :l9[w] + 1] for w in range(100)]))
    with pytest.raises(SkwError):                                                            # 256 does not fit a byte
        ctx.walk_packed(starts[:100], 257, seed=3, lengths_u8=True)


def test_online_direct_slots_every_degree_class(ctx, oracle):
    """The online walk computes the slot it draws without a table: one step from every list of the
    degree-class zoo, enough walkers per list to draw most columns, against the oracle's built tables."""
    rng = np.random.default_rng(5)
    lists = []
    for n in [1, 2, 3, 4, 5, 31, 32, 33, 127, 128, 129, 255, 256, 257, 1000, 4097, 20000, 70000]:
        lists.append(rng.uniform(1, 10, n).astype(np.float32))
    lists.append(np.asarray([0.5] * 35 + [2.0] * 5, np.float32))
    lists.append(np.full(130, 3.0, np.float32))                        # uniform: every slot is its own bucket
    lists.append(np.asarray([1e-3] * 300 + [1000.0], np.float32))      # one dominant weight at the end
    lists.append(np.asarray([1000.0] + [1e-3] * 300, np.float32))      # ... and at the start
    lists.append(np.zeros(100, np.float32))                            # no usable weight: the walk ends
    lists.append(np.asarray([0, 1, 2, 0, 5] * 40, np.float32))         # zeros inside
    lists.append(np.asarray([np.nan, -1, np.inf, 2, 3], np.float32))
    lists.append(rng.uniform(0, 1, 3000).astype(np.float32) ** 8)      # skewed, many tiny
    lists.append(np.asarray([1e-40, 2e-40, 3e-41, 0, 1e-45], np.float32))           # denormals only
    lists.append(np.asarray([1e-38, 1e-40, 1.0, 3e-39] * 20, np.float32))           # denormals beside normals
    lists.append(np.asarray([3.0e38, 1.0, 2.9e38, 1e-30] * 10, np.float32))         # near the largest float
    # long lists whose crossings lie far from the drawn slot (the prefix checkpoints of lists of 2,048
    # weights and more decide where a sweep starts)
    lists.append(np.concatenate([np.full(5000, 1e-3), rng.uniform(1, 2, 5000)]).astype(np.float32))   # smalls, then larges
    lists.append(np.concatenate([rng.uniform(1, 2, 5000), np.full(5000, 1e-3)]).astype(np.float32))   # larges, then smalls
    lists.append(np.full(5000, 2.5, np.float32))                                                       # no small at all
    lists.append(np.asarray([1000.0] + [1e-3] * 6000, np.float32))                                     # one donor for 6000 smalls
    lists.append(np.asarray([1e-3] * 6000 + [1000.0], np.float32))
    lists.append(np.tile(np.asarray([1.0, 3.0], np.float32), 1500))                                    # ties between the prefixes
    lists.append(rng.uniform(1, 10, 2048).astype(np.float32))                                          # exactly one checkpoint
    lists.append(rng.uniform(1, 10, 2049).astype(np.float32))
    lists.append(rng.uniform(1, 10, 3073).astype(np.float32))
    xadj, adj, w = _star_graph(lists)
    ctx.upload(xadj, adj, w)
    starts = np.concatenate([np.full(min(4 * len(l), 6000), i, np.uint32) for i, l in enumerate(lists)])
    paths, lens, _, edges = ctx.walk(starts, 3, mode=MODE_ONLINE, seed=31, flags=8)
    opaths, olens = oracle.walk(xadj, adj, w, None, starts, 3, online=True, seed=31)
    _cmp_walks(paths, lens, opaths, olens)
    assert edges == int(olens.sum())
    built, blens, _, _ = ctx.walk(starts, 3, mode=MODE_ONLINE, seed=31, flags=4)
    _cmp_walks(built, blens, opaths, olens)


def test_ppr_records_chunk_edges_and_long_rows(ctx, oracle, rmat12):
    """The chunked PPR kernel: walker counts around its chunk size, paths longer than its staging
    rows, and rows too long for it (hop_num > 65535 takes the lane-per-walker kernel)."""
    g = rmat12
    _upload(ctx, g)
    ctx.alias_build_offline()
    ctx.walk_records_build()
    table = oracle.alias_build(g.xadj, g.adjwgt)
    for n in (1, 63, 64, 65, 511, 513):
        starts = oracle.gen_starts(n, g.V, 100 + n)
        paths, lens, _, edges = ctx.walk(starts, 40, app=APP_PPR, tp=0.02, seed=n, walker_base=7)   # long walks
        opaths, olens = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, 40, app=APP_PPR, tp=0.02, seed=n,
                                    walker_base=7)
        _cmp_walks(paths, lens, opaths, olens)
        assert edges == int(olens.sum())
    starts = oracle.gen_starts(48, g.V, 3)
    paths, lens, _, _ = ctx.walk(starts, 70000, app=APP_PPR, tp=0.3, seed=2)
    opaths, olens = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, 70000, app=APP_PPR, tp=0.3, seed=2)
    _cmp_walks(paths, lens, opaths, olens)


def test_packed_result_sliced_pipeline(ctx, oracle, rmat16):
    """Batches of a million walkers and more leave the GPU slice by slice; the packed result and the
    lengths are those of one big call, whatever the slicing."""
    from skywalker_b200.api import SkwError
    g = rmat16
    _upload(ctx, g)
    ctx.alias_build_offline()
    table = oracle.alias_build(g.xadj, g.adjwgt)
    for n in ((1 << 20) + 12345, (1 << 21) + 77):          # two slices, four slices
        starts = oracle.gen_starts(n, g.V, 5)
        opaths, olens = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, 21, app=APP_PPR, tp=0.3, seed=8,
                                    walker_base=11)
        live = np.arange(21)[None, :] <= olens[:, None]
        want = opaths[live]                                  # row-major: walks back to back
        out, lens, cells, ms, edges = ctx.walk_packed(starts, 21, app=APP_PPR, tp=0.3, seed=8, walker_base=11)
        assert cells == len(want) and edges == int(olens.sum()) and ms > 0
        assert np.array_equal(lens, olens)
        assert np.array_equal(out[:cells], want)
        out8, lens8, cells8, _, _ = ctx.walk_packed(starts, 21, app=APP_PPR, tp=0.3, seed=8, walker_base=11,
                                                    lengths_u8=True)           # byte lengths, slice by slice
        assert cells8 == cells and np.array_equal(lens8, olens) and np.array_equal(out8[:cells], want)
        # too small by one cell: the overflow shows up in the last slice; lengths and size still come back
        small = np.zeros(cells - 1, np.uint32)
        lens2 = np.zeros(n, np.uint32)
        with pytest.raises(SkwError) as e:
            ctx.walk_packed(starts, 21, app=APP_PPR, tp=0.3, seed=8, walker_base=11, packed=small, lengths=lens2)
        assert str(cells) in str(e.value) and np.array_equal(lens2, olens)
    # the packing buffers keep the size the PPR calls gave them; fixed-length walks of the same batch
    # outgrow them, so every slice is packed a second time into a larger buffer
    n = (1 << 20) + 5
    starts = oracle.gen_starts(n, g.V, 6)
    opaths, olens = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, 11, seed=9)
    live = np.arange(11)[None, :] <= olens[:, None]
    out, lens, cells, _, edges = ctx.walk_packed(starts, 11, seed=9)
    assert cells == int(live.sum()) and edges == int(olens.sum())
    assert np.array_equal(lens, olens) and np.array_equal(out[:cells], opaths[live])


def test_malformed_csr_is_refused(ctx, rmat12):
    """A CSR with decreasing offsets or a destination >= V is refused at upload / adopt with an error
    code (no kernel ever indexes with it), and the context stays usable."""
    import torch
    from skywalker_b200.api import SkwError
    g = rmat12
    bad_x = g.xadj.copy()
    bad_x[5], bad_x[6] = bad_x[6] + 3, bad_x[5]            # offsets go down
    with pytest.raises(SkwError) as e:
        ctx.upload(bad_x, g.adjncy, g.adjwgt)
    assert e.value.code == -1
    bad_a = g.adjncy.copy()
    bad_a[len(bad_a) // 2] = g.V + 7                       # destination out of range
    with pytest.raises(SkwError) as e:
        ctx.upload(g.xadj, bad_a, g.adjwgt)
    assert e.value.code == -1
    d_x = torch.from_numpy(g.xadj.astype(np.int32)).cuda()
    d_a = torch.from_numpy(bad_a.astype(np.int64).astype(np.int32)).cuda()
    with pytest.raises(SkwError) as e:
        ctx.adopt_device(g.V, g.E, d_x, d_a)
    assert e.value.code == -1
    with pytest.raises(SkwError):                          # nothing resident after a refusal
        ctx.alias_build_offline()
    _upload(ctx, g)
    ctx.alias_build_offline()
    paths, lens, _, _ = ctx.walk(np.asarray([1], np.uint32), 5)
    assert paths[0, 0] == 1


def test_foreign_or_corrupt_table_is_refused(ctx, oracle, rmat12, tmp_path):
    """Tables that do not fit the resident graph: an imported alias outside its list, a checkpoint of
    another graph with the same V and E, a checkpoint with a corrupted slot."""
    from skywalker_b200.api import SkwError
    g = rmat12
    _upload(ctx, g)
    prob, alias, valid = oracle.alias_build(g.xadj, g.adjwgt)
    bad = alias.copy()
    v = int(np.argmax(np.diff(g.xadj.astype(np.int64)) > 3))
    bad[g.xadj[v]] = 1 << 20
    with pytest.raises(SkwError) as e:
        ctx.alias_import(prob, bad, valid)
    assert e.value.code == -1
    with pytest.raises(SkwError):                          # the refused table is not usable
        ctx.walk(np.zeros(2, np.uint32), 3)
    ctx.alias_import(prob, alias, valid)
    path = str(tmp_path / "t.skw")
    ctx.alias_save(path)
    # same V and E, other offsets: move one edge from vertex a to vertex b
    deg = np.diff(g.xadj.astype(np.int64))
    a = int(np.argmax(deg > 2))
    x2 = g.xadj.astype(np.int64).copy()
    if a + 1 < g.V:
        x2[a + 1] -= 1                                      # vertex a loses its last edge to a + 1
    ctx.upload(x2.astype(np.uint32), g.adjncy, g.adjwgt)
    with pytest.raises(SkwError) as e:
        ctx.alias_load(path)
    assert "another graph" in str(e.value)
    # right graph, one slot of the file overwritten with an alias far outside its list
    _upload(ctx, g)
    raw = bytearray(open(path, "rb").read())
    slot0 = 48 + 8 * int(g.xadj[v])
    raw[slot0 + 4:slot0 + 8] = (0x7FFFFFF0).to_bytes(4, "little")
    open(path, "wb").write(bytes(raw))
    with pytest.raises(SkwError) as e:
        ctx.alias_load(path)
    assert e.value.code == -1


def test_walk_over_a_partly_built_table_ends_at_unbuilt_vertices(ctx, oracle, rmat12):
    """After a build of a vertex slice only, walkers that reach a vertex outside the slice stop
    there (its slots still say "no table"), they do not read garbage."""
    g = rmat12
    _upload(ctx, g)
    half = g.V // 2
    ctx.alias_build_offline(0, half)
    starts = oracle.gen_starts(2000, g.V, 8)
    paths, lens, _, _ = ctx.walk(starts, 21, seed=3)
    prob, alias, valid = oracle.alias_build(g.xadj, g.adjwgt)
    valid2 = valid.copy()
    valid2[half:] = 0
    op, ol = oracle.walk(g.xadj, g.adjncy, g.adjwgt, (prob, alias, valid2), starts, 21, seed=3)
    _cmp_walks(paths, lens, op, ol)
    assert (ol == 0).any() and (ol > 0).any()


@pytest.mark.parametrize("mode", [MODE_OFFLINE, MODE_ONLINE])
def test_khop_distinct_bit_exact(ctx, oracle, rmat16, rmat12, mode):
    """SKW_KHOP_DISTINCT (the rule of the reference's online sampler, src/online_sample_new.cu:73-111):
    bit-exact against the oracle, children of one parent are distinct, a parent whose degree is at most
    the fan-out hands over all of its neighbours."""
    from skywalker_b200 import KHOP_DISTINCT
    for g, fanout, nseeds in ((rmat16, [25, 10], 1500), (rmat12, [6, 5], 800), (rmat12, [40], 500)):
        _upload(ctx, g)
        ctx.alias_build_offline()
        table = oracle.alias_build(g.xadj, g.adjwgt)
        seeds = oracle.gen_starts(nseeds, g.V, 12)
        data, sl, _, edges = ctx.sample_khop(seeds, fanout, mode=mode, flags=KHOP_DISTINCT, seed=9)
        odata, osl = oracle.khop(g.xadj, g.adjncy, g.adjwgt, table, seeds, fanout, online=(mode == MODE_ONLINE),
                                 flags=KHOP_DISTINCT, seed=9)
        assert np.array_equal(sl, osl)
        assert np.array_equal(data, odata)
        assert edges == int(sl.sum())
        deg = np.diff(g.xadj.astype(np.int64))
        f1 = fanout[0]
        for s in range(0, nseeds, 7):                      # hop 1 of a sample of the seeds
            d = int(deg[seeds[s]])
            kids = data[s, 1:1 + f1]
            got = int(sl[s, 0])
            assert got == min(d, f1) or (d > f1 and got <= f1)
            assert (kids[got:] == 0xFFFFFFFF).all()
            lo, hi = int(g.xadj[seeds[s]]), int(g.xadj[seeds[s] + 1])
            if d <= f1:
                assert np.array_equal(kids[:got], g.adjncy[lo:hi])
            else:
                assert len(set(kids[:got].tolist())) == got   # adjacency lists hold no duplicates


def test_khop_distinct_runs_out_of_trials(ctx, oracle):
    """One neighbour carries almost all the weight: most trials repeat it, so fewer than fan-out
    distinct neighbours are found within the 352 trials, and the length says how many."""
    from skywalker_b200 import KHOP_DISTINCT
    n = 64
    w = np.full(n, 1e-6, np.float32)
    w[5] = 1.0
    xadj = np.asarray([0, n] + [n] * n, np.uint32)
    adj = np.arange(1, n + 1, dtype=np.uint32)
    ctx.upload(xadj, adj, w)
    ctx.alias_build_offline()
    table = oracle.alias_build(xadj, w)
    seeds = np.zeros(300, np.uint32)
    data, sl, _, _ = ctx.sample_khop(seeds, [20], flags=KHOP_DISTINCT, seed=4)
    odata, osl = oracle.khop(xadj, adj, w, table, seeds, [20], flags=KHOP_DISTINCT, seed=4)
    assert np.array_equal(sl, osl) and np.array_equal(data, odata)
    assert (sl[:, 0] >= 1).all() and (sl[:, 0] < 20).any()
    with pytest.raises(Exception):                          # fan-outs above 256 are refused with the flag
        ctx.sample_khop(seeds, [300], flags=KHOP_DISTINCT, seed=4)


@pytest.mark.parametrize("n", [3000, (1 << 16) + 1234])               # one slice, two slices
@pytest.mark.parametrize("mode,flags", [(MODE_OFFLINE, 0), (MODE_ONLINE, 0), (MODE_ONLINE, KHOP_DISTINCT),
                                        (MODE_OFFLINE, KHOP_TAKE_ALL)])
def test_khop_packed_host_result(ctx, oracle, rmat16, mode, flags, n):
    """skw_sample_khop_packed: the cells of the dense tree that hold a sample, seed after seed in row order,
    plus the per-vertex sample counts; a buffer that is too small gets the counts and the needed size."""
    from skywalker_b200.api import SkwError
    g = rmat16
    _upload(ctx, g)
    ctx.alias_build_offline()
    table = oracle.alias_build(g.xadj, g.adjwgt)
    seeds = oracle.gen_starts(n, g.V, 17)
    fan = [5, 3]
    odata, osl = oracle.khop(g.xadj, g.adjncy, g.adjwgt, table, seeds, fan, online=(mode == MODE_ONLINE),
                             seed=29, instance_base=7, flags=flags)
    want = odata[odata != INVALID_VERTEX]                  # row-major: seeds back to back, rows in order
    packed = np.full(len(want) + 5, 0xABCDEF01, np.uint32)
    out, sl, cells, ms, edges = ctx.sample_khop_packed(seeds, fan, mode=mode, flags=flags, seed=29, instance_base=7,
                                                       packed=packed)
    assert cells == len(want) and edges == int(osl.sum())
    assert np.array_equal(sl, osl)
    assert np.array_equal(out[:cells], want) and (out[cells:] == 0xABCDEF01).all()
    small = np.full(cells - 1, 0xABCDEF01, np.uint32)
    sl2 = np.zeros_like(osl)
    with pytest.raises(SkwError) as e:
        ctx.sample_khop_packed(seeds, fan, mode=mode, flags=flags, seed=29, instance_base=7, packed=small,
                               sample_lengths=sl2)
    assert str(cells) in str(e.value) and np.array_equal(sl2, osl)
    # the dense entry point still works on the same context afterwards
    data, sl3, _, _ = ctx.sample_khop(seeds[:100], fan, mode=mode, flags=flags, seed=29, instance_base=7)
    assert np.array_equal(data, odata[:100]) and np.array_equal(sl3, osl[:100])


@pytest.mark.parametrize("n", [(1 << 16) + 1234, (1 << 19) + 77])     # two slices, four slices
@pytest.mark.parametrize("mode", [MODE_OFFLINE, MODE_ONLINE])
def test_khop_host_entry_sliced_pipeline(ctx, oracle, rmat16, mode, n):
    """Batches of 2^16 seeds and more run as slices whose result copies overlap the next slice's
    kernels (online: a table built for an earlier slice or hop is not built again): the host entry
    point returns what the oracle computes, slice boundaries included."""
    g = rmat16
    _upload(ctx, g)
    ctx.alias_build_offline()
    seeds = oracle.gen_starts(n, g.V, 21)
    data, sl, _, edges = ctx.sample_khop(seeds, [3, 2], mode=mode, seed=13, instance_base=5)
    assert edges == int(sl.sum())
    table = oracle.alias_build(g.xadj, g.adjwgt)
    pick = np.concatenate([np.arange(0, 2000), np.arange(n // 2 - 1000, n // 2 + 1000), np.arange(n - 2000, n)])
    for lo in (0, n // 2 - 1000, n - 2000):
        sel = np.arange(lo, lo + 2000)
        odata, osl = oracle.khop(g.xadj, g.adjncy, g.adjwgt, table, seeds[sel], [3, 2], online=(mode == MODE_ONLINE),
                                 seed=13, instance_base=5 + lo)
        assert np.array_equal(data[sel], odata) and np.array_equal(sl[sel], osl)


@pytest.mark.parametrize("app,kw", [(APP_DEEPWALK, {}), (APP_PPR, {"tp": 0.15})])
def test_walk_host_rows_large_batch_scatter(ctx, oracle, rmat16, app, kw):
    """Batches of 2^18 walkers and more reach the caller's n x hop_num host matrix as a packed transfer
    that host threads scatter into the rows: every row equals the oracle's, and cells past a walk's end
    keep what the caller had there."""
    g = rmat16
    _upload(ctx, g)
    ctx.alias_build_offline()
    n, hop = (1 << 18) + 777, 21
    starts = oracle.gen_starts(n, g.V, 31)
    paths = np.full((n, hop), 0xABABABAB, np.uint32)
    lens = np.zeros(n, np.uint32)
    _, _, _, edges = ctx.walk(starts, hop, app=app, seed=8, walker_base=11, paths=paths, lengths=lens, **kw)
    table = oracle.alias_build(g.xadj, g.adjwgt)
    op, ol = oracle.walk(g.xadj, g.adjncy, g.adjwgt, table, starts, hop, app=app, seed=8, walker_base=11,
                         fill=0xABABABAB, **kw)
    assert np.array_equal(lens, ol) and edges == int(ol.sum())
    assert np.array_equal(paths, op)
