"""Host-side logic of the multi-GPU path, run as two gloo ranks on the CPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n_total, out_dir):
    sys.path.insert(0, ROOT)
    import bench
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # every rank owns a contiguous range of global walker ids; the oracle stands in for the kernels
    x, a = O.gen_rmat(10, 16 << 10, seed=1)
    w = O.gen_weights(len(a), 7)
    table = O.alias_build(x, w)
    lo, n_local = bench.shard(n_total, world, rank)
    starts = O.gen_starts(n_local, len(x) - 1, 42, id_base=lo)
    paths, lens = O.walk(x, a, w, table, starts, 21, app=O.PPR, tp=0.15, seed=5, walker_base=lo)
    mx, sm = bench.combine_over_ranks(dist, [float(rank + 1), float(lens.sum())])
    # results gather to rank 0, as bench.py does with the per-walker lengths
    sizes = [bench.shard(n_total, world, r)[1] for r in range(world)]
    pad = max(sizes)
    mine = torch.zeros(pad, dtype=torch.int64)
    mine[:n_local] = torch.from_numpy(lens.astype(np.int64))
    bufs = [torch.zeros(pad, dtype=torch.int64) for _ in range(world)] if rank == 0 else None
    dist.gather(mine, bufs, dst=0)
    if rank == 0:
        got = np.concatenate([b.numpy()[:s] for b, s in zip(bufs, sizes)])
        np.save(os.path.join(out_dir, "gathered.npy"), got)
        np.save(os.path.join(out_dir, "stats.npy"), np.asarray([mx[0], sm[1]]))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_walks_equal_single_rank(tmp_path, oracle):
    sys.path.insert(0, ROOT)
    import bench
    n_total, world = 1001, 2          # odd on purpose: ragged shards
    assert [bench.shard(n_total, world, r) for r in range(world)] == [(0, 500), (500, 501)]
    assert sum(bench.shard(7, 8, r)[1] for r in range(8)) == 7
    mp.spawn(_worker, args=(world, _free_port(), n_total, str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "gathered.npy")
    stats = np.load(tmp_path / "stats.npy")
    x, a = oracle.gen_rmat(10, 16 << 10, seed=1)
    w = oracle.gen_weights(len(a), 7)
    table = oracle.alias_build(x, w)
    starts = oracle.gen_starts(n_total, len(x) - 1, 42)
    _, lens = oracle.walk(x, a, w, table, starts, 21, app=oracle.PPR, tp=0.15, seed=5)
    assert np.array_equal(got, lens.astype(np.int64))       # the split is invisible in the result
    assert stats[0] == 2.0 and stats[1] == float(lens.sum())  # max over ranks, sum over ranks


def test_edge_balanced_ranges_partition_the_vertices(oracle):
    sys.path.insert(0, ROOT)
    from skywalker_b200.api import edge_balanced_ranges
    x, a = oracle.gen_rmat(12, 16 << 12, seed=2)
    E = int(x[-1])
    for parts in (1, 2, 3, 8):
        r = edge_balanced_ranges(x, parts)
        assert r[0][0] == 0 and r[-1][1] == len(x) - 1
        assert all(r[i][1] == r[i + 1][0] for i in range(parts - 1))
        sizes = [int(x[e]) - int(x[b]) for b, e in r]
        assert sum(sizes) == E
        assert max(sizes) <= E // parts + int(np.diff(x.astype(np.int64)).max()) + parts
    # degenerate: empty graph, more parts than vertices
    assert edge_balanced_ranges(np.zeros(3, np.uint32), 4) == [(0, 0), (0, 0), (0, 0), (0, 2)]


def test_edge_chunk_ranges_cover_every_chunk(oracle):
    sys.path.insert(0, ROOT)
    from skywalker_b200.api import edge_chunk_ranges
    x, a = oracle.gen_rmat(12, 16 << 12, seed=2)
    E, V = int(x[-1]), len(x) - 1
    for parts in (1, 2, 3, 8):
        S, r = edge_chunk_ranges(x, parts)
        assert S * parts >= E and S * (parts - 1) < E + S
        assert r[0][0] == 0 and r[-1][1] == V
        covered = np.zeros(V, bool)
        for k, (vb, ve) in enumerate(r):
            covered[vb:ve] = True
            lo, hi = min(k * S, E), min((k + 1) * S, E)
            if hi > lo:     # every slot of the chunk belongs to a vertex of the range
                assert int(x[vb]) <= lo and int(x[ve]) >= hi
        assert covered.all()
    S, r = edge_chunk_ranges(np.zeros(5, np.uint32), 3)
    assert r[0][0] == 0 and r[-1][1] == 4 and all(b <= e for b, e in r)


def test_pipelined_table_assembly_covers_the_table(oracle):
    """The multi-GPU table build of bench.py and the command-line driver: the slot array in N * P equal
    chunks, rank r builds chunks r, N + r, 2N + r ..., piece k (chunks k*N .. k*N + N - 1) is all-gathered in
    place while piece k + 1 is built.  Simulated on the CPU with the oracle as builder: the pieces tile the
    slot array without a gap, every rank's chunk sits where the in-place all-gather expects it, and the
    assembled table equals the table built in one go."""
    sys.path.insert(0, ROOT)
    from skywalker_b200.api import edge_chunk_ranges
    x, a = oracle.gen_rmat(11, 12 << 11, seed=5)
    w = oracle.gen_weights(len(a), 3)
    E, V = int(x[-1]), len(x) - 1
    prob, alias, valid = oracle.alias_build(x, w)
    for world, pieces in ((2, 4), (4, 4), (8, 4), (3, 2)):
        S, ranges = edge_chunk_ranges(x, world * pieces)
        assert world * pieces * S >= E > (world * pieces - 1) * S - S
        got_p = np.full(world * pieces * S, np.nan, np.float32)
        got_a = np.zeros(world * pieces * S, np.uint32)
        got_v = np.zeros(V, np.uint8)
        for k in range(pieces):
            piece = slice(k * world * S, (k + 1) * world * S)          # the all-gather's receive buffer
            for rank in range(world):
                c = k * world + rank
                assert piece.start + rank * S == c * S                 # in place: send buffer inside it
                vb, ve = ranges[c]
                p_r, a_r, v_r = oracle.alias_build(x, w, vb, ve)       # this rank's build of its vertices
                lo, hi = min(c * S, E), min((c + 1) * S, E)
                got_p[lo:hi] = p_r[lo:hi]                              # what the gather takes from this rank
                got_a[lo:hi] = a_r[lo:hi]
                got_v[vb:ve] = np.maximum(got_v[vb:ve], v_r[vb:ve])    # flags: all-reduce (max)
        assert np.array_equal(got_p[:E].view(np.uint32), prob.view(np.uint32))
        assert np.array_equal(got_a[:E], alias) and np.array_equal(got_v, valid)
