#!/usr/bin/env python
"""Generates tests/golden/small_graph.npz from the CPU oracle.

    python tests/golden/make_golden.py

The reference ships no golden vectors for this path (its outputs are not reproducible), so the
fixture pins the definitions of this build instead: a seeded R-MAT graph (scale 8, 16 edges per
vertex, plus one hub and hand-made corner vertices), its alias table, and walks / k-hop trees for
every application and mode, weighted and unbiased.  Tests compare both the oracle (so that it cannot drift silently) and
the CUDA library against the stored arrays.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as O  # noqa: E402


def build_inputs():
    x, a = O.gen_rmat(8, 16 << 8, 0.57, 0.19, 0.19, True, seed=11)     # symmetric: node2vec needs it
    w = O.gen_weights(len(a), 12)
    # corner vertices appended: a hub pointing at everybody, a vertex with zero weights, an isolated one
    V = len(x) - 1
    hub = np.arange(V, dtype=np.uint32)
    hub_w = (1.0 + (np.arange(V) % 17) * 0.5).astype(np.float32)
    dead = np.asarray([0, 1, 2], np.uint32)
    dead_w = np.zeros(3, np.float32)
    adj = np.concatenate([a, hub, dead]).astype(np.uint32)
    wgt = np.concatenate([w, hub_w, dead_w]).astype(np.float32)
    xadj = np.concatenate([x, [x[-1] + V, x[-1] + V + 3, x[-1] + V + 3]]).astype(np.uint32)
    return xadj, adj, wgt


def main():
    xadj, adj, wgt = build_inputs()
    V = len(xadj) - 1
    prob, alias, valid = O.alias_build(xadj, wgt)
    starts = np.concatenate([O.gen_starts(200, V, 42), np.asarray([V - 3, V - 2, V - 1], np.uint32)])
    out = dict(xadj=xadj, adjncy=adj, adjwgt=wgt, prob=prob, alias=alias, valid=valid, starts=starts)
    table = (prob, alias, valid)
    for name, kw in (("deepwalk", dict(app=O.DEEPWALK)), ("ppr", dict(app=O.PPR, tp=0.15)),
                     ("node2vec", dict(app=O.NODE2VEC, p=2.0, q=0.5))):
        p, l = O.walk(xadj, adj, wgt, table, starts, 21, seed=42, walker_base=5, **kw)
        out["walk_%s_paths" % name], out["walk_%s_lengths" % name] = p, l
        p2, l2 = O.walk(xadj, adj, wgt, None, starts, 21, seed=42, walker_base=5, online=True, **kw)
        assert np.array_equal(p, p2) and np.array_equal(l, l2)
        # unbiased (uniform neighbour choice, no table, no weights)
        pu, lu = O.walk(xadj, adj, None, None, starts, 21, seed=42, walker_base=5, unbiased=True, **kw)
        out["walk_unbiased_%s_paths" % name], out["walk_unbiased_%s_lengths" % name] = pu, lu
    for flags in (0, 1):
        d, s = O.khop(xadj, adj, wgt, table, starts, [5, 3], flags=flags, seed=42, instance_base=9)
        out["khop_flags%d_data" % flags], out["khop_flags%d_lengths" % flags] = d, s
    d, s = O.khop(xadj, adj, None, None, starts, [5, 3], flags=2, seed=42, instance_base=9)
    out["khop_unbiased_data"], out["khop_unbiased_lengths"] = d, s
    np.savez_compressed(os.path.join(HERE, "small_graph.npz"), **out)
    print("wrote small_graph.npz: V=%d E=%d" % (V, len(adj)))


if __name__ == "__main__":
    main()
