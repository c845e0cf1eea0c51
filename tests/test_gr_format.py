"""The Galois .gr reader of the library against the writer in skywalker_b200/gr.py."""
import numpy as np
import pytest


def test_gr_python_roundtrip(tmp_path):
    from skywalker_b200.gr import read_gr, write_gr
    xadj = np.asarray([0, 2, 2, 5], np.uint32)
    adj = np.asarray([1, 2, 0, 1, 2], np.uint32)
    w = np.asarray([3, 1, 4, 1, 5], np.uint32)
    p = str(tmp_path / "g.gr")
    write_gr(p, xadj, adj, w)
    # header + 3 offsets + 5 dst + pad + 5 data
    assert (tmp_path / "g.gr").stat().st_size == 32 + 24 + 20 + 4 + 20
    x2, a2, d2 = read_gr(p)
    assert np.array_equal(x2, xadj) and np.array_equal(a2, adj) and np.array_equal(d2, w)


@pytest.mark.gpu
def test_gr_library_reader(ctx, tmp_path, rmat12):
    from skywalker_b200.gr import write_gr
    g = rmat12
    data = np.floor(g.adjwgt).astype(np.uint32)
    p = str(tmp_path / "g.gr")
    write_gr(p, g.xadj, g.adjncy, data)
    ctx.load_gr(p, weight_mode=0)
    x, a, w = ctx.download()
    assert np.array_equal(x, g.xadj) and np.array_equal(a, g.adjncy)
    assert np.array_equal(w, data.astype(np.float32))          # uint -> float by value (graph.cuh:294-298)
    ctx.load_gr(p, weight_mode=2)                               # --dw: weight = out-degree of the source
    x, a, w = ctx.download()
    deg = np.diff(g.xadj.astype(np.int64))
    assert np.array_equal(w, np.repeat(deg, deg).astype(np.float32))
    ctx.load_gr(p, weight_mode=1)
    assert (ctx.download()[2] == 1.0).all()


@pytest.mark.gpu
def test_gr_malformed_files(ctx, tmp_path):
    from skywalker_b200.api import SkwError
    from skywalker_b200.gr import write_gr
    xadj = np.asarray([0, 2, 2, 5], np.uint32)
    adj = np.asarray([1, 2, 0, 1, 2], np.uint32)
    good = tmp_path / "good.gr"
    write_gr(str(good), xadj, adj, np.ones(5, np.uint32))
    raw = good.read_bytes()
    cases = {
        "short.gr": raw[:40],
        "badver.gr": (2).to_bytes(8, "little") + raw[8:],
        "truncdata.gr": raw[:-8],
        "badoffset.gr": raw[:32] + (9).to_bytes(8, "little") + raw[40:],
    }
    bad_dst = bytearray(raw)
    bad_dst[32 + 24:32 + 28] = (77).to_bytes(4, "little")
    cases["baddst.gr"] = bytes(bad_dst)
    for name, blob in cases.items():
        (tmp_path / name).write_bytes(blob)
        with pytest.raises(SkwError):
            ctx.load_gr(str(tmp_path / name))
    with pytest.raises(SkwError):
        ctx.load_gr(str(tmp_path / "missing.gr"))
    ctx.load_gr(str(good))      # context still usable


@pytest.mark.gpu
def test_gr_library_reader_many_pieces(ctx, tmp_path):
    """A file larger than the reader's 64 MB pieces (offsets, destinations and edge data each span
    several of them, the last piece is ragged): what comes out of the pipelined device ingest equals
    what went into the file."""
    from skywalker_b200.gr import write_gr
    ctx.generate_rmat(21, 18 << 21, graph_seed=5, weight_seed=6)
    x, a, w = ctx.download()
    assert len(a) * 4 > 2 * (64 << 20)
    data = np.floor(w * 100).astype(np.uint32)
    p = str(tmp_path / "big.gr")
    write_gr(p, x, a, data)
    ctx.load_gr(p, weight_mode=0)
    x2, a2, w2 = ctx.download()
    assert np.array_equal(x2, x) and np.array_equal(a2, a)
    assert np.array_equal(w2, data.astype(np.float32))
    V, E, md = ctx.graph_info()
    assert (V, E, md) == (len(x) - 1, len(a), int(np.diff(x.astype(np.int64)).max()))
