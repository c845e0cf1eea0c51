"""Galois .gr (version 1) files: the input format of the reference (include/graph.cuh:164-327).

Layout, little endian: 4 x u64 header {version = 1, sizeEdgeTy, numNode, numEdge}; numNode x u64 END
offsets (offset of the first edge past each node); numEdge x u32 destinations; 4 bytes of padding
when numEdge is odd; numEdge x u32 edge data when sizeEdgeTy == 4.
"""
import numpy as np


def write_gr(path, xadj, adjncy, edge_data=None):
    xadj = np.asarray(xadj, np.uint64)
    adjncy = np.ascontiguousarray(adjncy, np.uint32)
    V, E = len(xadj) - 1, len(adjncy)
    with open(path, "wb") as f:
        np.asarray([1, 4 if edge_data is not None else 0, V, E], np.uint64).tofile(f)
        xadj[1:].astype(np.uint64).tofile(f)
        adjncy.tofile(f)
        if edge_data is not None:
            if E & 1:
                np.zeros(1, np.uint32).tofile(f)
            np.ascontiguousarray(edge_data, np.uint32).tofile(f)


def read_gr(path):
    """Returns (xadj u32[V+1], adjncy u32[E], edge_data u32[E] or None)."""
    with open(path, "rb") as f:
        hdr = np.fromfile(f, np.uint64, 4)
        if len(hdr) != 4 or hdr[0] != 1:
            raise ValueError("%s: not a version-1 .gr file" % path)
        size_ty, V, E = int(hdr[1]), int(hdr[2]), int(hdr[3])
        ends = np.fromfile(f, np.uint64, V)
        adj = np.fromfile(f, np.uint32, E)
        if len(ends) != V or len(adj) != E:
            raise ValueError("%s: truncated" % path)
        data = None
        if size_ty == 4:
            if E & 1:
                np.fromfile(f, np.uint32, 1)
            data = np.fromfile(f, np.uint32, E)
            if len(data) != E:
                raise ValueError("%s: truncated edge data" % path)
    xadj = np.zeros(V + 1, np.uint32)
    xadj[1:] = ends.astype(np.uint32)
    return xadj, adj, data
