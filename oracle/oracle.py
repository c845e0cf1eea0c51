"""ctypes front end of the CPU oracle (oracle/skw_oracle.cpp).

TEST INFRASTRUCTURE: imported by tests/, by the smoke check and by the benchmark's CPU-baseline
and reference legs only.  The shipped package never imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
u64p = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def build(force=False):
    """Compile the oracle next to its source (g++ + OpenMP)."""
    so = os.path.join(_HERE, "libskw_oracle.so")
    src = os.path.join(_HERE, "skw_oracle.cpp")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "libskw_oracle.so")
        if not os.path.exists(so):
            build()
        L = C.CDLL(so)
        L.orc_philox4x32_10.argtypes = [u32p, u32p, u32p]
        L.orc_num_threads.restype = C.c_int
        L.orc_free.argtypes = [C.c_void_p]
        L.orc_alias_build_vertex.argtypes = [C.c_uint32, f32p, f32p, u32p]
        L.orc_alias_build_vertex.restype = C.c_int
        L.orc_alias_vertex_masses.argtypes = [C.c_uint32, f32p, u64p]
        L.orc_alias_vertex_masses.restype = C.c_int
        L.orc_alias_build.argtypes = [C.c_uint32, C.c_uint32, u32p, f32p, f32p, u32p, u8p, C.c_int]
        L.orc_alias_reconstruct_maxrel.argtypes = [C.c_uint32, u32p, f32p, f32p, u32p, u8p]
        L.orc_alias_reconstruct_maxrel.restype = C.c_double
        L.orc_walk.argtypes = [u32p, u32p, f32p, f32p, u32p, u8p, C.c_int, C.c_int, C.c_int, C.c_uint32,
                               C.c_float, C.c_float, C.c_float, C.c_uint64, C.c_uint64, C.c_uint64, u32p,
                               C.c_uint64, u32p, u32p, C.c_int]
        L.orc_khop.argtypes = [u32p, u32p, f32p, f32p, u32p, u8p, C.c_int, C.c_uint32, u32p,
                               C.c_uint32, C.c_uint64, C.c_uint64, C.c_uint64, u32p, C.c_uint64, u32p, u32p,
                               C.c_int]
        L.orc_gen_rmat.argtypes = [C.c_uint32, C.c_uint32, C.c_uint64, C.c_double, C.c_double, C.c_double,
                                   C.c_int, C.c_uint64, C.POINTER(C.c_uint32),
                                   C.POINTER(C.c_uint64), C.POINTER(C.c_void_p),
                                   C.POINTER(C.c_void_p)]
        L.orc_gen_rmat.restype = C.c_int
        L.orc_powerlaw_targets.argtypes = [C.c_uint32, C.c_double, C.c_double, C.c_uint32,
                                           C.c_uint64, u64p]
        L.orc_gen_powerlaw.argtypes = [C.c_uint32, C.c_uint64, C.c_double, C.c_double, C.c_uint32,
                                       C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_void_p),
                                       C.POINTER(C.c_void_p)]
        L.orc_gen_powerlaw.restype = C.c_int
        L.orc_gen_weights.argtypes = [C.c_uint64, C.c_uint64, f32p]
        L.orc_gen_starts.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, u32p]
        _LIB = L
    return _LIB


def num_threads():
    return int(lib().orc_num_threads())


def philox(ctr, key):
    out = np.zeros(4, np.uint32)
    lib().orc_philox4x32_10(np.asarray(ctr, np.uint32), np.asarray(key, np.uint32), out)
    return out


def _take(ptr, n, dtype):
    """Copy a malloc'ed array into numpy and free it."""
    n = int(n)
    buf = (C.c_char * (n * np.dtype(dtype).itemsize)).from_address(ptr.value) if n else b""
    arr = np.frombuffer(buf, dtype=dtype, count=n).copy()
    lib().orc_free(ptr)
    return arr


def gen_rmat(scale, raw_edges, a=0.57, b=0.19, c=0.19, symmetric=False, seed=1, num_vertices=0):
    V, E = C.c_uint32(), C.c_uint64()
    px, pa = C.c_void_p(), C.c_void_p()
    rc = lib().orc_gen_rmat(scale, num_vertices, raw_edges, a, b, c, int(symmetric), seed, C.byref(V),
                            C.byref(E), C.byref(px), C.byref(pa))
    if rc:
        raise ValueError("orc_gen_rmat failed")
    xadj = _take(px, V.value + 1, np.uint32)
    adj = _take(pa, max(E.value, 1), np.uint32)[: E.value]
    return xadj, adj


def powerlaw_targets(V, exponent, dmin, cap, seed):
    cum = np.zeros(V + 1, np.uint64)
    lib().orc_powerlaw_targets(V, exponent, dmin, cap, seed, cum)
    return cum


def gen_powerlaw(V, raw_edges, exponent=2.1, dmin=8.0, cap=33000, seed=1):
    E = C.c_uint64()
    px, pa = C.c_void_p(), C.c_void_p()
    rc = lib().orc_gen_powerlaw(V, raw_edges, exponent, dmin, cap, seed, C.byref(E),
                                C.byref(px), C.byref(pa))
    if rc:
        raise ValueError("orc_gen_powerlaw failed")
    xadj = _take(px, V + 1, np.uint32)
    adj = _take(pa, max(E.value, 1), np.uint32)[: E.value]
    return xadj, adj


def gen_weights(E, seed):
    w = np.zeros(E, np.float32)
    lib().orc_gen_weights(E, seed, w)
    return w


def gen_starts(n, V, seed, id_base=0):
    s = np.zeros(n, np.uint32)
    lib().orc_gen_starts(n, id_base, V, seed, s)
    return s


def alias_vertex(w):
    w = np.ascontiguousarray(w, np.float32)
    prob = np.zeros(len(w), np.float32)
    alias = np.zeros(len(w), np.uint32)
    ok = lib().orc_alias_build_vertex(len(w), w, prob, alias)
    return prob, alias, bool(ok)


def alias_vertex_masses(w):
    w = np.ascontiguousarray(w, np.float32)
    M = np.zeros(len(w), np.uint64)
    B = lib().orc_alias_vertex_masses(len(w), w, M)
    return M, B


def alias_build(xadj, adjwgt, v_begin=0, v_end=None, threads=0):
    V = len(xadj) - 1
    v_end = V if v_end is None else v_end
    E = int(xadj[-1])
    prob = np.ones(max(E, 1), np.float32)[:E]
    alias = np.zeros(max(E, 1), np.uint32)[:E]
    valid = np.zeros(V, np.uint8)
    lib().orc_alias_build(v_begin, v_end, xadj, _nz(adjwgt, np.float32), _nz(prob, np.float32),
                          _nz(alias, np.uint32), valid, threads)
    return prob, alias, valid


def _nz(a, dtype):
    """ctypes ndpointer rejects size-0 arrays' null data pointers on some numpy builds."""
    a = np.ascontiguousarray(a, dtype)
    return a if a.size else np.zeros(1, dtype)


def alias_reconstruct_maxrel(xadj, adjwgt, prob, alias, valid):
    return float(lib().orc_alias_reconstruct_maxrel(len(xadj) - 1, xadj, _nz(adjwgt, np.float32),
                                                    _nz(prob, np.float32), _nz(alias, np.uint32),
                                                    valid))


DEEPWALK, PPR, NODE2VEC = 0, 1, 2


def walk(xadj, adjncy, adjwgt, table, starts, hop_num, app=DEEPWALK, online=False, tp=0.0,
         p=2.0, q=0.5, seed=42, walker_base=0, threads=0, fill=0xFFFFFFFF, walker_stride=1, unbiased=False):
    """table = (prob, alias, valid) or None for online.  Returns (paths[n, hop_num], lengths[n]);
    cells after the walk's end keep `fill`."""
    n = len(starts)
    E, V = int(xadj[-1]), len(xadj) - 1
    if table is None:
        prob, alias, valid = np.ones(1, np.float32), np.zeros(1, np.uint32), np.ones(V, np.uint8)
    else:
        prob, alias, valid = table
    paths = np.full((n, hop_num), fill, np.uint32)
    lengths = np.zeros(n, np.uint32)
    lib().orc_walk(xadj, _nz(adjncy, np.uint32), _nz(adjwgt, np.float32), _nz(prob, np.float32),
                   _nz(alias, np.uint32), valid, int(online), int(unbiased), app, hop_num, tp, p, q, seed,
                   walker_base, walker_stride, _nz(starts, np.uint32), n, paths.reshape(-1) if n else np.zeros(1, np.uint32),
                   _nz(lengths, np.uint32) if n else np.zeros(1, np.uint32), threads)
    return paths, lengths


def khop_layout(fanout):
    cells, w, offs = 0, 1, []
    for h in range(len(fanout) + 1):
        if h:
            w *= fanout[h - 1]
        offs.append(cells)
        cells += w
    return cells, offs[len(fanout)], offs


def khop(xadj, adjncy, adjwgt, table, seeds, fanout, online=False, flags=0, seed=42,
         instance_base=0, threads=0, instance_stride=1):
    n = len(seeds)
    V = len(xadj) - 1
    if table is None:
        prob, alias, valid = np.ones(1, np.float32), np.zeros(1, np.uint32), np.ones(V, np.uint8)
    else:
        prob, alias, valid = table
    cells, lens, _ = khop_layout(fanout)
    data = np.zeros((max(n, 1), cells), np.uint32)
    sl = np.zeros((max(n, 1), lens), np.uint32)
    lib().orc_khop(xadj, _nz(adjncy, np.uint32), _nz(adjwgt, np.float32), _nz(prob, np.float32),
                   _nz(alias, np.uint32), valid, int(online), len(fanout),
                   np.asarray(fanout, np.uint32), flags, seed, instance_base, instance_stride,
                   _nz(seeds, np.uint32), n, data.reshape(-1), sl.reshape(-1), threads)
    return data[:n], sl[:n]
