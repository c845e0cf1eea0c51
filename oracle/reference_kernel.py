"""ctypes front end of oracle/_ref/libskw_ref.so: the reference's OWN offline walk kernel
(wpybtw/Skywalker, OfflineWalk -> sample_kernel_static, src/offline_walk.cu:75-124, 181-230), built
from the reference sources by oracle/ref_cuda/Makefile.

TEST / MEASUREMENT INFRASTRUCTURE: used by tests/ and by the benchmark's "reference_cuda" figure
only.  Only this entry function of the reference is driven (a bounded per-thread loop); its table
constructors and online kernels contain unbounded loops and are never launched.  The reference's
random stream is cuRAND XORWOW seeded by thread id, so its walks are comparable with this project's
only statistically and in throughput, never bit for bit.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libskw_ref.so")
_LIB = None

u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def build(reference_root=None):
    """Compile the harness against the reference tree when that tree is present (by default a directory
    named `reference` beside this repository, or $SKYWALKER_REFERENCE); returns the path of the library
    or None.  A machine without the tree uses the library built earlier."""
    if reference_root is None:
        reference_root = os.environ.get("SKYWALKER_REFERENCE") or os.path.join(
            os.path.dirname(os.path.dirname(_HERE)), "reference")
    if os.path.isdir(os.path.join(reference_root, "src")):
        subprocess.check_call(["make", "-C", os.path.join(_HERE, "ref_cuda"), "-s", "REF=" + reference_root])
    return _SO if os.path.exists(_SO) else None


def available():
    return os.path.exists(_SO)


def lib():
    global _LIB
    if _LIB is None:
        L = C.CDLL(_SO)
        L.skwref_offline_walk.argtypes = [C.c_int, C.c_uint32, C.c_uint64, u32p, u32p, f32p, u32p, u8p, u32p,
                                          C.c_uint32, C.c_uint32, C.c_int, u32p, u32p, C.POINTER(C.c_double)]
        L.skwref_offline_walk.restype = C.c_int
        L.skwref_offline_sample.argtypes = [C.c_int, C.c_uint32, C.c_uint64, u32p, u32p, f32p, u32p, u8p, u32p,
                                            C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, C.c_int, u32p, u32p,
                                            C.POINTER(C.c_double), C.POINTER(C.c_ulonglong)]
        L.skwref_offline_sample.restype = C.c_int
        L.skwref_unbiased_walk.argtypes = [C.c_int, C.c_uint32, C.c_uint64, u32p, u32p, u32p, C.c_uint32, C.c_uint32,
                                           C.c_double, C.c_int, C.c_void_p, u32p, C.POINTER(C.c_double)]
        L.skwref_unbiased_walk.restype = C.c_int
        _LIB = L
    return _LIB


def offline_walk(xadj, adjncy, table, starts, hop_num, device=0, repeats=1):
    """Run the reference's static offline walk over `starts` with the given alias table
    (prob, alias, valid -- the reference's own three arrays).  Returns (paths[n, hop_num],
    lengths[n], seconds) where seconds is the best OfflineWalk() return value of `repeats` runs."""
    prob, alias, valid = table
    xadj = np.ascontiguousarray(xadj, np.uint32)
    adjncy = np.ascontiguousarray(adjncy, np.uint32)
    starts = np.ascontiguousarray(starts, np.uint32)
    n, V, E = len(starts), len(xadj) - 1, len(adjncy)
    paths = np.zeros((n, hop_num), np.uint32)
    lengths = np.zeros(n, np.uint32)
    sec = C.c_double()
    rc = lib().skwref_offline_walk(device, V, E, xadj, adjncy, np.ascontiguousarray(prob, np.float32),
                                   np.ascontiguousarray(alias, np.uint32), np.ascontiguousarray(valid, np.uint8),
                                   starts, n, hop_num, repeats, paths.reshape(-1), lengths, C.byref(sec))
    if rc:
        raise RuntimeError("reference offline walk failed with code %d (-1 argument check, -2 CUDA call, "
                           "-3 kernel)" % rc)
    return paths, lengths, sec.value


def offline_sample(xadj, adjncy, table, seeds, f1, f2, device=0, repeats=1, blocks_per_sm=0):
    """Run the reference's offline 2-hop sampler (OfflineSample -> sample_kernel, fan-outs f1 then f2)
    over `seeds` with the given alias table.  Returns (data[n, 1 + f1 + f1 * f2], sample_lengths[n, 1 + f1],
    seconds, sampled_edges): the reference's Jobs_result<NS> arrays, its own best wall time of `repeats`
    runs and its own count of sampled edges.  A vertex with fewer than f neighbours hands over all of them
    (src/offline_sample.cu:120-128); cells without a sample keep the reference's initial value.
    blocks_per_sm: the reference's --m (thread blocks per SM, 4 when 0).  The reference's kernel drops
    hop-2 jobs that it reads from its queue before they are written, so hop-2 counts can be 0 under a
    sampled vertex that has neighbours; hop 1 is complete."""
    prob, alias, valid = table
    xadj = np.ascontiguousarray(xadj, np.uint32)
    adjncy = np.ascontiguousarray(adjncy, np.uint32)
    seeds = np.ascontiguousarray(seeds, np.uint32)
    n, V, E = len(seeds), len(xadj) - 1, len(adjncy)
    data = np.zeros((n, 1 + f1 + f1 * f2), np.uint32)
    sl = np.zeros((n, 1 + f1), np.uint32)
    sec, edges = C.c_double(), C.c_ulonglong()
    rc = lib().skwref_offline_sample(device, V, E, xadj, adjncy, np.ascontiguousarray(prob, np.float32),
                                     np.ascontiguousarray(alias, np.uint32), np.ascontiguousarray(valid, np.uint8),
                                     seeds, n, f1, f2, blocks_per_sm, repeats, data.reshape(-1), sl.reshape(-1), C.byref(sec),
                                     C.byref(edges))
    if rc:
        raise RuntimeError("reference offline sample failed with code %d (-1 argument check, -2 CUDA call, "
                           "-3 kernel, -4 layout)" % rc)
    return data, sl, sec.value, edges.value


def unbiased_walk(xadj, adjncy, starts, hop_num, tp=0.0, device=0, repeats=1, want_paths=True):
    """Run the reference's unbiased walk (UnbiasedWalk -> UnbiasedWalkKernelStatic: uniform neighbour, every
    step ends the walk with probability tp) over `starts`.  Returns (paths[n, hop_num] or None, lengths[n],
    seconds) with the reference's own best wall time of `repeats` runs."""
    xadj = np.ascontiguousarray(xadj, np.uint32)
    adjncy = np.ascontiguousarray(adjncy, np.uint32)
    starts = np.ascontiguousarray(starts, np.uint32)
    n, V, E = len(starts), len(xadj) - 1, len(adjncy)
    paths = np.zeros((n, hop_num), np.uint32) if want_paths else None
    lengths = np.zeros(n, np.uint32)
    sec = C.c_double()
    rc = lib().skwref_unbiased_walk(device, V, E, xadj, adjncy, starts, n, hop_num, float(tp), repeats,
                                    paths.ctypes.data if want_paths else None, lengths, C.byref(sec))
    if rc:
        raise RuntimeError("reference unbiased walk failed with code %d (-1 argument check, -2 CUDA call, "
                           "-3 kernel)" % rc)
    return paths, lengths, sec.value
