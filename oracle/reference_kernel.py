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
