"""ctypes binding of libskywalker_b200.so (the C ABI declared in include/skywalker_b200.h).

There is no fallback: if the shared library is missing, importing this module raises.
"""
import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# SKYWALKER_B200_LIB points at an alternative build of the same library (e.g. a tuning variant)
LIB_PATH = os.environ.get("SKYWALKER_B200_LIB") or os.path.join(_PKG, "libskywalker_b200.so")

SKW_OK = 0
APP_DEEPWALK, APP_PPR, APP_NODE2VEC = 0, 1, 2
MODE_OFFLINE, MODE_ONLINE = 0, 1
KHOP_TAKE_ALL = 1
WALK_CACHE_TABLES = 1
WALK_UNBIASED = 2
WALK_BUILD_TABLES = 4
WALK_DIRECT_SLOTS = 8
KHOP_UNBIASED = 2
KHOP_DISTINCT = 4
INVALID_VERTEX = 0xFFFFFFFF


class WalkParams(C.Structure):
    _fields_ = [("app", C.c_uint32), ("mode", C.c_uint32), ("hop_num", C.c_uint32),
                ("tp", C.c_float), ("p", C.c_float), ("q", C.c_float),
                ("seed", C.c_uint64), ("walker_base", C.c_uint64), ("walker_stride", C.c_uint64), ("flags", C.c_uint32)]


class KhopParams(C.Structure):
    _fields_ = [("mode", C.c_uint32), ("nhops", C.c_uint32), ("fanout", C.c_uint32 * 4),
                ("flags", C.c_uint32), ("seed", C.c_uint64), ("instance_base", C.c_uint64),
                ("instance_stride", C.c_uint64)]


# name -> (restype, argtypes); every symbol include/skywalker_b200.h declares
SIGNATURES = {
    "skw_ctx_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "skw_ctx_destroy": (None, [C.c_void_p]),
    "skw_last_error": (C.c_char_p, [C.c_void_p]),
    "skw_last_global_error": (C.c_char_p, []),
    "skw_ctx_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "skw_ctx_synchronize": (C.c_int, [C.c_void_p]),
    "skw_ctx_kernel_launches": (C.c_uint64, [C.c_void_p]),
    "skw_graph_upload": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "skw_graph_adopt_device": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "skw_graph_load_gr": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int, C.c_uint32, C.c_uint64]),
    "skw_graph_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)]),
    "skw_graph_download": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "skw_graph_device_ptrs": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "skw_graph_free_weights": (C.c_int, [C.c_void_p]),
    "skw_graph_generate_rmat": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64, C.c_double, C.c_double, C.c_double,
                                          C.c_int, C.c_uint64, C.c_uint64]),
    "skw_graph_generate_powerlaw": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint64, C.c_double, C.c_double,
                                              C.c_uint32, C.c_uint64, C.c_uint64]),
    "skw_generate_starts_device": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p]),
    "skw_alias_build_offline": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(C.c_float)]),
    "skw_alias_export": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "skw_alias_import": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "skw_alias_save": (C.c_int, [C.c_void_p, C.c_char_p]),
    "skw_alias_load": (C.c_int, [C.c_void_p, C.c_char_p]),
    "skw_alias_device_ptrs": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "skw_alias_build_list_static": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_char_p, C.c_size_t]),
    "skw_ctx_take_sampled_edges": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "skw_walk_records_build": (C.c_int, [C.c_void_p, C.POINTER(C.c_float)]),
    "skw_walk_records_free": (C.c_int, [C.c_void_p]),
    "skw_walk_device": (C.c_int, [C.c_void_p, C.POINTER(WalkParams), C.c_void_p, C.c_uint64, C.c_void_p,
                                  C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_uint64)]),
    "skw_walk": (C.c_int, [C.c_void_p, C.POINTER(WalkParams), C.c_void_p, C.c_uint64, C.c_void_p,
                           C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_uint64)]),
    "skw_walk_packed": (C.c_int, [C.c_void_p, C.POINTER(WalkParams), C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64,
                                  C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_float), C.POINTER(C.c_uint64)]),
    "skw_walk_packed_u8": (C.c_int, [C.c_void_p, C.POINTER(WalkParams), C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64,
                                     C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_float), C.POINTER(C.c_uint64)]),
    "skw_khop_layout": (C.c_int, [C.POINTER(KhopParams), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "skw_sample_khop_device": (C.c_int, [C.c_void_p, C.POINTER(KhopParams), C.c_void_p, C.c_uint64, C.c_void_p,
                                         C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_uint64)]),
    "skw_sample_khop": (C.c_int, [C.c_void_p, C.POINTER(KhopParams), C.c_void_p, C.c_uint64, C.c_void_p,
                                  C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_uint64)]),
    "skw_sample_khop_packed": (C.c_int, [C.c_void_p, C.POINTER(KhopParams), C.c_void_p, C.c_uint64, C.c_void_p,
                                         C.c_uint64, C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_float),
                                         C.POINTER(C.c_uint64)]),
    "skw_probe_random_gather": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint32, C.POINTER(C.c_double)]),
    "skw_selftest_bounded_wait": (C.c_int, [C.c_void_p]),
    "skw_host_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "skw_host_free": (None, [C.c_void_p]),
    "skw_version": (C.c_char_p, []),
}

_LIB = None


def load():
    """Load the shared library and bind every symbol.  Raises if it is absent or incomplete."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "%s is missing: build it with `python -m skywalker_b200.build` (needs nvcc). "
                "skywalker_b200 has no CPU or pure-Python path." % LIB_PATH)
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _LIB = lib
    return _LIB
