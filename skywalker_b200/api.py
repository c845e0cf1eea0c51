"""Host-side mirror of the reference's operator interface, on top of the C ABI.

The reference drives its kernels through owner objects and free functions that return the kernel
time in seconds (declarations: include/sampler.cuh:510-529 of the reference):

    Graph, gpu_graph            -> Graph (host CSR) / Context.upload
    Sampler, Walker             -> Sampler, Walker
    ConstructTable(sampler)     -> ConstructTable(sampler)
    OfflineWalk(walker)         -> OfflineWalk(walker)
    OnlineWalkShMem(walker)     -> OnlineWalkShMem(walker)
    OfflineSample(sampler)      -> OfflineSample(sampler)
    OnlineGBSampleNew(sampler)  -> OnlineGBSampleNew(sampler)

Buffers may be numpy arrays (host entry points; copies happen inside the call) or anything with a
`data_ptr()` method such as a CUDA torch tensor (device entry points; no copies).
"""
import ctypes as C

import numpy as np

from . import _capi
from ._capi import (APP_DEEPWALK, APP_NODE2VEC, APP_PPR, INVALID_VERTEX, KHOP_TAKE_ALL,
                    MODE_OFFLINE, MODE_ONLINE, WALK_CACHE_TABLES, WALK_UNBIASED, KHOP_UNBIASED, KHOP_DISTINCT, KhopParams,
                    WalkParams)


class SkwError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("skywalker_b200 error %d: %s" % (code, msg))
        self.code = code


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        if not x.flags["C_CONTIGUOUS"]:
            raise ValueError("array must be C-contiguous")
        return C.c_void_p(x.ctypes.data)
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    return C.c_void_p(int(x))


def _is_device(x):
    return hasattr(x, "data_ptr") and getattr(x, "is_cuda", False)


class DeviceArray:
    """A borrowed 1-D device array, exported through __cuda_array_interface__ (version 2) so that
    torch / cupy / numba can wrap it without a copy: torch.as_tensor(arr, device="cuda")."""

    def __init__(self, ptr, n, typestr, owner=None):
        self.ptr, self.n, self.owner = int(ptr or 0), int(n), owner
        self.__cuda_array_interface__ = {"shape": (self.n,), "typestr": typestr, "data": (self.ptr, False),
                                         "version": 2, "strides": None}


class Context:
    """One GPU.  Owns the resident graph and alias table (reference: gpu_graph + Sampler state)."""

    def __init__(self, device=0):
        self._lib = _capi.load()
        h = C.c_void_p()
        rc = self._lib.skw_ctx_create(device, C.byref(h))
        if rc:
            raise SkwError(rc, self._lib.skw_last_global_error().decode())
        self._h = h
        self.device = device

    def close(self):
        if getattr(self, "_h", None):
            self._lib.skw_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc):
        if rc:
            raise SkwError(rc, self._lib.skw_last_error(self._h).decode())

    # -- plumbing
    def set_stream(self, cuda_stream):
        self._ck(self._lib.skw_ctx_set_stream(self._h, C.c_void_p(cuda_stream or 0)))

    def synchronize(self):
        self._ck(self._lib.skw_ctx_synchronize(self._h))

    @property
    def kernel_launches(self):
        return int(self._lib.skw_ctx_kernel_launches(self._h))

    # -- graph
    def upload(self, xadj, adjncy, adjwgt=None):
        xadj = np.ascontiguousarray(xadj, np.uint32)
        adjncy = np.ascontiguousarray(adjncy, np.uint32)
        if adjwgt is not None:
            adjwgt = np.ascontiguousarray(adjwgt, np.float32)
        V, E = len(xadj) - 1, len(adjncy)
        self._ck(self._lib.skw_graph_upload(self._h, V, E, _ptr(xadj), _ptr(adjncy) if E else _ptr(np.zeros(1, np.uint32)),
                                            _ptr(adjwgt) if adjwgt is not None and E else None))

    def adopt_device(self, V, E, d_xadj, d_adjncy, d_adjwgt=None):
        self._ck(self._lib.skw_graph_adopt_device(self._h, V, E, _ptr(d_xadj), _ptr(d_adjncy), _ptr(d_adjwgt)))

    def load_gr(self, path, weight_mode=0, weightrange=2, weight_seed=0):
        self._ck(self._lib.skw_graph_load_gr(self._h, path.encode(), weight_mode, weightrange, weight_seed))

    def generate_rmat(self, scale, raw_edges, a=0.57, b=0.19, c=0.19, symmetric=False, graph_seed=1, weight_seed=7,
                      num_vertices=0):
        self._ck(self._lib.skw_graph_generate_rmat(self._h, scale, num_vertices, raw_edges, a, b, c, int(symmetric),
                                                   graph_seed, weight_seed))

    def generate_powerlaw(self, V, raw_edges, exponent=2.1, dmin=8.0, cap=33000, graph_seed=1, weight_seed=7):
        self._ck(self._lib.skw_graph_generate_powerlaw(self._h, V, raw_edges, exponent, dmin, cap,
                                                       graph_seed, weight_seed))

    def graph_info(self):
        V, E, md = C.c_uint32(), C.c_uint64(), C.c_uint32()
        self._ck(self._lib.skw_graph_info(self._h, C.byref(V), C.byref(E), C.byref(md)))
        return V.value, E.value, md.value

    def download(self, weights=True):
        V, E, _ = self.graph_info()
        xadj = np.zeros(V + 1, np.uint32)
        adjncy = np.zeros(max(E, 1), np.uint32)
        w = np.zeros(max(E, 1), np.float32) if weights else None
        self._ck(self._lib.skw_graph_download(self._h, _ptr(xadj), _ptr(adjncy), _ptr(w)))
        return xadj, adjncy[:E], (w[:E] if weights else None)

    def graph_device_ptrs(self):
        a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
        self._ck(self._lib.skw_graph_device_ptrs(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    def free_weights(self):
        self._ck(self._lib.skw_graph_free_weights(self._h))

    def generate_starts(self, n, seed, d_out, id_base=0):
        self._ck(self._lib.skw_generate_starts_device(self._h, n, id_base, seed, _ptr(d_out)))

    # -- alias table
    def alias_build_offline(self, v_begin=0, v_end=None):
        """Returns the build kernels' time in milliseconds."""
        if v_end is None:
            v_end = self.graph_info()[0]
        ms = C.c_float()
        self._ck(self._lib.skw_alias_build_offline(self._h, v_begin, v_end, C.byref(ms)))
        return ms.value

    def alias_export(self):
        V, E, _ = self.graph_info()
        prob = np.zeros(max(E, 1), np.float32)
        alias = np.zeros(max(E, 1), np.uint32)
        valid = np.zeros(max(V, 1), np.uint8)
        self._ck(self._lib.skw_alias_export(self._h, _ptr(prob), _ptr(alias), _ptr(valid)))
        return prob[:E], alias[:E], valid[:V]

    def alias_import(self, prob, alias, valid):
        prob = np.ascontiguousarray(prob, np.float32)
        alias = np.ascontiguousarray(alias, np.uint32)
        valid = np.ascontiguousarray(valid, np.uint8)
        pad = lambda a: a if a.size else np.zeros(1, a.dtype)
        self._ck(self._lib.skw_alias_import(self._h, _ptr(pad(prob)), _ptr(pad(alias)), _ptr(pad(valid))))

    def alias_save(self, path):
        self._ck(self._lib.skw_alias_save(self._h, path.encode()))

    def alias_load(self, path):
        self._ck(self._lib.skw_alias_load(self._h, path.encode()))

    SLOT_SLACK = 1024   # spare slots allocated past E (see skw_alias_device_ptrs)

    def alias_device_arrays(self, padded=False):
        """(slots as int64[E] -- one packed {f32 prob, u32 alias} per element --, valid as uint8[V]),
        borrowed from the context: for collectives over table slices (multi-GPU sliced build).
        padded=True exposes the E + SLOT_SLACK allocated slots (in-place equal-chunk all-gather)."""
        V, E, _ = self.graph_info()
        a, b = C.c_void_p(), C.c_void_p()
        self._ck(self._lib.skw_alias_device_ptrs(self._h, C.byref(a), C.byref(b)))
        return (DeviceArray(a.value, E + (self.SLOT_SLACK if padded else 0), "<i8", self),
                DeviceArray(b.value, V, "|u1", self))

    def download_xadj(self):
        V, _, _ = self.graph_info()
        xadj = np.zeros(V + 1, np.uint32)
        self._ck(self._lib.skw_graph_download(self._h, _ptr(xadj), None, None))
        return xadj

    def walk_records_build(self):
        """Build the fused 32-byte walk records from the alias table; returns milliseconds."""
        ms = C.c_float()
        self._ck(self._lib.skw_walk_records_build(self._h, C.byref(ms)))
        return ms.value

    def walk_records_free(self):
        self._ck(self._lib.skw_walk_records_free(self._h))

    def probe_random_gather(self, footprint_bytes=16 << 30, iters=128):
        """Giga random 32-byte accesses per second this GPU sustains (dependent chains, like a walk)."""
        v = C.c_double()
        self._ck(self._lib.skw_probe_random_gather(self._h, footprint_bytes, iters, C.byref(v)))
        return v.value

    # -- walks
    def walk(self, starts, hop_num, app=APP_DEEPWALK, mode=MODE_OFFLINE, tp=0.0, p=2.0, q=0.5, seed=42,
             walker_base=0, paths=None, lengths=None, n=None, walker_stride=1, enqueue_only=False, flags=0):
        """Host arrays (numpy) or device buffers.  Returns (paths, lengths, ms, sampled_edges).
        enqueue_only (device buffers only): queue the kernels and return at once with ms = edges = None;
        collect the edge count later with take_sampled_edges()."""
        prm = WalkParams(app, mode, hop_num, tp, p, q, seed, walker_base, walker_stride, flags)
        ms, edges = C.c_float(), C.c_uint64()
        if _is_device(starts):
            n = int(starts.numel()) if n is None else n
            fn = self._lib.skw_walk_device
        else:
            starts = np.ascontiguousarray(starts, np.uint32)
            n = len(starts) if n is None else n
            if paths is None:
                paths = np.full((n, hop_num), INVALID_VERTEX, np.uint32)
            if lengths is None:
                lengths = np.zeros(n, np.uint32)
            fn = self._lib.skw_walk
        if enqueue_only:
            if fn is not self._lib.skw_walk_device:
                raise ValueError("enqueue_only needs device buffers")
            self._ck(fn(self._h, C.byref(prm), _ptr(starts) if n else None, n, _ptr(paths) if n else None,
                        _ptr(lengths) if n else None, None, None))
            return paths, lengths, None, None
        self._ck(fn(self._h, C.byref(prm), _ptr(starts) if n else None, n, _ptr(paths) if n else None,
                    _ptr(lengths) if n else None, C.byref(ms), C.byref(edges)))
        return paths, lengths, ms.value, edges.value

    def walk_packed(self, starts, hop_num, app=APP_DEEPWALK, mode=MODE_OFFLINE, tp=0.0, p=2.0, q=0.5, seed=42,
                    walker_base=0, packed=None, lengths=None, n=None, walker_stride=1, flags=0, lengths_u8=False):
        """Host arrays in, packed result out: returns (packed, lengths, cells, ms, sampled_edges) with the
        walks back to back in packed[:cells] (walk w holds lengths[w] + 1 vertices).  `packed` may be a
        numpy array or a pinned buffer; without one a buffer of n * hop_num cells is allocated.
        lengths_u8: the lengths come back as bytes (skw_walk_packed_u8; hop_num <= 256)."""
        prm = WalkParams(app, mode, hop_num, tp, p, q, seed, walker_base, walker_stride, flags)
        starts = starts if _is_device(starts) else np.ascontiguousarray(starts, np.uint32)
        n = (int(starts.numel()) if _is_device(starts) else len(starts)) if n is None else n
        if packed is None:
            packed = np.empty(max(n * hop_num, 1), np.uint32)
        if lengths is None:
            lengths = np.zeros(max(n, 1), np.uint8 if lengths_u8 else np.uint32)[:n]
        cap = int(packed.numel()) if hasattr(packed, "numel") else int(packed.size)
        ms, edges, cells = C.c_float(), C.c_uint64(), C.c_uint64()
        fn = self._lib.skw_walk_packed_u8 if lengths_u8 else self._lib.skw_walk_packed
        self._ck(fn(self._h, C.byref(prm), _ptr(starts) if n else None, n, _ptr(packed), cap,
                    _ptr(lengths) if n else None, C.byref(cells), C.byref(ms), C.byref(edges)))
        return packed, lengths, cells.value, ms.value, edges.value

    def take_sampled_edges(self):
        """Wait for enqueued walks, raise on a device error of any of them, return their edge count."""
        v = C.c_uint64()
        self._ck(self._lib.skw_ctx_take_sampled_edges(self._h, C.byref(v)))
        return v.value

    # -- k-hop
    @staticmethod
    def khop_layout(fanout):
        if not 1 <= len(fanout) <= 4:
            raise SkwError(-1, "k-hop sampling takes 1 to 4 hops, got %d" % len(fanout))
        prm = KhopParams(0, len(fanout), (C.c_uint32 * 4)(*(list(fanout) + [0] * (4 - len(fanout)))), 0, 0, 0, 1)
        cells, lens = C.c_uint32(), C.c_uint32()
        rc = _capi.load().skw_khop_layout(C.byref(prm), C.byref(cells), C.byref(lens))
        if rc:
            raise SkwError(rc, "bad fan-out list %r" % (list(fanout),))
        return cells.value, lens.value

    def sample_khop(self, seeds, fanout, mode=MODE_OFFLINE, flags=0, seed=42, instance_base=0, data=None,
                    sample_lengths=None, n=None, instance_stride=1):
        """Returns (data[n, cells], sample_lengths[n, lens], ms, sampled_edges)."""
        cells, lens = self.khop_layout(fanout)
        prm = KhopParams(mode, len(fanout), (C.c_uint32 * 4)(*(list(fanout) + [0] * (4 - len(fanout)))),
                         flags, seed, instance_base, instance_stride)
        ms, edges = C.c_float(), C.c_uint64()
        if _is_device(seeds):
            n = int(seeds.numel()) if n is None else n
            fn = self._lib.skw_sample_khop_device
        else:
            seeds = np.ascontiguousarray(seeds, np.uint32)
            n = len(seeds) if n is None else n
            if data is None:
                data = np.zeros((n, cells), np.uint32)
            if sample_lengths is None:
                sample_lengths = np.zeros((n, lens), np.uint32)
            fn = self._lib.skw_sample_khop
        self._ck(fn(self._h, C.byref(prm), _ptr(seeds) if n else None, n, _ptr(data) if n else None,
                    _ptr(sample_lengths) if n else None, C.byref(ms), C.byref(edges)))
        return data, sample_lengths, ms.value, edges.value

    def sample_khop_packed(self, seeds, fanout, mode=MODE_OFFLINE, flags=0, seed=42, instance_base=0, packed=None,
                           sample_lengths=None, n=None, instance_stride=1):
        """Host arrays in, packed tree out: returns (packed, sample_lengths[n, lens], cells, ms, sampled_edges);
        packed[:cells] holds, seed after seed, the cells of the dense tree that are not INVALID_VERTEX."""
        cells_per, lens = self.khop_layout(fanout)
        prm = KhopParams(mode, len(fanout), (C.c_uint32 * 4)(*(list(fanout) + [0] * (4 - len(fanout)))),
                         flags, seed, instance_base, instance_stride)
        seeds = np.ascontiguousarray(seeds, np.uint32)
        n = len(seeds) if n is None else n
        if packed is None:
            packed = np.empty(max(n * cells_per, 1), np.uint32)
        if sample_lengths is None:
            sample_lengths = np.zeros((n, lens), np.uint32)
        cap = int(packed.numel()) if hasattr(packed, "numel") else int(packed.size)
        ms, edges, cells = C.c_float(), C.c_uint64(), C.c_uint64()
        self._ck(self._lib.skw_sample_khop_packed(self._h, C.byref(prm), _ptr(seeds) if n else None, n, _ptr(packed),
                                                  cap, _ptr(sample_lengths) if n else None, C.byref(cells),
                                                  C.byref(ms), C.byref(edges)))
        return packed, sample_lengths, cells.value, ms.value, edges.value


# ---------------------------------------------------------------------------------------------
# Reference-shaped surface (names and return values of include/sampler.cuh:510-529).

class Graph:
    """Host CSR graph (reference: class Graph, include/graph.cuh:47-328)."""

    def __init__(self, xadj, adjncy, adjwgt=None):
        self.xadj = np.ascontiguousarray(xadj, np.uint32)
        self.adjncy = np.ascontiguousarray(adjncy, np.uint32)
        self.adjwgt = None if adjwgt is None else np.ascontiguousarray(adjwgt, np.float32)
        self.numNode = len(self.xadj) - 1
        self.numEdge = len(self.adjncy)
        deg = np.diff(self.xadj.astype(np.int64))
        self.MaxDegree = int(deg.max()) if len(deg) else 0


class Sampler:
    """Owner of the device graph, the alias table and a k-hop job (reference: Sampler / Sampler_new,
    include/sampler.cuh:30-400)."""

    def __init__(self, graph, device=0, ctx=None):
        self.ctx = ctx or Context(device)
        self.graph = graph
        if graph is not None:
            self.ctx.upload(graph.xadj, graph.adjncy, graph.adjwgt)
        self.sampled_edges = 0
        self.seeds = None
        self.hops = None
        self.result = None
        self.seed = 42
        self.flags = KHOP_TAKE_ALL

    def SetSeed(self, seeds, hops, dev_num=1, dev_id=0):
        """hops = [1, f1, f2, ...] as in the reference (src/main.cu:193-202)."""
        self.seeds = np.ascontiguousarray(seeds, np.uint32)
        self.hops = list(hops)
        self.instance_base = 0


class Walker:
    """Owner of a batch of walks (reference: Walker, include/sampler.cuh:402-508)."""

    def __init__(self, sampler):
        self.sampler = sampler
        self.ctx = sampler.ctx
        self.sampled_edges = 0
        self.app = APP_DEEPWALK
        self.tp, self.p, self.q = 0.0, 2.0, 0.5
        self.seed = 42
        self.walker_base = 0

    def SetSeed(self, starts, hop_num, dev_num=1, dev_id=0):
        self.starts = np.ascontiguousarray(starts, np.uint32)
        self.num_seed = len(self.starts)
        self.hop_num = hop_num
        self.result = None


class _WalkResult:
    def __init__(self, data, length):
        self.data, self.length = data, length


class _SampleResult:
    def __init__(self, data, sample_lengths):
        self.data, self.sample_lengths = data, sample_lengths


def edge_balanced_ranges(xadj, parts):
    """Vertex ranges holding ~E/parts edges each, as the reference cuts the table build between GPUs
    (--edgecut, include/sampler.cuh:151-158): part r starts at the first vertex whose first edge is
    at or after r * E / parts."""
    E = int(xadj[-1])
    V = len(xadj) - 1
    cuts = [int(np.searchsorted(xadj[:V], E // parts * r, side="left")) for r in range(parts)] + [V]
    cuts[0] = 0
    return [(cuts[r], cuts[r + 1]) for r in range(parts)]


def edge_chunk_ranges(xadj, parts):
    """For an in-place all-gather of the table in equal chunks of S = ceil(E / parts) slots: part r owns
    slots [r*S, (r+1)*S) and must build every vertex that overlaps them, so a vertex straddling a chunk
    boundary is built by both neighbours (same bits either way).  Returns (S, [(v_begin, v_end), ...]);
    the ranges cover every vertex, also those without edges."""
    E = int(xadj[-1])
    V = len(xadj) - 1
    S = max(1, -(-E // parts))
    out = []
    for r in range(parts):
        lo, hi = min(r * S, E), min((r + 1) * S, E)
        if hi > lo:
            vb = int(np.searchsorted(xadj, lo, side="right")) - 1
            ve = int(np.searchsorted(xadj, hi - 1, side="right"))
        else:
            vb = ve = V
        out.append([vb, ve])
    out[0][0] = 0
    out[-1][1] = V
    for r in range(parts - 1):     # vertices without edges between two chunks go to the earlier part
        out[r][1] = max(out[r][1], min(out[r + 1][0], V))
        if out[r][0] > out[r][1]:
            out[r][0] = out[r][1]
    return S, [tuple(x) for x in out]


def ConstructTable(sampler, ngpu=1, index=0):
    """Build the alias table; returns seconds (src/createTable.cu:119-179).  With ngpu > 1 builds the
    edge-balanced slice `index` only; the caller assembles the slices (NCCL all-gather of
    Context.alias_device_arrays() segments, replacing AliasTable::Assemble, include/gpu_graph.cuh:282-291)."""
    if ngpu <= 1:
        return sampler.ctx.alias_build_offline() * 1e-3
    vb, ve = edge_balanced_ranges(sampler.ctx.download_xadj(), ngpu)[index]
    return sampler.ctx.alias_build_offline(vb, ve) * 1e-3


def _walk(walker, mode, flags=0):
    paths, lengths, ms, edges = walker.ctx.walk(walker.starts, walker.hop_num, app=walker.app, mode=mode,
                                                tp=walker.tp, p=walker.p, q=walker.q, seed=walker.seed,
                                                walker_base=walker.walker_base, flags=flags)
    walker.result = _WalkResult(paths, lengths)
    walker.sampled_edges = edges
    return ms * 1e-3


def OfflineWalk(walker):
    """src/offline_walk.cu:181-230."""
    return _walk(walker, MODE_OFFLINE)


def OnlineWalkShMem(walker):
    """src/online_walk.cu:245-327."""
    return _walk(walker, MODE_ONLINE)


OnlineWalkGMem = OnlineWalkShMem  # same result; the reference differs only in scratch placement


def UnbiasedWalk(walker):
    """Uniform neighbour choice, no table (src/unbiased_walk.cu:194-247)."""
    return _walk(walker, MODE_OFFLINE, WALK_UNBIASED)


def _sample(sampler, mode, flags=0):
    data, lens, ms, edges = sampler.ctx.sample_khop(sampler.seeds, sampler.hops[1:], mode=mode,
                                                    flags=sampler.flags | flags,
                                                    seed=sampler.seed, instance_base=sampler.instance_base)
    sampler.result = _SampleResult(data, lens)
    sampler.sampled_edges = edges
    return ms * 1e-3


def OfflineSample(sampler):
    """src/offline_sample.cu:443-513."""
    return _sample(sampler, MODE_OFFLINE)


def OnlineGBSampleNew(sampler, with_replacement=False):
    """src/online_sample_new.cu:459-547.  The reference's online sampler keeps only draws of columns it
    has not drawn before (roll_atomic, src/online_sample_new.cu:73-111): KHOP_DISTINCT.
    with_replacement=True gives independent draws instead (sampler.flags then apply as they are)."""
    return _sample(sampler, MODE_ONLINE, 0 if with_replacement else KHOP_DISTINCT)


def UnbiasedSample(sampler):
    """Uniform draws with replacement, no table (src/unbiased_sample.cu:322-384)."""
    return _sample(sampler, MODE_OFFLINE, KHOP_UNBIASED)
