"""The allocation-free entry point against the regular builder.

skw_alias_build_list_static exists for callers that cannot allocate device memory when they call
(a plug-in in a process whose framework owns all of HBM through its pool; a serving loop that
cannot take cudaMalloc's device-wide synchronisation).  Its scratch is a fixed array inside the
library, shared by all calls, so the test makes two calls in a row with lists of different
length and checks each against skw_alias_build_offline on a one-vertex graph with the same
weights, bit for bit.  This file sorts last so that a -x run has finished every other test first.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _regular(ctx, w):
    """Table of one vertex whose out-edges carry w, through the regular entry points."""
    n = len(w)
    xadj = np.asarray([0, n] + [n] * n, np.uint32)
    adj = np.arange(1, n + 1, dtype=np.uint32)
    ctx.upload(xadj, adj, w)
    ctx.alias_build_offline()
    prob, alias, valid = ctx.alias_export()
    return prob[:n], alias[:n], int(valid[0])


def _static(lib, w):
    import torch
    n = len(w)
    d_w = torch.from_numpy(w).cuda()
    d_slots = torch.full((max(n, 1), 2), 0x7FFFFFFF, dtype=torch.int32, device="cuda")
    d_valid = torch.full((1,), 9, dtype=torch.uint8, device="cuda")
    err = C.create_string_buffer(256)
    rc = lib.skw_alias_build_list_static(C.c_void_p(d_w.data_ptr()), n, C.c_void_p(d_slots.data_ptr()),
                                         C.c_void_p(d_valid.data_ptr()),
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
    slots = d_slots.cpu().numpy()
    return rc, err.value.decode(), slots[:, 0].copy().view(np.float32), slots[:, 1].copy().view(np.uint32), int(d_valid.item())


def test_static_scratch_builder_matches_regular_builder(ctx):
    import torch
    from skywalker_b200 import _capi
    lib = _capi.load()
    torch.cuda.set_device(0)
    rng = np.random.default_rng(11)
    first = rng.uniform(1, 10, 50000).astype(np.float32)      # long list: fills most of the scratch
    second = (rng.uniform(0, 1, 3001) ** 6).astype(np.float32)  # shorter: stale entries stay behind it
    for w in (first, second):
        rc, msg, prob, alias, valid = _static(lib, w)
        assert rc == 0, msg
        rprob, ralias, rvalid = _regular(ctx, w)
        assert valid == rvalid == 1
        assert np.array_equal(alias, ralias)
        assert np.array_equal(prob.view(np.uint32), rprob.view(np.uint32))
    # short lists around every internal boundary (warp, tile of 1024 threads), with zeros, denormals
    # and one dominant weight mixed in
    for n in (1, 2, 4, 31, 33, 256, 257, 1024, 1025, 4096, 4097, 16385):
        w = rng.uniform(1, 10, n).astype(np.float32)
        if n >= 4:
            w[rng.integers(0, n, n // 4)] = 0.0
            w[rng.integers(0, n)] = 1e-42               # denormal
            w[rng.integers(0, n)] = 3.0e7               # dominates the list
        w[0] = max(w[0], 1.0)
        rc, msg, prob, alias, valid = _static(lib, w)
        assert rc == 0, msg
        rprob, ralias, rvalid = _regular(ctx, w)
        assert valid == rvalid == 1, n
        assert np.array_equal(alias, ralias), n
        assert np.array_equal(prob.view(np.uint32), rprob.view(np.uint32)), n
    # output buffers that are not device memory are refused before anything is launched
    host_slots = np.zeros((8, 2), np.int32)
    d_w = torch.ones(8, device="cuda")
    d_valid = torch.zeros(1, dtype=torch.uint8, device="cuda")
    err = C.create_string_buffer(256)
    rc = lib.skw_alias_build_list_static(C.c_void_p(d_w.data_ptr()), 8, C.c_void_p(host_slots.ctypes.data),
                                         C.c_void_p(d_valid.data_ptr()), C.c_void_p(0), err, 256)
    assert rc == -1 and b"d_slots" in err.value
    # a list without usable weight: flagged, every slot marked
    rc, msg, prob, alias, valid = _static(lib, np.zeros(40, np.float32))
    assert rc == 0 and valid == 0 and (prob == -1.0).all()
    # sizes outside the scratch are refused with a message, and nothing is launched
    too_long = np.ones(131073, np.float32)
    rc, msg, *_ = _static(lib, too_long)
    assert rc == -1 and "131072" in msg
    # the largest size still works
    rc, msg, prob, alias, valid = _static(lib, np.ones(131072, np.float32))
    assert rc == 0 and valid == 1 and (prob == 1.0).all() and np.array_equal(alias, np.arange(131072, dtype=np.uint32))
