"""A bounded device wait that runs out, made to run out on purpose (needs a B200; faults nothing).

The library's kernels wait for other parties in three places (a peer's flag in the all-reduce, the grid
barrier of the persistent step, a kernel's own copies); every such wait has a limit, after which the kernel
raises the context's status word and returns.  Here a group of two seats lives on ONE GPU and only one seat
calls: its wait for the other seat's flag runs out after a few milliseconds, the kernel returns, and the host
reads the refusal.  The calls are issued one after the other on one stream, so no two kernels ever wait on
each other at the same time.
"""
import ctypes

import numpy as np
import pytest

import neura_b200 as nb
from neura_b200.runtime import _check

pytestmark = pytest.mark.gpu


def seats(rt, count):
    """Two communicators of this process on the runtime's GPU, connected to each other."""
    lib, ctx = rt._lib, rt._ctx
    handles = (ctypes.c_void_p * 2)()
    scratch = (ctypes.c_ubyte * 64)()
    for rank in range(2):
        comm = ctypes.c_void_p()
        _check(lib.neura_cuda_comm_create(ctx, count, ctypes.byref(comm), scratch))
        handles[rank] = comm.value
    for rank in range(2):
        _check(lib.neura_cuda_comm_connect_local(ctx, ctypes.c_void_p(handles[rank]), rank, 2, handles))
    return [ctypes.c_void_p(handles[0]), ctypes.c_void_p(handles[1])]


def test_an_all_reduce_whose_peer_never_comes_gives_up_and_the_context_stays_usable(runtime):
    rt, lib = runtime, runtime._lib
    count = 1024
    first, second = seats(rt, count)
    a, b = rt.tensor(count), rt.tensor(count)
    va = np.arange(count, dtype=np.float32)
    vb = np.full(count, 0.5, dtype=np.float32)
    rt.write(a, va)
    rt.write(b, vb)
    rt.set_wait_limit(5_000_000)   # five milliseconds
    try:
        # seat 0 calls alone: nothing ever publishes seat 1's flag
        _check(lib.neura_cuda_allreduce(rt._ctx, rt.stream, first, ctypes.c_void_p(a.ptr), count))
        with pytest.raises(nb.NeuraCudaError) as refusal:
            rt.sync()
        assert refusal.value.code == -3 and "all-reduce gave up" in str(refusal.value)
        assert np.array_equal(rt.read(a).reshape(-1), va), "a rank that gives up leaves its input untouched"
        rt.sync()   # the refusal was reported once; the context is usable again
        # seat 1 comes: it finds seat 0's numbers from the call that gave up
        _check(lib.neura_cuda_allreduce(rt._ctx, rt.stream, second, ctypes.c_void_p(b.ptr), count))
        rt.sync()
        assert np.array_equal(rt.read(b).reshape(-1), va + vb)
        # and seat 0's repeated call completes with the same sum
        _check(lib.neura_cuda_allreduce(rt._ctx, rt.stream, first, ctypes.c_void_p(a.ptr), count))
        rt.sync()
        assert np.array_equal(rt.read(a).reshape(-1), va + vb)
        # a second round, in the other slot, with both seats present from the start
        _check(lib.neura_cuda_allreduce(rt._ctx, rt.stream, second, ctypes.c_void_p(b.ptr), count))
        with pytest.raises(nb.NeuraCudaError):
            rt.sync()   # seat 1 alone gives up as well
        _check(lib.neura_cuda_allreduce(rt._ctx, rt.stream, first, ctypes.c_void_p(a.ptr), count))
        rt.sync()
        assert np.array_equal(rt.read(a).reshape(-1), 2 * (va + vb))
    finally:
        rt.set_wait_limit(2_000_000_000)
        for comm in (first, second):
            lib.neura_cuda_comm_destroy(rt._ctx, comm)
        rt.free(a.ptr)
        rt.free(b.ptr)


def test_a_wait_limit_of_zero_is_refused(runtime):
    with pytest.raises(nb.NeuraCudaError):
        runtime.set_wait_limit(0)
