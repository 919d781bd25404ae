"""The allocation-free batched copy, called through its exported C symbol.

Some callers of this library cannot allocate device memory (a plug-in inside another
framework's fixed memory plan, a serving loop where an allocation could stall the device).
For them `b200ep_batched_copy_noalloc` keeps its descriptor table in a fixed array inside the
library image. This test calls it twice in a row and checks both results against the regular
entry point (`CopyEngine` in kernel mode, whose table comes from cudaMalloc); copies are exact,
so the comparison is bit for bit, like the other copy tests. It lives in its own file, collected
last, so a failure here cannot hide the other tests' results.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from gpu_data_transfer_profile_b200 import _ext
    _ext.load()
    lib = ctypes.CDLL(_ext.loaded_path())
    fn = lib.b200ep_batched_copy_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                   ctypes.POINTER(ctypes.c_longlong), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.b200ep_noalloc_error_string.restype = ctypes.c_char_p
    lib.b200ep_noalloc_error_string.argtypes = [ctypes.c_int]
    return lib, fn


def _call(fn, dsts, srcs, sizes, ctas=4, threads=256):
    n = len(sizes)
    d = (ctypes.c_void_p * n)(*dsts)
    s = (ctypes.c_void_p * n)(*srcs)
    z = (ctypes.c_longlong * n)(*sizes)
    return fn(d, s, z, n, ctas, threads, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _pattern(n, seed):
    i = torch.arange(n, device="cuda", dtype=torch.int64)
    return ((i * 131 + seed * 7919 + (i >> 11) * 17) % 251).to(torch.uint8)


def test_no_alloc_batched_copy_matches_regular_entry_point_twice():
    from gpu_data_transfer_profile_b200.ops.copy import CopyEngine
    lib, fn = _lib()
    for call, sizes in enumerate([[4096, 65536, 100001, 16, 7], [300000, 48, 8192]]):
        gap = 64
        total = sum(sizes) + gap * len(sizes)
        src = _pattern(total, seed=call + 1)
        got = torch.full((total,), 253, dtype=torch.uint8, device="cuda")
        want = torch.full((total,), 253, dtype=torch.uint8, device="cuda")
        offs, o = [], 0
        for s in sizes:
            offs.append(o)
            o += s + gap
        eng = CopyEngine([(want.data_ptr() + o, 0, src.data_ptr() + o, 0, s) for o, s in zip(offs, sizes)],
                         "kernel", stream_device=0, use_proxy=False)
        eng.run(1)
        rc = _call(fn, [got.data_ptr() + o for o in offs], [src.data_ptr() + o for o in offs], sizes)
        assert rc == 0, lib.b200ep_noalloc_error_string(rc)
        torch.cuda.synchronize()
        assert torch.equal(got, want)            # copied ranges equal, gaps untouched
        for o, s in zip(offs, sizes):
            assert torch.equal(got[o:o + s], src[o:o + s])


def test_no_alloc_batched_copy_accepts_the_full_table():
    """Exactly 1024 copies (the limit) of 48 bytes each, with 16-byte gaps that must stay untouched."""
    lib, fn = _lib()
    n, size, pitch = 1024, 48, 64
    src = _pattern(n * pitch, seed=9)
    got = torch.full((n * pitch,), 253, dtype=torch.uint8, device="cuda")
    rc = _call(fn, [got.data_ptr() + i * pitch for i in range(n)],
               [src.data_ptr() + i * pitch for i in range(n)], [size] * n, ctas=1, threads=64)
    assert rc == 0, lib.b200ep_noalloc_error_string(rc)
    torch.cuda.synchronize()
    g2, s2 = got.view(n, pitch), src.view(n, pitch)
    assert torch.equal(g2[:, :size], s2[:, :size])
    assert bool((g2[:, size:] == 253).all())


def test_no_alloc_batched_copy_refuses_a_capturing_stream():
    """The descriptors are uploaded from the callee's stack, so a captured call would replay
    garbage: the entry point must refuse (-7) and issue nothing."""
    lib, fn = _lib()
    src = _pattern(256, seed=3)
    dst = torch.full((256,), 253, dtype=torch.uint8, device="cuda")
    assert _call(fn, [dst.data_ptr()], [src.data_ptr()], [256]) == 0     # first call on this device: outside capture
    torch.cuda.synchronize()
    dst.fill_(253)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        dst.add_(0)                                                       # something to capture
        rc = _call(fn, [dst.data_ptr()], [src.data_ptr()], [256])
    assert rc == -7 and b"captur" in lib.b200ep_noalloc_error_string(rc)
    graph.replay()
    torch.cuda.synchronize()
    assert bool((dst == 253).all())                                       # nothing was recorded for the copy


def test_no_alloc_batched_copy_rejects_bad_arguments():
    lib, fn = _lib()
    buf = torch.zeros(64, dtype=torch.uint8, device="cuda")
    too_many = 1025
    rc = _call(fn, [buf.data_ptr()] * too_many, [buf.data_ptr()] * too_many, [1] * too_many)
    assert rc == -3 and b"1024" in lib.b200ep_noalloc_error_string(rc)
    assert _call(fn, [buf.data_ptr()], [buf.data_ptr()], [-1]) == -5
    assert _call(fn, [buf.data_ptr()], [buf.data_ptr()], [8], ctas=0) == -4
