"""The allocation-free table-gradient entry point, lffn_gather_bwd_tables_sorted_static.

Some callers of this library may not allocate device memory while they run: a plugin inside a host that took
all GPU memory into its own pool at start-up (cudaMalloc fails there, or is forbidden), a latency-critical loop
that must not take the allocator's lock.  They cannot provide the scratch buffer the sorted table gradient sorts
into, so the library carries a 32 MiB array of its own for them.  This test calls the entry point through the
C ABI twice in a row on different inputs and requires each result to be bit-identical to the regular entry
point's (the regular one is itself checked bit for bit against the CPU oracle in test_gpu_parity.py).  The
second call finds the first call's leftovers in the shared array, which must not matter.

"Allocates nothing" is checked with cudaMemGetInfo (free bytes of the device), not with torch's own counters,
which see only torch's caching allocator: after one warm-up call -- the first use on a device is when the CUDA
runtime loads the library's code and reserves the built-in array -- the two calls must leave the free bytes of
the device unchanged.  The file is named to be collected last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, N, T, m, rows, d, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    idx = (torch.randint(0, rows, (N, T, m), generator=g, device=dev, dtype=torch.int32)
           + (torch.arange(T, device=dev, dtype=torch.int32) * rows)[None, :, None]).reshape(N, T * m).contiguous()
    w = torch.randn(N, T * m, generator=g, device=dev)
    dy = torch.randn(N, d, generator=g, device=dev)
    return idx, w, dy


def test_static_scratch_entry_point_matches_regular_one_twice():
    from lookupffn_b200 import _lib as L

    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    lib = L.lib()
    shapes = [(3000, 24, 1, 256, 512), (700, 6, 9, 256, 768)]
    with torch.cuda.device(dev):
        sp = L.stream_ptr(dev)
        # everything the calls under test touch is allocated first; the regular entry point gives the expected bits
        cases = []
        for seed, (N, T, m, rows, d) in enumerate(shapes):
            idx, w, dy = _inputs(seed, N, T, m, rows, d, dev)
            S = T * rows
            ref = torch.empty(S, d, device=dev)
            out = torch.full((S, d), float("nan"), device=dev)
            nbytes = lib.lffn_gather_bwd_tables_sorted_scratch_bytes(N, T, m, rows)
            assert nbytes <= L.STATIC_SCRATCH_BYTES
            scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            L.check(lib.lffn_gather_bwd_tables_sorted(L.ptr(idx), L.ptr(w), L.ptr(dy), L.ptr(ref), N, T, m, rows, d,
                                                      L.ptr(scratch), nbytes, sp))
            cases.append((idx, w, dy, ref, out, (N, T, m, rows, d)))

        def call(case):
            idx, w, dy, _, out, (N, T, m, rows, d) = case
            L.check(lib.lffn_gather_bwd_tables_sorted_static(L.ptr(idx), L.ptr(w), L.ptr(dy), L.ptr(out), N, T, m,
                                                             rows, d, sp))

        call(cases[0])  # warm-up: the first use on the device loads the code and looks up the array's address
        torch.cuda.synchronize()
        cases[0][4].fill_(float("nan"))
        torch.cuda.synchronize()
        # Free bytes of the device as the driver reports them.  Another process on the same GPU could move the
        # number, so a changed reading is re-taken (up to three rounds); an allocation by the calls themselves
        # would change it every time.
        unchanged = False
        for _ in range(3):
            free_before = torch.cuda.mem_get_info(dev)[0]
            for case in cases:
                call(case)
            torch.cuda.synchronize()
            if torch.cuda.mem_get_info(dev)[0] == free_before:
                unchanged = True
                break
        assert unchanged, "free device memory changed across the allocation-free calls"
        for i, (_, _, _, ref, out, _) in enumerate(cases):
            assert torch.equal(out, ref), f"call {i}: static-scratch result differs from the regular entry point"
            assert float(out.abs().sum()) > 0
        assert L.device_status(dev) == 0


def test_static_scratch_entry_point_rejects_oversize():
    from lookupffn_b200 import _lib as L

    lib = L.lib()
    dev = torch.device("cuda:0")
    N, T, m, rows, d = 1 << 20, 64, 1, 256, 64  # 67 M entries: far beyond the built-in array
    assert lib.lffn_gather_bwd_tables_sorted_scratch_bytes(N, T, m, rows) > L.STATIC_SCRATCH_BYTES
    buf = torch.zeros(64, device=dev)
    with torch.cuda.device(dev):
        rc = lib.lffn_gather_bwd_tables_sorted_static(L.ptr(buf), L.ptr(buf), L.ptr(buf), L.ptr(buf), N, T, m, rows, d,
                                                      L.stream_ptr(dev))
    assert rc == -5
    msg = lib.lffn_last_error_string().decode()
    assert "scratch" in msg and str(L.STATIC_SCRATCH_BYTES) in msg
