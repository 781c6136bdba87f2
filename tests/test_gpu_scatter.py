"""The gather fused with the reduce-scatter exchange (lffn_gather_fwd_scatter), on ONE GPU.

In the table-sharded mode every rank runs this kernel over all tokens with its own tables and sends the row of
token n to the rank that owns it through a device array of buffer addresses.  Nothing in the kernel depends on
the buffers living on different GPUs, so here all "owners" are ordinary local allocations: each emulated rank
makes its call in turn (ranks are sequential launches on one stream, never kernels that wait on each other) and
the owners' buffers are then compared with the CPU oracle's partial sums.  Covered: both add modes (one bulk
reduction per row, 16-byte vector reductions), the slab mode, every first_owner, ragged N (the last owner only
partly filled), fp32 and bf16 tables, wide rows that take two column tiles.  Also: the bounded-wait self-test,
which makes a wait run out on purpose (a barrier nobody signals, nothing in flight) and expects the timeout bit.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

ADD_BULK, ADD_VECTOR = -1, -2


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from lookupffn_b200 import _lib

    _lib.lib()
    return torch.device("cuda:0")


def _rank_inputs(rng, N, I, S, d, bf16):
    idx = rng.randint(0, S, size=(N, I)).astype(np.int32)
    w = rng.randn(N, I).astype(np.float32)
    tables = (0.02 * rng.randn(S, d)).astype(np.float32)
    if bf16:
        bits = O.f32_to_bf16_bits(tables)
        return idx, w, bits, O.bf16_bits_to_f32(bits)
    return idx, w, tables, tables


def _to_dev(a, dev, bf16=False):
    if bf16:
        return torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16)
    return torch.from_numpy(a).to(dev)


def _scatter_call(L, idx, w, tables, ptr_array, n_owners, rows, slab, first_owner, N, dev):
    with torch.cuda.device(dev):
        L.check(L.lib().lffn_gather_fwd_scatter(L.ptr(idx), L.ptr(w), L.ptr(tables), L.dtype_code(tables.dtype),
                                                L.ptr(ptr_array), n_owners, rows, slab, first_owner, N,
                                                idx.shape[1], tables.shape[0], tables.shape[1], L.stream_ptr(dev)))


CASES = [
    # N, I, S, d, n_owners, bf16
    (64, 8, 512, 64, 2, False),
    (301, 24, 3000, 768, 2, True),      # ragged: 2 owners x 151 rows cover 301 tokens
    (500, 16, 4096, 1024, 4, True),     # the 2 KB bf16 rows of the table-sharded sweep
    (130, 5, 700, 1536, 3, False),      # fp32 rows wider than one column tile (two launches per call)
    (97, 33, 900, 256, 8, False),
]


@pytest.mark.parametrize("case", CASES, ids=[f"s{i}" for i in range(len(CASES))])
@pytest.mark.parametrize("mode", [ADD_BULK, ADD_VECTOR])
def test_scatter_add_modes_match_oracle_partials(dev, case, mode):
    from lookupffn_b200 import _lib as L

    N, I, S, d, n_owners, bf16 = case
    rows = -(-N // n_owners)
    rng = np.random.RandomState(N + I + d)
    ranks = [_rank_inputs(rng, N, I, S, d, bf16) for _ in range(n_owners)]
    bias = (0.01 * rng.randn(d)).astype(np.float32)
    partials = [O.gather(idx, w, t32) for idx, w, _, t32 in ranks]
    want = np.broadcast_to(bias, (N, d)).astype(np.float64) + sum(p.astype(np.float64) for p in partials)
    scale = np.abs(want).max()
    dev_ranks = [(_to_dev(idx, dev), _to_dev(w, dev), _to_dev(tb, dev, bf16)) for idx, w, tb, _ in ranks]
    for first_owner_shift in range(n_owners):
        bufs = [torch.from_numpy(np.broadcast_to(bias, (rows, d)).copy()).to(dev) for _ in range(n_owners)]
        ptr_array = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
        for r, (idx, w, tb) in enumerate(dev_ranks):  # the ranks' calls, one after the other
            _scatter_call(L, idx, w, tb, ptr_array, n_owners, rows, mode, (r + first_owner_shift) % n_owners, N, dev)
        torch.cuda.synchronize()
        got = torch.cat(bufs)[:N].cpu().numpy()
        # the ranks' rows are added in launch order here, each one fp32-rounded: 1e-6 of the largest value
        assert np.abs(got - want).max() <= 1e-6 * scale, (first_owner_shift, np.abs(got - want).max() / scale)
        if N < rows * n_owners:  # rows past the last token keep their initial value
            tail = torch.cat(bufs)[N:].cpu().numpy()
            np.testing.assert_array_equal(tail, np.broadcast_to(bias, tail.shape))
    assert L.device_status(dev) == 0


@pytest.mark.parametrize("case", CASES[:4], ids=[f"s{i}" for i in range(4)])
@pytest.mark.parametrize("bulk", [0, 0x40000000], ids=["stores16", "bulk_copy"])
def test_scatter_slab_mode_is_exact(dev, case, bulk):
    from lookupffn_b200 import _lib as L

    N, I, S, d, n_owners, bf16 = case
    rows = -(-N // n_owners)
    rng = np.random.RandomState(7 * N + d)
    ranks = [_rank_inputs(rng, N, I, S, d, bf16) for _ in range(n_owners)]
    bufs = [torch.full((n_owners, rows, d), float("nan"), device=dev) for _ in range(n_owners)]
    ptr_array = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    for r, (idx, w, tb, _) in enumerate(ranks):
        _scatter_call(L, _to_dev(idx, dev), _to_dev(w, dev), _to_dev(tb, dev, bf16), ptr_array, n_owners, rows, r | bulk,
                      (r + 1) % n_owners, N, dev)
    torch.cuda.synchronize()
    for r, (idx, w, _, t32) in enumerate(ranks):
        want = O.gather(idx, w, t32)  # rank r's partial rows, bit for bit, in slab r of each owner
        got = torch.cat([b[r] for b in bufs])[:N].cpu().numpy()
        np.testing.assert_array_equal(got, want)
    assert L.device_status(dev) == 0


def test_scatter_flags_out_of_range_rows_and_rejects_bad_modes(dev):
    from lookupffn_b200 import _lib as L

    N, I, S, d = 40, 6, 100, 64
    rng = np.random.RandomState(3)
    idx, w, tb, t32 = _rank_inputs(rng, N, I, S, d, False)
    idx[5, 2] = S + 7
    idx[9, 0] = -1
    buf = torch.zeros(N, d, device=dev)
    ptr_array = torch.tensor([buf.data_ptr()], dtype=torch.int64, device=dev)
    _scatter_call(L, _to_dev(idx, dev), _to_dev(w, dev), _to_dev(tb, dev), ptr_array, 1, N, ADD_BULK, 0, N, dev)
    assert L.device_status(dev) == L.STATUS_INDEX_RANGE
    wz = w.copy()
    wz[5, 2] = 0.0
    wz[9, 0] = 0.0
    idx_ok = np.clip(idx, 0, S - 1)
    np.testing.assert_array_equal(buf.cpu().numpy(), O.gather(idx_ok, wz, t32))
    lib = L.lib()
    with torch.cuda.device(dev):
        rc = lib.lffn_gather_fwd_scatter(L.ptr(buf), L.ptr(buf), L.ptr(buf), 0, L.ptr(ptr_array), 1, N, -3, 0, N, I,
                                         S, d, L.stream_ptr(dev))
    assert rc == -1 and b"slab" in lib.lffn_last_error_string()


def test_bounded_wait_runs_out_and_reports_timeout(dev):
    from lookupffn_b200 import _lib as L

    assert L.device_status(dev) == 0
    with torch.cuda.device(dev):
        L.check(L.lib().lffn_selftest_bounded_wait(1000, L.stream_ptr(dev)))
    assert L.device_status(dev) == L.STATUS_TIMEOUT  # the wait gave up and said so
    assert L.device_status(dev) == 0                  # reading cleared it
    # the device is still usable
    x = torch.randn(4, 64, device=dev)
    from lookupffn_b200 import ops

    np.testing.assert_array_equal(ops.hadamard(x).cpu().numpy(), O.fwht(x.cpu().numpy()))
