"""Host-side logic of the multi-GPU modes, run as world_size-2 gloo processes on CPU.  The per-rank
partial sums come from the CPU oracle here (the CUDA kernels need a GPU); what is under test is the
partitioning, the chunked reduce-scatter plumbing and the token ownership map."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lookupffn_b200 import sharded


def test_ranges_partition_exactly():
    for n, world in [(10, 3), (512, 8), (7, 8), (128, 1)]:
        spans = [sharded.token_range(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    assert sharded.table_range(512, 3, 8) == (192, 64)
    # k = 6 does not divide D = 1024: a rank's tables can start inside a rotation and end in a later one
    assert sharded.rotations_needed(1024, 1024, 6, 1024) == (6, 11)
    assert sharded.rotations_needed(0, 170, 6, 1024) == (0, 0)
    assert sharded.rotations_needed(0, 171, 6, 1024) == (0, 1)


def test_chunk_plan_and_ownership():
    N, world, chunk = 1000, 4, 300
    plan = sharded.chunk_plan(N, world, chunk)
    assert sum(n for _, n in plan) == N and all(n % world == 0 for _, n in plan)
    owned = [sharded.owned_tokens(N, r, world, chunk) for r in range(world)]
    assert all(len(o) == N // world for o in owned)
    assert sorted(torch.cat(owned).tolist()) == list(range(N))
    with pytest.raises(ValueError):
        sharded.chunk_plan(1001, 4, 300)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O

        rng = np.random.RandomState(0)  # same data on every rank
        N, d_in, D, T, k, d_out = 48, 100, 128, 22, 6, 64   # k does not divide D: tables straddle rotations
        R = -(-T * k // D)
        x = rng.randn(N, d_in).astype(np.float32)
        signs = (2.0 * rng.randint(0, 2, size=(R, 2, D, 1, 1)) - 1.0).astype(np.float32)
        tables = (0.02 * rng.randn(T << k, d_out)).astype(np.float32)
        bias = rng.randn(d_out).astype(np.float32)
        y_full = O.layer_fwd(x, signs, tables, T, k, mix_a=1.0, mix_b=0.0, bias=bias)

        tb, tc = sharded.table_range(T, rank, world)
        local = tables[tb << k:(tb + tc) << k]
        z = O.project(x, signs, T * k, mix_a=1.0, mix_b=0.0)

        def partial(start, size):
            idx, w = O.code_weights(z[start:start + size, tb * k:(tb + tc) * k], tc, k)
            return torch.from_numpy(O.gather(idx, w, local))

        chunk = 20
        y_loc = sharded.reduce_scatter_partials(partial, N, d_out, torch.device("cpu"), chunk_tokens=chunk,
                                                bias=torch.from_numpy(bias))
        owned = sharded.owned_tokens(N, rank, world, chunk)
        ref = y_full[owned.numpy()]
        # partial sums are added in another order than the single fmaf chain: 1e-6 of the largest output
        ok = np.abs(y_loc.numpy() - ref).max() <= 1e-6 * np.abs(y_full).max()
        # a partial of the wrong shape is rejected on the host, before any collective is posted
        try:
            sharded.reduce_scatter_partials(lambda s, n: torch.zeros(n, d_out + 1), N, d_out, torch.device("cpu"))
            bad_shape_caught = False
        except ValueError:
            bad_shape_caught = True
        q.put((rank, bool(ok), bad_shape_caught, int(y_loc.shape[0])))
    finally:
        dist.destroy_process_group()


def test_table_sharded_reduce_scatter_world2():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == [(0, True, True, 24), (1, True, True, 24)]


def _adam_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        T, rows, d = 8, 16, 12
        init = torch.randn(T, rows, d)
        tables = torch.nn.Parameter(init.clone())
        ref = torch.nn.Parameter(init.clone())
        opt = sharded.ShardedTableAdamW(tables, lr=1e-2, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.01)
        ref_opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.01)
        for step in range(3):
            g_local = torch.randn(T, rows, d, generator=torch.Generator().manual_seed(100 * step + rank))
            tables.grad = g_local.clone()
            opt.step()
            # what DDP does: all-reduce (mean) the dense gradient, then the full update on every rank
            g_avg = g_local.clone()
            dist.all_reduce(g_avg)
            ref.grad = g_avg / world
            ref_opt.step()
        err = float((tables.detach() - ref.detach()).abs().max())
        q.put((rank, err, tuple(opt.exp_avg.shape)))
    finally:
        dist.destroy_process_group()


def test_sharded_table_adamw_equals_ddp_allreduce_world2():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + os.getpid() % 90
    procs = [ctx.Process(target=_adam_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, shape in res:
        assert shape == (4, 16, 12)   # optimizer state covers half of the tables
        assert err < 1e-6
