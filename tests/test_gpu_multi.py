"""Two-GPU checks of the multi-GPU modes over NCCL (skipped on a single-GPU box): the table-sharded
forward must equal the single-GPU forward of the whole layer on the rows each rank ends up owning."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import numpy as np
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from lookupffn_b200 import ops, sharded

        dev = torch.device("cuda", rank)
        N, d_in, D, T, k, d_out = 4096, 768, 1024, 96, 8, 512
        R = -(-T * k // D)
        g = torch.Generator(device=dev).manual_seed(5)   # same values on both ranks
        x = torch.randn(N, d_in, generator=g, device=dev).to(torch.bfloat16)
        signs = (2 * torch.randint(0, 2, (R, 2, D, 1, 1), generator=g, device=dev) - 1).float()
        tables = (0.02 * torch.randn(T << k, d_out, generator=g, device=dev)).to(torch.bfloat16)
        bias = torch.randn(d_out, generator=g, device=dev)
        desc = ops.make_hash_desc(d_in, signs, None, T, k, had_scale=1 / 32, mix_a=1.0, mix_b=0.0)
        idx, w, _ = ops.hash_fwd(x, desc)
        y_full = ops.weighted_vector_gather_add(idx, tables, w, bias=bias, out_dtype=torch.float32)
        tb, tc = sharded.table_range(T, rank, world)
        y_loc, owned = sharded.lookup_forward_table_sharded(x, desc, tables[tb << k:(tb + tc) << k].contiguous(), tb, tc,
                                                            bias=bias, chunk_tokens=1024)
        torch.cuda.synchronize()
        err = (y_loc - y_full[owned.to(dev)]).abs().max() / y_full.abs().max()
        q.put((rank, float(err), tuple(y_loc.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_table_sharded_forward_two_gpus():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, err, shape in res:
        assert shape == (2048, 512)
        assert err < 1e-6  # fp32 partial sums added in another order than the single fmaf chain


def _fused_worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from lookupffn_b200 import ops, sharded

        dev = torch.device("cuda", rank)
        N, d_in, D, T, k, d_out = 4096, 768, 1024, 96, 8, 512
        R = -(-T * k // D)
        g = torch.Generator(device=dev).manual_seed(5)
        x = torch.randn(N, d_in, generator=g, device=dev).to(torch.bfloat16)
        signs = (2 * torch.randint(0, 2, (R, 2, D, 1, 1), generator=g, device=dev) - 1).float()
        tables = (0.02 * torch.randn(T << k, d_out, generator=g, device=dev)).to(torch.bfloat16)
        bias = torch.randn(d_out, generator=g, device=dev)
        desc = ops.make_hash_desc(d_in, signs, None, T, k, had_scale=1 / 32, mix_a=1.0, mix_b=0.0)
        idx, w, _ = ops.hash_fwd(x, desc)
        y_full = ops.weighted_vector_gather_add(idx, tables, w, bias=bias, out_dtype=torch.float32)
        tb, tc = sharded.table_range(T, rank, world)
        errs = []
        local = tables[tb << k:(tb + tc) << k].contiguous()
        lo = rank * (N // world)
        for mode in ("store", "add", "copy"):
            peers = sharded.PeerOutput(N // world, d_out, dev, mode="store" if mode == "copy" else mode)
            fn = sharded.lookup_forward_table_sharded_copy if mode == "copy" else sharded.lookup_forward_table_sharded_fused
            for _ in range(3):  # repeatedly: the buffers are reused
                y_loc = fn(x, desc, local, tb, tc, peers, bias=bias)
                errs.append(float((y_loc - y_full[lo:lo + N // world]).abs().max() / y_full.abs().max()))
        q.put((rank, max(errs), tuple(y_loc.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_gather_reduce_scatter_two_gpus():
    """Gather + reduce-scatter in one kernel through peer-mapped output buffers vs the single-GPU forward."""
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29750 + os.getpid() % 200
    procs = [ctx.Process(target=_fused_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, err, shape in res:
        assert shape == (2048, 512)
        assert err < 1e-6


def _module_worker(rank, world, port, q):
    from argparse import Namespace

    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from lookupffn_b200 import LookupFFN, sharded

        dev = torch.device("cuda", rank)
        torch.manual_seed(0)  # the same module on every rank
        cfg = Namespace(hidden_size=512, ffn_num_table=256, ffn_table_size=256, layer_norm_eps=1e-5,
                        projection_type="bh4", block_size=64)
        full = LookupFFN(cfg, 512).to(dev).eval()
        x = torch.randn(2048, 512, device=dev, generator=torch.Generator(device=dev).manual_seed(1))
        with torch.no_grad():
            y_full = full(x)
        errs = {}
        for mode in ("nccl", "fused", "copy", "auto"):
            mod = sharded.TableShardedLookupFFN(full, chunk_tokens=512, exchange=mode)
            y_loc, owned = mod(x)
            errs[mode] = float((y_loc - y_full[owned.to(dev)]).abs().max() / y_full.abs().max())
        q.put((rank, errs, mod.t_count))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_table_sharded_module_two_gpus():
    """TableShardedLookupFFN (reference BH4 projection, tables split by T) with each exchange mode vs the whole
    module on one GPU."""
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 90
    procs = [ctx.Process(target=_module_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, errs, t_count in res:
        assert t_count == 128
        assert all(e < 1e-6 for e in errs.values()), errs


def _optimizer_worker(rank, world, port, q):
    """Data-parallel table update two ways on NCCL: the reference's way (DDP: all-reduce of the dense [T, 2^k, d]
    gradient, then the same AdamW step on every rank; main.py:40-47) and ShardedTableAdamW (reduce-scatter, update
    of the owned shard, all-gather).  Same tables afterwards, and both timed on the table set of one layer of the
    RoBERTa-small configuration (256 tables x 256 rows x 512, 134 MB)."""
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from lookupffn_b200.sharded import ShardedTableAdamW

        dev = torch.device("cuda", rank)
        T, rows, d = 256, 256, 512
        g0 = torch.Generator(device=dev).manual_seed(1)          # same initial tables on every rank
        init = 0.02 * torch.randn(T, rows, d, generator=g0, device=dev)
        gr = torch.Generator(device=dev).manual_seed(100 + rank)  # rank-specific gradients
        grads = [torch.randn(T, rows, d, generator=gr, device=dev) * 1e-3 for _ in range(3)]
        hyper = dict(lr=1e-3, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.01)

        dense = torch.nn.Parameter(init.clone())
        opt_d = torch.optim.AdamW([dense], **hyper)
        shard = torch.nn.Parameter(init.clone())
        opt_s = ShardedTableAdamW(shard, **hyper)

        def dense_step(gi):
            gsum = gi.clone()
            dist.all_reduce(gsum)
            dense.grad = gsum / world
            opt_d.step()

        def sharded_step(gi):
            shard.grad = gi.clone()
            opt_s.step()

        def timed(fn):
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for gi in grads:
                fn(gi)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / len(grads)

        ms_dense = timed(dense_step)
        ms_shard = timed(sharded_step)
        err = float((dense.data - shard.data).abs().max() / dense.data.abs().max())
        moved = float((dense.data - init).abs().max())
        q.put((rank, err, moved, ms_dense, ms_shard))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_table_adamw_matches_dense_allreduce_on_nccl():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + os.getpid() % 90
    procs = [ctx.Process(target=_optimizer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, err, moved, ms_dense, ms_shard in res:
        assert moved > 1e-4          # the steps changed the tables
        assert err < 1e-6, (rank, err)
    print("table update per step on 2 GPUs, ms: dense all-reduce + AdamW %.3f, reduce-scatter + sharded AdamW + "
          "all-gather %.3f" % (max(r[3] for r in res), max(r[4] for r in res)))
