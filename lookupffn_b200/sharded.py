"""Multi-GPU forms of the LookupFFN forward, one process per GPU over torch.distributed.

Token sharding (the default; tables replicated): tokens are independent, rank g runs the ordinary
module on its own rows and no collective is needed in the forward.  `token_range` gives the split.

Table sharding (table sets too large to replicate): rank g owns tables [t_begin, t_begin + t_count),
sees all N tokens, computes the partial sum over its tables in fp32 and the partials are combined
by a reduce-scatter(sum) over tokens, chunk by chunk so that the collective of chunk c overlaps the
kernels of chunk c+1 (NCCL runs on its own stream).  After the call rank g holds N/world rows; the
rows it owns are returned with it.  The reference has no counterpart (it is data-parallel only,
main.py:40-47); the partition is the one of the benchmark's table-sharded sweep (1 GB of tables split by T
over 8 GPUs, every GPU seeing all 262,144 tokens).
"""
import torch
import torch.distributed as dist
import torch.nn as nn

from . import ops

SCATTER_SLAB_BULK = 0x40000000  # lookupffn.h: store a row into its slab as one bulk copy


def token_range(N, rank, world):
    """Contiguous split of N tokens; the first N % world ranks take one more."""
    base, rem = divmod(N, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def table_range(T, rank, world):
    """(t_begin, t_count) of rank's contiguous share of T tables; the first T % world ranks take one more."""
    lo, hi = token_range(T, rank, world)
    return lo, hi - lo


def rotations_needed(t_begin, t_count, k, D):
    """Inclusive range of projection rotations whose coordinates tables [t_begin, t_begin+t_count) read
    (tables may straddle a rotation boundary when k does not divide D)."""
    return (t_begin * k) // D, ((t_begin + t_count) * k - 1) // D


def chunk_plan(N, world, chunk_tokens):
    """[(start, size)] covering N tokens; every size is a multiple of world."""
    if N % world != 0:
        raise ValueError(f"table sharding needs N ({N}) divisible by the world size ({world})")
    step = max(world, (chunk_tokens // world) * world)
    return [(s, min(step, N - s)) for s in range(0, N, step)]


def owned_tokens(N, rank, world, chunk_tokens):
    """Token indices (ascending within each chunk) that end up on `rank` after the chunked reduce-scatter."""
    out = []
    for s, n in chunk_plan(N, world, chunk_tokens):
        per = n // world
        out.append(torch.arange(s + rank * per, s + (rank + 1) * per))
    return torch.cat(out) if out else torch.empty(0, dtype=torch.long)


def reduce_scatter_partials(partial_fn, N, d_out, device, group=None, chunk_tokens=32768, bias=None,
                            out_dtype=torch.float32):
    """Runs partial_fn(start, size) -> fp32 [size, d_out] (this rank's partial sum for tokens
    [start, start+size)) over all chunks and reduce-scatters each chunk.  Returns [N/world, d_out]."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    plan = chunk_plan(N, world, chunk_tokens)
    out = torch.empty((N // world, d_out), dtype=torch.float32, device=device)
    works, keep, pos = [], [], 0
    for s, n in plan:
        part = partial_fn(s, n)
        if part.dtype != torch.float32 or part.shape != (n, d_out):
            raise ValueError("partial_fn must return fp32 [size, d_out]")
        dst = out[pos:pos + n // world]
        works.append(dist.reduce_scatter_tensor(dst, part.contiguous(), op=dist.ReduceOp.SUM, group=group,
                                                async_op=True))
        keep.append(part)  # the collective reads it asynchronously
        pos += n // world
    for w in works:
        w.wait()
    del keep, rank
    if bias is not None:
        out += bias.to(out.dtype)
    return out if out_dtype == torch.float32 else out.to(out_dtype)


def lookup_forward_table_sharded(x, desc, tables_local, t_begin, t_count, bias=None, group=None,
                                 chunk_tokens=32768, out_dtype=torch.float32):
    """x [N, d_in] (the same on every rank); desc describes the WHOLE layer's projection;
    tables_local [t_count * 2^k, d_out] are this rank's tables.  Returns (y_local [N/world, d_out],
    owned token indices)."""
    N = x.shape[0]
    d_out = tables_local.shape[1]

    def partial(start, size):
        idx, w, _ = ops.hash_fwd(x[start:start + size], desc, t_begin=t_begin, t_count=t_count)
        return ops.weighted_vector_gather_add(idx, tables_local, w, out_dtype=torch.float32)

    y = reduce_scatter_partials(partial, N, d_out, x.device, group=group, chunk_tokens=chunk_tokens, bias=bias,
                                out_dtype=out_dtype)
    world = dist.get_world_size(group)
    return y, owned_tokens(N, dist.get_rank(group), world, chunk_tokens)


class TableShardedLookupFFN(nn.Module):
    """A LookupFFN whose tables are split by T across the ranks of `group`.  Built from a full module
    (every rank constructs or loads the same one) and keeps only its own slice of `tables`;
    LayerNorm, projection and bias stay replicated."""

    def __init__(self, full, group=None, chunk_tokens=32768, exchange="auto"):
        """exchange: "nccl" (chunked reduce-scatter), "fused" (one bulk reduction per row from the gather kernel into
        the owner's buffer), "copy" (copy-engine transfers into per-rank slabs, summed in rank order) or "auto": when
        the tokens divide evenly over the ranks, copy (262,144 tokens, 256 tables per rank: 10.3 ms against 12.4
        fused and 12.0 NCCL on 8 GPUs, 10.4 / 11.3 / 11.6 on 2), except short gathers on 2 ranks, where fused leads
        (16 tables per rank: 2.6 ms against 2.9 copy and 3.3 NCCL); NCCL otherwise."""
        super().__init__()
        self.group = group
        self.chunk_tokens = chunk_tokens
        self.exchange = exchange
        self._peers = None
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.t_begin, self.t_count = table_range(full.num_table, rank, world)
        self.LayerNorm = full.LayerNorm
        self.hash = full.hash
        self.bias = full.bias
        self.table_size = full.table_size
        self.output_size = full.output_size
        self.tables = nn.Parameter(full.tables.detach()[self.t_begin:self.t_begin + self.t_count].clone(),
                                   requires_grad=False)

    @torch.no_grad()
    def forward(self, hidden_states):
        """hidden_states [N, hidden], identical on all ranks -> (y_local [N/world, out], owned token indices)."""
        if not hidden_states.is_cuda:
            raise RuntimeError("lookupffn_b200 runs on CUDA tensors only (no CPU fallback)")
        u = self.LayerNorm(hidden_states)
        N = u.shape[0]
        flat = self.tables.reshape(self.t_count * self.table_size, self.output_size)
        world = dist.get_world_size(self.group)
        rows_per_token = self.t_count * self.hash.candidates
        if self.exchange == "copy" or (self.exchange == "auto" and world > 1 and N % world == 0
                                       and (rows_per_token >= 128 or world >= 4)):
            if self._peers is None or self._peers.rows != N // world or self._peers.mode != "store":
                self._peers = PeerOutput(N // world, self.output_size, u.device, group=self.group, mode="store")
            rank = dist.get_rank(self.group)
            y = _copy_exchange(lambda lo, hi: self.hash(u[lo:hi], t_begin=self.t_begin, t_count=self.t_count), N, u.device,
                               flat, self._peers, self.bias)
            return y, torch.arange(rank * self._peers.rows, (rank + 1) * self._peers.rows)
        fused = self.exchange == "fused" or (self.exchange == "auto" and world > 1 and N % world == 0
                                             and rows_per_token >= 16)
        if fused:
            if self._peers is None or self._peers.rows != N // world:
                self._peers = PeerOutput(N // world, self.output_size, u.device, group=self.group)
            peers = self._peers
            peers.reset(self.bias)
            idx, w = self.hash(u, t_begin=self.t_begin, t_count=self.t_count)
            from . import _lib as L
            with torch.cuda.device(u.device):
                L.check(L.lib().lffn_gather_fwd_scatter(L.ptr(idx), L.ptr(w), L.ptr(flat), L.dtype_code(flat.dtype),
                                                        L.ptr(peers.ptr_array), world, peers.rows, -1,
                                                        (peers.rank + 1) % world, N, idx.shape[1], flat.shape[0],
                                                        self.output_size, L.stream_ptr(u.device)))
            rank = dist.get_rank(self.group)
            return peers.finish().clone(), torch.arange(rank * peers.rows, (rank + 1) * peers.rows)

        def partial(start, size):
            idx, w = self.hash(u[start:start + size], t_begin=self.t_begin, t_count=self.t_count)
            return ops.weighted_vector_gather_add(idx, flat, w, out_dtype=torch.float32)

        y = reduce_scatter_partials(partial, N, self.output_size, u.device, group=self.group,
                                    chunk_tokens=self.chunk_tokens, bias=self.bias)
        world = dist.get_world_size(self.group)
        return y, owned_tokens(N, dist.get_rank(self.group), world, self.chunk_tokens)


class ShardedTableAdamW:
    """Data-parallel training step for the `tables` parameter without a dense all-reduce.

    Under the reference's DDP (main.py:40-47) every rank all-reduces the full [T, 2^k, d] table gradient
    (67-134 MB per layer) and then runs the same optimizer update on every GPU.  Here the gradients are
    reduce-scattered over the table dimension, rank g updates only tables [t_begin, t_begin + t_count) with
    AdamW state for that shard only (1/world of the optimizer memory and arithmetic), and the updated shards
    are all-gathered back.  Bytes on the wire equal an all-reduce; state and update work are divided by world.
    T must be divisible by the world size.  The arithmetic is torch.optim.AdamW's (decoupled weight decay).
    """

    def __init__(self, tables, group=None, lr=1e-4, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.01):
        self.tables, self.group = tables, group
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        T = tables.shape[0]
        if T % self.world != 0:
            raise ValueError(f"T = {T} tables must be divisible by the world size {self.world}")
        self.t_count = T // self.world
        self.t_begin = self.rank * self.t_count
        shard_shape = (self.t_count,) + tuple(tables.shape[1:])
        self.exp_avg = torch.zeros(shard_shape, dtype=torch.float32, device=tables.device)
        self.exp_avg_sq = torch.zeros(shard_shape, dtype=torch.float32, device=tables.device)
        self.steps = 0

    @torch.no_grad()
    def step(self):
        g_full = self.tables.grad
        if g_full is None:
            raise RuntimeError("tables.grad is None: run backward first")
        g_full = g_full.float().contiguous()
        g = torch.empty_like(self.exp_avg)
        dist.reduce_scatter_tensor(g, g_full, op=dist.ReduceOp.SUM, group=self.group)
        g /= self.world  # DDP averages gradients over ranks
        self.steps += 1
        b1, b2 = self.betas
        shard = self.tables.data[self.t_begin:self.t_begin + self.t_count]
        p = shard.float()
        p.mul_(1 - self.lr * self.weight_decay)
        self.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        bc1, bc2 = 1 - b1 ** self.steps, 1 - b2 ** self.steps
        denom = (self.exp_avg_sq.sqrt() / (bc2 ** 0.5)).add_(self.eps)
        p.addcdiv_(self.exp_avg, denom, value=-self.lr / bc1)
        new_shard = p.to(self.tables.dtype).contiguous()
        dist.all_gather_into_tensor(self.tables.data, new_shard, group=self.group)

    def zero_grad(self):
        self.tables.grad = None


class PeerOutput:
    """Output buffers of all ranks, each mapped into every process (torch symmetric memory: CUDA peer mappings
    over NVLink), plus the device array of their addresses that lffn_gather_fwd_scatter takes.
    mode "add" (default): every rank owns [N/world, d] fp32 and partial rows are added in place, one bulk
    reduction per row (summation order across ranks not fixed).
    mode "store": every rank owns a staging buffer [world, N/world, d] fp32; rank r's partial rows go into slab r
    of the owner's buffer (one bulk copy per row from the gather kernel, or one copy-engine transfer per owner in
    lookup_forward_table_sharded_copy) and the owner sums the slabs in rank order (deterministic).
    Allocate once and reuse across steps."""

    def __init__(self, rows_per_rank, d, device, group=None, mode="add"):
        import torch.distributed._symmetric_memory as symm_mem

        assert mode in ("store", "add")
        self.mode = mode
        self.group = dist.group.WORLD if group is None else group
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.rows, self.d = rows_per_rank, d
        shape = (self.world, rows_per_rank, d) if mode == "store" else (rows_per_rank, d)
        self.local = symm_mem.empty(shape, dtype=torch.float32, device=device)
        self.handle = symm_mem.rendezvous(self.local, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.ptr_array = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self._flag = torch.zeros(1, dtype=torch.float32, device=device)
        self._copy = None  # lookup_forward_table_sharded_copy: (stream, two staging buffers, their events, peer views)

    def _rank_barrier(self):
        """Orders the ranks on the device, without stopping the host: a one-element all-reduce enqueued on every
        rank's stream.  It completes on a rank only after every rank has reached it, i.e. after everything each rank
        enqueued before it has finished; what this rank enqueues afterwards waits for it."""
        dist.all_reduce(self._flag, group=self.group)

    def reset(self, bias=None):
        """Before a step.  "add": the owner writes the initial value (zeros or the bias) of its rows.  Both
        modes end with a rank barrier: no peer may write into a buffer its owner is still reading or initialising."""
        if self.mode == "add":
            if bias is None:
                self.local.zero_()
            else:
                self.local.copy_(bias.to(torch.float32)[None].expand_as(self.local))
        self._rank_barrier()

    def finish(self, bias=None):
        """After every rank's kernel has finished all partial rows have landed; returns this rank's [N/world, d]."""
        self._rank_barrier()
        if self.mode == "add":
            return self.local
        out = self.local.sum(0)
        if bias is not None:
            out += bias.to(out.dtype)
        return out


def lookup_forward_table_sharded_copy(x, desc, tables_local, t_begin, t_count, peers, bias=None):
    """The table-sharded forward with the exchange done by the copy engines: the rank gathers the partial rows of
    one owner at a time into a local staging buffer and a peer-to-peer copy on a second stream moves them into its
    slab of that owner's buffer while the next owner's rows are gathered; the rank's own rows come last and go
    straight into its own slab, so no copy is left exposed at the end.  The owner then sums its slabs in rank order
    (deterministic).  No SM issues a remote store: sending rows from the gather kernel itself slows that kernel by
    1.2-2.5 ms per GiB sent (2 GPUs, one direction, 256 tables per rank), more than the transfer takes.
    `peers` is a PeerOutput(mode="store").  Returns this rank's [N/world, d] fp32 rows."""
    def hash_rows(lo, hi):
        idx, w, _ = ops.hash_fwd(x[lo:hi], desc, t_begin=t_begin, t_count=t_count)
        return idx, w

    return _copy_exchange(hash_rows, x.shape[0], x.device, tables_local, peers, bias)


def _copy_exchange(hash_rows, N, dev, tables_local, peers, bias):
    """hash_rows(lo, hi) -> (idx, w) of tokens [lo, hi) for this rank's tables; see lookup_forward_table_sharded_copy."""
    from . import _lib as L

    if peers.mode != "store":
        raise ValueError("the copy-engine exchange needs PeerOutput(mode='store')")
    world, rank, rows = peers.world, peers.rank, peers.rows
    if N != rows * world:
        raise ValueError(f"N = {N} tokens but the peer buffers hold {rows} x {world} rows")
    tables_local = tables_local if tables_local.is_contiguous() else tables_local.contiguous()
    S, d = tables_local.shape
    if peers._copy is None:
        shape = (world, rows, d)
        peers._copy = (torch.cuda.Stream(device=dev), [torch.empty((rows, d), dtype=torch.float32, device=dev) for _ in range(2)],
                       [None, None], [peers.handle.get_buffer(o, shape, torch.float32) for o in range(world)])
    cstream, stage, stage_free, views = peers._copy
    bias32 = None if bias is None else bias.to(torch.float32).contiguous()
    main = torch.cuda.current_stream(dev)
    peers.reset()  # every owner has finished reading its slabs of the previous step
    for c in range(world):
        o = (rank + 1 + c) % world  # the rank's own rows last
        idx, w = hash_rows(o * rows, (o + 1) * rows)
        if o == rank:
            dst = peers.local[rank]
        else:
            dst = stage[c & 1]
            if stage_free[c & 1] is not None:
                main.wait_event(stage_free[c & 1])  # the copy that last read this staging buffer has finished
        with torch.cuda.device(dev):
            L.check(L.lib().lffn_gather_fwd(L.ptr(idx), L.ptr(w), L.ptr(tables_local), L.dtype_code(tables_local.dtype),
                                            L.ptr(dst), L.dtype_code(torch.float32), rows, idx.shape[1], S, d,
                                            L.ptr(bias32) if o == rank else None, L.stream_ptr(dev)))
        if o != rank:
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(cstream):
                cstream.wait_event(ready)
                views[o][rank].copy_(dst, non_blocking=True)
                done = torch.cuda.Event()
                done.record(cstream)
            stage_free[c & 1] = done
    main.wait_stream(cstream)  # this rank's copies have landed before it enters the barrier of finish()
    return peers.finish()      # the bias went into the rank's own slab with the gather's epilogue


def lookup_forward_table_sharded_fused(x, desc, tables_local, t_begin, t_count, peers, bias=None):
    """The table-sharded forward with the exchange step of the reduce-scatter fused into the gather kernel: each
    rank's gather sends its partial rows straight to the owner's buffer through peer-mapped memory over NVLink
    (plain stores into its slab, or one in-place bulk reduction per row), so the [N, d] partial sums are never written to
    or read from this GPU's HBM and no NCCL collective moves data.  Token n is owned by rank n // (N / world).
    Returns this rank's [N/world, d] fp32 rows."""
    from . import _lib as L

    N = x.shape[0]
    if N != peers.rows * peers.world:
        raise ValueError(f"N = {N} tokens but the peer buffers hold {peers.rows} x {peers.world} rows")
    peers.reset(bias)
    idx, w, _ = ops.hash_fwd(x, desc, t_begin=t_begin, t_count=t_count)
    tables_local = tables_local if tables_local.is_contiguous() else tables_local.contiguous()
    S, d = tables_local.shape
    slab = (peers.rank | SCATTER_SLAB_BULK) if peers.mode == "store" else -1
    with torch.cuda.device(x.device):
        L.check(L.lib().lffn_gather_fwd_scatter(L.ptr(idx), L.ptr(w), L.ptr(tables_local),
                                                L.dtype_code(tables_local.dtype), L.ptr(peers.ptr_array), peers.world,
                                                peers.rows, slab, (peers.rank + 1) % peers.world, N, idx.shape[1], S, d,
                                                L.stream_ptr(x.device)))
    return peers.finish(bias if peers.mode == "store" else None)
