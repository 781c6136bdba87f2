#!/usr/bin/env python
"""Benchmark of the LookupFFN layer forward (hash -> gather-add) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c1|c2|c5k8] [--impl ours|reference]

One "step" = one pass of the layer forward over one batch of synthetic tokens.  Default workload
"c3": N = 65536 tokens per GPU, d = 768 (zero-padded to D = 1024), T = 512 tables of 2^8 rows,
bf16 x / tables / y, fp32 accumulation, projection v = H diag(s2) H diag(s1) x with seeded +-1
diagonals (4 rotations), reference score weights, MSB-first codes.  For N GPUs the tokens are
partitioned (each rank its own N tokens, tables replicated, no collective): weak scaling.

Prints ONE JSON line (rank 0).  `value` = tokens/s with inputs resident in HBM; `e2e` = the same
through the host-buffer C-ABI call (pinned host x in, pinned host y out, copies inside the timed
region); `roofline` = the gather kernel's algorithmic bytes per launch over its CUDA-event time;
`cpu_baseline` = the reference's CPU path timed on this box's host cores on a bounded sample.
`--impl reference` times only that CPU path.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

WORKLOADS = {
    # name: N per GPU, d_in, d_out, T, k, storage dtype, projection, weight_mode, bit_order
    "c1": dict(N=4096, d_in=512, d_out=512, T=128, k=8, dtype="f32", weight_mode="ones", bit_order="lsb"),
    "c2": dict(N=16384, d_in=512, d_out=512, T=256, k=8, dtype="f32", weight_mode="score", bit_order="msb"),
    "c3": dict(N=65536, d_in=768, d_out=768, T=512, k=8, dtype="bf16", weight_mode="score", bit_order="msb"),
    # config 5 (table-sharded sweep): T here = tables PER GPU = (1 GB / (2^k * 1024 * 2 B)) / 8
    "c5k6": dict(N=262144, d_in=1024, d_out=1024, T=1024, k=6, dtype="bf16", weight_mode="score", bit_order="msb"),
    "c5k8": dict(N=262144, d_in=1024, d_out=1024, T=256, k=8, dtype="bf16", weight_mode="score", bit_order="msb"),
    "c5k10": dict(N=262144, d_in=1024, d_out=1024, T=64, k=10, dtype="bf16", weight_mode="score", bit_order="msb"),
    "c5k12": dict(N=262144, d_in=1024, d_out=1024, T=16, k=12, dtype="bf16", weight_mode="score", bit_order="msb"),
}
# Counters of the gather kernel from one ncu capture of this binary's kernel (dram__bytes_read.sum +
# dram__bytes_write.sum, lts__t_sector_hit_rate.pct), per launch.  c3: captured on a 16384-token launch and
# scaled by 4 to the 65536-token launch, DRAM traffic being proportional to the waves of tokens (the tables are
# re-fetched once per wave of resident warps).  `commit` is the source revision the capture was taken from.
NCU_PROFILE = {"c3": {"traffic_bytes_per_launch": 4 * 1.4844e9, "l2_hit_rate": 0.772, "commit": "2a0dc9b",
                      "capture": "ncu --set full, 16384-token launch of the same kernel, traffic x 4"}}


def padded_dim(d):
    return 1 << int(np.ceil(np.log2(d)))


def algorithmic_bytes_per_token(w):
    eb = 2 if w["dtype"] == "bf16" else 4
    # every gathered row once per use + x in + y out; codes/weights not counted
    return w["T"] * w["d_out"] * eb + w["d_in"] * eb + w["d_out"] * eb


def load_peaks():
    p = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---- clocks ------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) every 20 ms."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        while not self.stop_flag.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                r = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self.stop_flag.wait(0.02)

    def result(self):
        self.stop_flag.set()
        if self.is_alive():
            self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ---- host placement ---------------------------------------------------------------------------------
def _parse_cpulist(text):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_node(local):
    """NUMA node and local CPU list of GPU `local` from sysfs (read-only), or (None, set())."""
    try:
        p = torch.cuda.get_device_properties(local)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        base = f"/sys/bus/pci/devices/{bus}"
        node = int(open(base + "/numa_node").read())
        cpus = _parse_cpulist(open(base + "/local_cpulist").read())
        return (node if node >= 0 else None), cpus
    except Exception:
        return None, set()


def bind_rank_to_gpu(local, world):
    """Process placement only (no GPU or driver setting): this rank's threads go to a share of the CPUs that are
    local to its GPU, disjoint from the other ranks' shares, and its future host allocations prefer the GPU's NUMA
    node (set_mempolicy, MPOL_PREFERRED).  Returns what was done, for the JSON line."""
    info = {"gpu_numa_node": None, "cpus": None, "mempolicy": "unchanged"}
    try:
        allowed = sorted(os.sched_getaffinity(0))
        nodes = [gpu_numa_node(i) for i in range(torch.cuda.device_count())][:max(world, local + 1)]
        node, near = nodes[local]
        info["gpu_numa_node"] = node
        pool = sorted(set(allowed) & near) or allowed
        sharers = [i for i, (nd, nr) in enumerate(nodes) if (sorted(set(allowed) & nr) or allowed) == pool]
        pos, cnt = sharers.index(local), len(sharers)
        per = max(1, len(pool) // cnt)
        mine = pool[pos * per:(pos + 1) * per] or pool
        os.sched_setaffinity(0, mine)
        torch.set_num_threads(max(1, min(len(mine), 4)))
        info["cpus"] = f"{mine[0]}-{mine[-1]} ({len(mine)} of {len(allowed)} allowed)"
        if node is not None:
            libc = C.CDLL(None, use_errno=True)
            mask = (C.c_ulong * 16)()
            mask[node // 64] = 1 << (node % 64)
            rc = libc.syscall(238, 1, mask, C.c_ulong(16 * 64))  # x86-64 set_mempolicy(MPOL_PREFERRED, mask, maxnode)
            info["mempolicy"] = f"preferred node {node}" if rc == 0 else f"set_mempolicy errno {C.get_errno()}"
    except Exception as e:  # placement is an optimisation; the run goes on without it
        info["error"] = repr(e)
    return info


def pinned_like(t):
    """Page-locked host tensor of t's shape and dtype.  Allocated with the process's own allocator (so that the
    NUMA preference set above applies on first touch) and then registered with the CUDA runtime."""
    h = torch.empty(t.shape, dtype=t.dtype)
    h.view(torch.int16 if h.element_size() == 2 else h.dtype).zero_()  # first touch, under the NUMA preference
    rc = torch.cuda.cudart().cudaHostRegister(h.data_ptr(), h.numel() * h.element_size(), 0)
    if int(rc) != 0:
        return torch.empty(t.shape, dtype=t.dtype).pin_memory()
    _REGISTERED.append(h)  # stays registered, and alive, until the process ends
    return h


_REGISTERED = []


# ---- synthetic workload ----------------------------------------------------------------------------
def make_inputs(w, device, seed):
    """Seeded synthetic stand-ins for the pre-training activations and trained tables: x ~ N(0,1),
    tables ~ N(0, 0.02), +-1 diagonals; the same on every rank except x (rank-specific tokens)."""
    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float32
    D = padded_dim(w["d_in"])
    R = max(1, -(-w["T"] * w["k"] // D))
    g = torch.Generator(device=device).manual_seed(1234)
    tables = (0.02 * torch.randn(w["T"] << w["k"], w["d_out"], generator=g, device=device)).to(dt)
    signs = (2 * torch.randint(0, 2, (R, 2, D, 1, 1), generator=g, device=device) - 1).float()
    bias = torch.zeros(w["d_out"], device=device)
    gx = torch.Generator(device=device).manual_seed(1000 + seed)
    x = torch.randn(w["N"], w["d_in"], generator=gx, device=device).to(dt)
    return x, tables, signs, bias, D, R


def layer_config(args, w, world):
    """The `config` object of the JSON line; identical for this arm and for the reference arm."""
    eb = 2 if w["dtype"] == "bf16" else 4
    D = padded_dim(w["d_in"])
    R = max(1, -(-w["T"] * w["k"] // D))
    N, T = w["N"], w["T"]
    return {"workload": f"{args.workload}: LookupFFN layer forward, N={N} tokens per GPU, d={w['d_in']}->D={D}, "
                        f"T={T}, k={w['k']}, d_out={w['d_out']}, {w['dtype']} x/tables/y, fp32 accumulate",
            "projection": f"sign-diagonal Hadamard, R={R} rotations x 2 stages, normalised",
            "weights": w["weight_mode"], "bit_order": w["bit_order"],
            "sharding": f"tokens x{world}, tables replicated",
            "l2": "inputs larger than L2: tables %.0f MB + idx/w %.0f MB + x/y %.0f MB per step" % (
                (T << w["k"]) * w["d_out"] * eb / 1e6, N * T * 8 / 1e6, 2 * N * w["d_in"] * eb / 1e6)}


def run_ours(args, rank, world, local):
    from lookupffn_b200 import _lib as L
    from lookupffn_b200 import ops

    w = dict(WORKLOADS[args.workload])
    if args.tokens:
        w["N"] = args.tokens
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    placement = bind_rank_to_gpu(local, world)
    lib = L.lib()
    x, tables, signs, bias, D, R = make_inputs(w, device, rank)
    N, T, k = w["N"], w["T"], w["k"]
    dt = x.dtype
    dcode = L.dtype_code(dt)
    wm = {"score": L.WEIGHT_SCORE, "ones": L.WEIGHT_ONES}[w["weight_mode"]]
    bo = {"msb": L.MSB_FIRST, "lsb": L.LSB_FIRST}[w["bit_order"]]
    desc = ops.make_hash_desc(w["d_in"], signs, None, T, k, had_scale=float(1.0 / np.sqrt(D)), mix_a=1.0, mix_b=0.0,
                              bit_order=bo, weight_mode=wm)
    idx = torch.empty((N, T), dtype=torch.int32, device=device)
    wgt = torch.empty((N, T), dtype=torch.float32, device=device)
    y = torch.empty((N, w["d_out"]), dtype=dt, device=device)
    stream = torch.cuda.current_stream(device)
    sp = C.c_void_p(stream.cuda_stream)

    def step(ev=None):
        if ev is not None:
            ev[0].record(stream)
        L.check(lib.lffn_hash_fwd(C.byref(desc), L.ptr(x), dcode, N, 0, T, L.ptr(idx), L.ptr(wgt), None, sp))
        if ev is not None:
            ev[1].record(stream)
        L.check(lib.lffn_gather_fwd(L.ptr(idx), L.ptr(wgt), L.ptr(tables), dcode, L.ptr(y), dcode, N, T, T << k,
                                    w["d_out"], L.ptr(bias), sp))
        if ev is not None:
            ev[2].record(stream)

    def barrier():
        if world > 1:
            torch.distributed.barrier()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()

    sampler = ClockSampler(physical_gpu_index(local))
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    torch.cuda.synchronize()
    sampler.start()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    for s in range(args.steps):
        step(events[s])
    t_end.record(stream)
    torch.cuda.synchronize()
    barrier()
    elapsed_ms = t_start.elapsed_time(t_end)
    clocks = sampler.result()
    hash_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in events)
    gather_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in events)
    status = L.device_status(device)

    # The gather's own ceiling when no row comes from DRAM: the same launch (same N, list length, row size) with
    # every index folded into the first 32 tables, a band that stays in L2.  Outside the timed region.
    band = min(T, 32) << k
    idx_l2 = torch.remainder(idx, band).contiguous()
    y_l2 = torch.empty_like(y)
    ev_l2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for i in range(4):
        if i == 1:
            ev_l2[0].record(stream)
        L.check(lib.lffn_gather_fwd(L.ptr(idx_l2), L.ptr(wgt), L.ptr(tables), dcode, L.ptr(y_l2), dcode, N, T, T << k,
                                    w["d_out"], L.ptr(bias), sp))
    ev_l2[1].record(stream)
    torch.cuda.synchronize()
    l2_resident_ms = ev_l2[0].elapsed_time(ev_l2[1]) / 3
    del idx_l2, y_l2

    # Hardware ceiling of that access pattern: plain coalesced 16-byte reads of a 32 or 64 MiB buffer that stays in L2
    # (lffn_probe_read), in four configurations of loads in flight per SM; the best one is the ceiling.  Outside the
    # timed region.  One launch reads about as many bytes as the gather launch does.
    sink = torch.zeros(1, dtype=torch.int32, device=device)
    l2_probe = {}
    for mbytes in (32, 64):
        probe_bytes = min(mbytes << 20, tables.numel() * tables.element_size()) // 16 * 16
        for mode, name in ((0, "12_loads_per_thread_gather_residency"), (1, "8_loads_per_thread"),
                           (2, "16_loads_per_thread"), (3, "4_loads_per_thread_64_warps")):
            got = C.c_size_t(0)
            L.check(lib.lffn_probe_read(L.ptr(tables), probe_bytes, 4, mode, L.ptr(sink), C.byref(got), sp))
            reps = max(8, int(algorithmic_bytes_per_token(w) * N // max(1, got.value)))
            ev_p = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev_p[0].record(stream)
            L.check(lib.lffn_probe_read(L.ptr(tables), probe_bytes, reps, mode, L.ptr(sink), C.byref(got), sp))
            ev_p[1].record(stream)
            torch.cuda.synchronize()
            l2_probe[f"{name}_{mbytes}MiB"] = got.value * reps / (ev_p[0].elapsed_time(ev_p[1]) * 1e-3) / 1e9  # GB/s
    l2_read_peak = max(l2_probe.values())

    if args.no_e2e:  # profiling runs: device path only
        if rank == 0:
            print(json.dumps({"workload": args.workload, "N": N, "hash_ms": hash_ms, "gather_ms": gather_ms,
                              "ms_per_step": elapsed_ms / args.steps,
                              "gather_GBps": algorithmic_bytes_per_token(w) * N / gather_ms / 1e6}), flush=True)
        return None

    # ---- end to end through the host-buffer entry point -------------------------------------------
    chunk = args.e2e_chunk
    ws_bytes = lib.lffn_layer_fwd_host_ws_bytes(C.byref(desc), dcode, dcode, w["d_out"], chunk)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
    x_host = pinned_like(x)
    x_host.copy_(x)
    y_host = pinned_like(y)

    # What the host side allows with no kernels at all: the step's x going in and a y coming out, both whole, on
    # two streams at once, all ranks at the same time.  The end-to-end number cannot beat this, nor the device path.
    cs_in, cs_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    x_tmp = torch.empty_like(x)

    def copy_step():
        with torch.cuda.stream(cs_in):
            x_tmp.copy_(x_host, non_blocking=True)
        with torch.cuda.stream(cs_out):
            y_host.copy_(y, non_blocking=True)

    copy_steps = max(5, min(args.steps, 30))
    for _ in range(3):
        copy_step()
    torch.cuda.synchronize()
    barrier()
    ev_c = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev_c[0].record(stream)
    cs_in.wait_stream(stream)
    cs_out.wait_stream(stream)
    for _ in range(copy_steps):
        copy_step()
    stream.wait_stream(cs_in)
    stream.wait_stream(cs_out)
    ev_c[1].record(stream)
    torch.cuda.synchronize()
    copy_s = ev_c[0].elapsed_time(ev_c[1]) * 1e-3 / copy_steps
    barrier()
    del x_tmp

    def e2e_step():
        L.check(lib.lffn_layer_fwd_host(C.byref(desc), L.ptr(x_host), dcode, N, L.ptr(tables), dcode, w["d_out"],
                                        L.ptr(bias), L.ptr(y_host), dcode, L.ptr(ws), ws_bytes, chunk, sp))

    for _ in range(max(1, min(args.warmup, 3))):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ok = bool(torch.equal(y_host.view(torch.int16) if dt == torch.bfloat16 else y_host,
                              y.cpu().view(torch.int16) if dt == torch.bfloat16 else y.cpu()))
    barrier()
    torch.cuda.synchronize()
    ev_e = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev_e[0].record(stream)
    for _ in range(args.steps):
        e2e_step()  # synchronous: returns when y_host is complete; its copies and kernels are ordered after `stream`
    ev_e[1].record(stream)
    torch.cuda.synchronize()
    e2e_s = ev_e[0].elapsed_time(ev_e[1]) * 1e-3
    barrier()

    if world > 1:
        t = torch.tensor([elapsed_ms, e2e_s, gather_ms, hash_ms, copy_s], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        elapsed_ms, e2e_s, gather_ms, hash_ms, copy_s = (float(v) for v in t.tolist())
        placements = [None] * world
        torch.distributed.all_gather_object(placements, placement)
    else:
        placements = [placement]

    if rank != 0:
        return None
    parity = comparator = None
    if world == 1 and not args.no_cpu_baseline and not args.tokens:
        step()
        torch.cuda.synchronize()
        parity = parity_sample(args, x, signs, tables, idx, wgt, y, float(1.0 / np.sqrt(D)))
        comparator = gpu_comparator(idx, wgt, tables, y, gather_ms)
    eb = 2 if w["dtype"] == "bf16" else 4
    alg = algorithmic_bytes_per_token(w)
    peak, peak_kind = load_peaks()
    achieved = alg * N / (gather_ms * 1e-3) / 1e9
    chunks = -(-N // chunk)
    prof = NCU_PROFILE.get(args.workload) if not args.tokens else None
    traffic = prof["traffic_bytes_per_launch"] if prof else None
    value = world * N * args.steps / (elapsed_ms * 1e-3)
    e2e_value = world * N * args.steps / e2e_s
    copy_ceiling = world * N / copy_s
    ceiling = min(copy_ceiling, value)
    out = {
        "metric": "lookupffn_layer_forward_throughput", "value": value,
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic",
        "config": layer_config(args, w, world),
        "kernels_ms": {"hash_fwd": hash_ms, "gather_fwd": gather_ms},
        # `achieved` counts every gathered row once per use (algorithmic bytes), so `frac` above 1 is not an HBM
        # fraction: each table row is used N / 2^k times per launch and most uses are served from L2.  What limits
        # the kernel is L2 read bandwidth; the DRAM side is `traffic` (ncu) over the same time.
        "roofline": {"bound": "hbm", "limiter": "l2 read bandwidth", "kernel": "gather_fwd_kernel",
                     "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                     "algorithmic_bytes_per_token": alg, "traffic": traffic,
                     "traffic_capture": {k: prof[k] for k in ("capture", "commit")} if prof else None,
                     "dram_achieved": traffic / (gather_ms * 1e-3) / 1e9 if traffic else None,
                     "dram_frac": traffic / (gather_ms * 1e-3) / 1e9 / peak if traffic else None,
                     "l2_hit_rate": prof["l2_hit_rate"] if prof else None,
                     "l2_read_peak": l2_read_peak, "frac_of_l2_read_peak": achieved / l2_read_peak,
                     "l2_read_peak_source": "lffn_probe_read: 16-byte loads of an L2-resident 32 / 64 MiB buffer, best of "
                                            "eight configurations, measured in this run",
                     "l2_read_probe_GBps": l2_probe,
                     # the same launch with all indices folded into an L2-resident band of 32 tables:
                     "l2_resident_launch_ms": l2_resident_ms, "frac_of_l2_resident_launch": l2_resident_ms / gather_ms},
        "e2e": {"value": e2e_value, "unit": "tokens/s",
                "h2d_bytes_per_step": N * w["d_in"] * eb, "d2h_bytes_per_step": N * w["d_out"] * eb,
                "api": "lffn_layer_fwd_host (pinned host x -> pinned host y)", "chunk_tokens": chunk,
                "matches_device_path": e2e_ok,
                # the same bytes copied both ways at once with no kernels, all ranks together (max over ranks)
                "host_copy_ceiling": {"value": copy_ceiling, "unit": "tokens/s", "ms_per_step": copy_s * 1e3,
                                      "GBps_per_direction_per_gpu": N * w["d_in"] * eb / copy_s / 1e9},
                "ceiling": ceiling, "frac_of_ceiling": e2e_value / ceiling,
                "placement": placements},
        "gpu_launches": 2 * args.steps + 2 * chunks * args.steps,
        "clocks": clocks, "device_status": status, "parity_sample": parity, "gpu_comparator": comparator,
    }
    return out


def table_sharded_setup(w, rank, world, device):
    """Inputs of the table-sharded mode (benchmark configuration 5): every rank sees all N tokens (identical x),
    owns T_per_gpu tables of a layer with T_per_gpu * world tables."""
    from lookupffn_b200 import ops

    N, k, d_in, d_out = w["N"], w["k"], w["d_in"], w["d_out"]
    t_count = w["T"]
    T = t_count * world
    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float32
    D = padded_dim(d_in)
    R = max(1, -(-T * k // D))
    g = torch.Generator(device=device).manual_seed(1234)
    signs = (2 * torch.randint(0, 2, (R, 2, D, 1, 1), generator=g, device=device) - 1).float()
    x = torch.randn(N, d_in, generator=g, device=device).to(dt)          # identical on every rank
    gt = torch.Generator(device=device).manual_seed(77 + rank)
    tables = (0.02 * torch.randn(t_count << k, d_out, generator=gt, device=device)).to(dt)
    bias = torch.zeros(d_out, device=device)
    desc = ops.make_hash_desc(d_in, signs, None, T, k, had_scale=float(1.0 / np.sqrt(D)), mix_a=1.0, mix_b=0.0)
    return dict(x=x, tables=tables, bias=bias, desc=desc, t_begin=rank * t_count, t_count=t_count, T=T, dt=dt)


def table_sharded_step_fn(S, rs, chunk, world, device):
    """One step of the table-sharded forward with exchange `rs`: "nccl" (chunked NCCL reduce-scatter), "fused" (one
    bulk reduction per row from the gather kernel into the owner's buffer over NVLink), "fused-store" (one bulk copy
    per row into the rank's slab of the owner's buffer, the owner sums its slabs in rank order), "copy" (the gather
    writes locally, one owner's rows at a time, and copy-engine transfers move them into the owners' slabs while the
    next rows are gathered), or "none" (no exchange: the rank's partial sums stay local -- the one-GPU pace of the same shape)."""
    from lookupffn_b200 import ops, sharded

    x, tables, bias, desc = S["x"], S["tables"], S["bias"], S["desc"]
    if rs == "none":
        def step():
            idx, wg, _ = ops.hash_fwd(x, desc, t_begin=S["t_begin"], t_count=S["t_count"])
            return ops.weighted_vector_gather_add(idx, tables, wg, out_dtype=torch.float32)
        return step, None
    if rs == "nccl":
        def step():
            return sharded.lookup_forward_table_sharded(x, desc, tables, S["t_begin"], S["t_count"], bias=bias,
                                                        chunk_tokens=chunk, out_dtype=torch.float32)[0]
        return step, None
    peers = sharded.PeerOutput(x.shape[0] // world, tables.shape[1], device, mode="add" if rs == "fused" else "store")
    fn = sharded.lookup_forward_table_sharded_copy if rs == "copy" else sharded.lookup_forward_table_sharded_fused

    def step():
        return fn(x, desc, tables, S["t_begin"], S["t_count"], peers, bias=bias)
    return step, peers


def time_steps(step, steps, warmup, device, world):
    """CUDA-event time per step in ms, max over ranks, bracketed by barriers and synchronisation."""
    for _ in range(warmup):
        y = step()
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        y = step()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t[0]), y


def table_sharded_record(args, rank, world, local):
    """Appended to the default line when more than one GPU runs: a short run of benchmark configuration 5 (tables
    split by T over the GPUs, every GPU sees all 262,144 tokens, partial sums combined by a reduce-scatter over
    NVLink) with every exchange (NCCL, the two fused forms, copy engines), beside the same per-GPU shape without any exchange.  k = 8 at every N; k = 6 and
    k = 12 too at 8 GPUs.  Every rank runs it; rank 0 reports."""
    device = torch.device("cuda", local)
    ks = args.table_sharded_ks.split(",") if args.table_sharded_ks else ["c5k8"] + (["c5k12", "c5k6"] if world >= 8 else [])
    steps, warmup = 5, 3
    rec = {"what": "tables sharded by T, all tokens on every GPU, fp32 partial sums reduce-scattered over tokens",
           "nccl_ranks": torch.distributed.get_world_size(), "steps": steps, "warmup": warmup, "runs": {}}
    for name in ks:
        w = dict(WORKLOADS[name])
        S = table_sharded_setup(w, rank, world, device)
        N, d_out = w["N"], w["d_out"]
        run = {"tokens": N, "tables_per_gpu": w["T"], "k": w["k"], "d": d_out,
               "reduce_scattered_bytes_per_gpu": N * d_out * 4,
               "bytes_leaving_each_gpu_over_nvlink": N * d_out * 4 * (world - 1) // world}
        keys = {"none": "one_gpu_pace_no_exchange", "nccl": "nccl_reduce_scatter", "fused": "fused_in_gather_kernel",
                "fused-store": "fused_in_gather_kernel_slabs", "copy": "copy_engine_slabs"}
        for rs in ("none", "nccl", "fused", "fused-store", "copy"):
            step, peers = table_sharded_step_fn(S, rs, args.rs_chunk, world, device)
            ms, _ = time_steps(step, steps, warmup, device, world)
            run[keys[rs]] = {"ms_per_step": ms, "tokens_per_s": N / (ms * 1e-3)}
            del step, peers
            torch.cuda.empty_cache()
        base = run["one_gpu_pace_no_exchange"]["ms_per_step"]
        for key in list(keys.values())[1:]:
            run[key]["pace_vs_no_exchange"] = base / run[key]["ms_per_step"]
        rec["runs"][name] = run
        del S
        torch.cuda.empty_cache()
    return rec if rank == 0 else None


def run_table_sharded(args, rank, world, local):
    """Config-5 style: every rank sees all N tokens, owns T_per_gpu tables (the whole layer has
    T_per_gpu * world), partial sums are reduce-scattered over NVLink chunk by chunk."""
    from lookupffn_b200 import sharded

    w = dict(WORKLOADS[args.workload])
    if args.tokens:
        w["N"] = args.tokens
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    S = table_sharded_setup(w, rank, world, device)
    N, k, d_in, d_out, t_count, T, dt = w["N"], w["k"], w["d_in"], w["d_out"], S["t_count"], S["T"], S["dt"]
    x = S["x"]
    chunk = args.rs_chunk
    step, peers = table_sharded_step_fn(S, args.rs, chunk, world, device)
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    ms, y = time_steps(step, args.steps, args.warmup, device, world)
    clocks = sampler.result()
    elapsed_ms = ms * args.steps

    # end to end: x from pinned host memory every step, the rank's rows of y back to pinned host memory
    x_host = pinned_like(x)
    x_host.copy_(x)
    y_host = pinned_like(y)

    def e2e_step():
        x.copy_(x_host, non_blocking=True)
        y_host.copy_(step(), non_blocking=True)
        return y_host

    e2e_ms, _ = time_steps(e2e_step, args.steps, 1, device, world)
    e2e_s = e2e_ms * 1e-3 * args.steps
    if rank != 0:
        return None
    eb = 2 if w["dtype"] == "bf16" else 4
    chunks = len(sharded.chunk_plan(N, world, chunk))
    return {
        "metric": "lookupffn_layer_forward_throughput", "value": N * args.steps / (elapsed_ms * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": f"{args.workload}, tables sharded: N={N} tokens on every GPU, d={d_in}, T={t_count} "
                               f"tables per GPU ({T} in the layer), k={k}, {w['dtype']} x/tables, fp32 partial sums, "
                               + (f"NCCL reduce-scatter in {chunks} chunks" if peers is None else
                                  f"exchange fused into the gather kernel (peer {peers.mode} over NVLink)"),
                   "sharding": f"tables x{world}", "l2": "inputs larger than L2"},
        "table_rows_per_s": world * N * t_count * args.steps / (elapsed_ms * 1e-3),
        "rs_bytes_per_step_per_gpu": N * d_out * 4,
        "e2e": {"value": N * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": N * d_in * eb,
                "d2h_bytes_per_step": (N // world) * d_out * 4, "api": "sharded.lookup_forward_table_sharded"},
        "gpu_launches": 2 * chunks * args.steps, "clocks": clocks,
    }


def run_train_gather(args, rank, world, local):
    """Benchmark configuration 4: training-mode weighted gather-add, forward and backward, fp32: N=16384 tokens, d=768,
    T=512, k=8, m=k+1 soft-flip candidates per (token, table) (tau=0.5), upstream gradient dy ~ N(0,1).
    One step = candidates/weights (hash kernel) + gather forward + gradient of the weights + gradient of the
    tables (sorted, deterministic)."""
    from lookupffn_b200 import _lib as L
    from lookupffn_b200 import ops

    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    lib = L.lib()
    N, d, T, k = (args.tokens or 16384), 768, 512, 8
    m, rows, D = k + 1, 1 << k, 1024
    R = -(-T * k // D)
    g = torch.Generator(device=device).manual_seed(4321 + rank)
    x = torch.randn(N, d, generator=g, device=device)
    signs = (2 * torch.randint(0, 2, (R, 2, D, 1, 1), generator=g, device=device) - 1).float()
    tables = 0.02 * torch.randn(T * rows, d, generator=g, device=device)
    dy = torch.randn(N, d, generator=g, device=device)
    desc = ops.make_hash_desc(d, signs, None, T, k, had_scale=1.0 / 32, mix_a=1.0, mix_b=0.0,
                              weight_mode=L.WEIGHT_SOFT_FLIP, tau=0.5)
    I = T * m
    idx = torch.empty(N, I, dtype=torch.int32, device=device)
    w = torch.empty(N, I, device=device)
    y = torch.empty(N, d, device=device)
    dw = torch.empty(N, I, device=device)
    dt = torch.empty(T * rows, d, device=device)
    nbytes = lib.lffn_gather_bwd_tables_sorted_scratch_bytes(N, T, m, rows)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream(device)
    sp = C.c_void_p(stream.cuda_stream)
    names = ["hash_soft_flip", "gather_fwd", "grad_weights", "grad_tables_sorted"]

    def step(ev=None):
        calls = [
            lambda: lib.lffn_hash_fwd(C.byref(desc), L.ptr(x), 0, N, 0, T, L.ptr(idx), L.ptr(w), None, sp),
            lambda: lib.lffn_gather_fwd(L.ptr(idx), L.ptr(w), L.ptr(tables), 0, L.ptr(y), 0, N, I, T * rows, d, None, sp),
            lambda: lib.lffn_gather_bwd_weights(L.ptr(idx), L.ptr(dy), L.ptr(tables), 0, L.ptr(dw), N, I, T * rows, d, sp),
            lambda: lib.lffn_gather_bwd_tables_sorted(L.ptr(idx), L.ptr(w), L.ptr(dy), L.ptr(dt), N, T, m, rows, d,
                                                      L.ptr(scratch), nbytes, sp),
        ]
        for i, c in enumerate(calls):
            if ev is not None:
                ev[i].record(stream)
            L.check(c())
        if ev is not None:
            ev[4].record(stream)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(local))
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps)]
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    sampler.start()
    for s_ in range(args.steps):
        step(events[s_])
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    clocks = sampler.result()
    elapsed_ms = events[0][0].elapsed_time(events[-1][4])
    per = {n: statistics.mean(e[i].elapsed_time(e[i + 1]) for e in events) for i, n in enumerate(names)}
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        elapsed_ms = float(t[0])
    if rank != 0:
        return None
    comparator = None
    if world == 1 and not args.no_cpu_baseline:
        # baseline leg: the reference's own fp32 CUDA kernels (oracle/_ref, unmodified, sm_100a) on the same tensors
        from oracle import build as obuild

        gat = obuild.load_ref_module("gather_add")
        if gat is not None:
            def once(fn):
                fn()  # warm-up
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                return e0.elapsed_time(e1)

            ry, rdw, rdt = torch.zeros_like(y), torch.zeros_like(dw), torch.zeros_like(dt)
            ref_ms = {
                "gather_fwd": once(lambda: gat.weighted_vector_gather_add_fp32(idx, tables, w, ry)),
                "grad_weights": once(lambda: gat.indexed_inner_product_fp32(idx, dy, tables, rdw)),
            }
            rdt.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gat.weighted_vector_scatter_add_fp32(idx, dy, w, rdt)  # one launch, into zeros: its result is checked
            e1.record()
            torch.cuda.synchronize()
            ref_ms["grad_tables_atomics"] = e0.elapsed_time(e1)

            def rel(a, b):
                return float((a - b).abs().max() / b.abs().max())

            comparator = {"kernels": "reference weighted_vector_gather_add / indexed_inner_product / "
                                     "weighted_vector_scatter_add fp32 (gather/cuda/extension, unmodified, sm_100a)",
                          "ms": ref_ms, "ms_total": sum(ref_ms.values()),
                          "ours_ms_total": per["gather_fwd"] + per["grad_weights"] + per["grad_tables_sorted"],
                          "max_abs_diff_over_max_abs": {"y": rel(y, ry), "dw": rel(dw, rdw), "dtables": rel(dt, rdt)}}
            del ry, rdw, rdt
    logical = N * I * d * 4
    return {
        "metric": "lookupffn_gather_forward_backward_throughput", "value": world * N * args.steps / (elapsed_ms * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"c4: training-mode weighted gather-add forward + backward, N={N} tokens per GPU, d={d}, "
                               f"T={T}, k={k}, m={m} soft-flip candidates (tau 0.5), fp32 tables",
                   "l2": "inputs larger than L2: tables 403 MB, indices+weights 604 MB"},
        "kernels_ms": per,
        "algorithmic_GBps": {n: logical / (per[n] * 1e-3) / 1e9 for n in names[1:]},
        "gpu_launches": 5 * args.steps, "clocks": clocks, "device_status": L.device_status(device),
        "gpu_comparator": comparator,
    }


def run_train_layer(args, rank, world, local):
    """One training step (forward + full backward: tables, bias, projection weights and bias, LayerNorm, input) of a
    LookupFFN layer with the reference's pre-training shape (cfgs/roberta/small-512/lookup-t128-s8-bh4.py: hidden
    512, 128 tables of 256 rows, BH4 projection with 64 x 64 blocks; 64 sequences x 512 tokens = 32768 tokens per
    GPU), fp32, beside the reference's autograd over its own CUDA kernels on the same module and inputs."""
    from argparse import Namespace

    from lookupffn_b200 import LookupFFN

    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    cfg = Namespace(hidden_size=512, ffn_num_table=128, ffn_table_size=256, layer_norm_eps=1e-5, projection_type="bh4",
                    block_size=64)
    torch.manual_seed(77)
    mod = LookupFFN(cfg, 512).to(device).train()
    N = args.tokens or 32768
    gen = torch.Generator(device=device).manual_seed(5 + rank)
    x = torch.randn(N, 512, generator=gen, device=device, requires_grad=True)
    dy = torch.randn(N, 512, generator=gen, device=device)

    def step(fn):
        for q in mod.parameters():
            q.grad = None
        x.grad = None
        y = fn(x)
        y.backward(dy)
        return y

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            step(fn)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step(fn)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    steps = min(args.steps, 10)
    ms = timed(mod, steps, 3)
    ours = {n: q.grad.clone() for n, q in mod.named_parameters()}
    ours["x"] = x.grad.clone()
    comparator = None
    if not args.no_cpu_baseline:
        from oracle import build as obuild

        fht = obuild.load_ref_module("fast_hadamard_transform_kernel")
        gat = obuild.load_ref_module("gather_add")
        if fht is not None and gat is not None:
            from oracle.ref_gpu_path import lookupffn_reference_gpu_training

            ref_fn = lambda t: lookupffn_reference_gpu_training(mod, t, fht, gat)  # noqa: E731
            ref_ms = timed(ref_fn, min(steps, 5), 2)
            ref = {n: q.grad.clone() for n, q in mod.named_parameters()}
            ref["x"] = x.grad.clone()
            comparator = {"what": "the reference's autograd over torch.einsum, its Hadamard, gather, inner-product and "
                                  "scatter-add CUDA kernels (compiled unmodified for sm_100a) on the same module",
                          "ms_per_step": ref_ms, "ratio": ref_ms / ms,
                          "gradient_max_abs_diff_over_max_abs":
                              {n: float((ours[n] - ref[n]).abs().max() / ref[n].abs().max()) for n in ours}}
    if rank != 0:
        return None
    return {"metric": "lookupffn_layer_training_step", "value": N / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
            "steps": steps, "config": f"LookupFFN forward + backward, N={N} tokens, hidden 512, T=128, k=8, bh4 64x64, fp32",
            "gpu_comparator": comparator}


def encoder_gpu_comparator(model, step, B, S, cfg, device):
    """Baseline leg of the encoder run (N = 1, outside the timed region): the same model with every FFN evaluated the
    way the reference does it on a GPU -- torch.einsum for the 64 x 64 blocks, the reference's own Hadamard and
    gather CUDA kernels (compiled unmodified for sm_100a into oracle/_ref), elementwise torch for codes and scores
    (oracle/ref_gpu_path.py restates the Python between the kernels).  Attention and embeddings are the same code in
    both arms."""
    from oracle import build as obuild

    fht = obuild.load_ref_module("fast_hadamard_transform_kernel")
    gat = obuild.load_ref_module("gather_add")
    if fht is None or gat is None or cfg.projection_type != "bh4":
        return None
    from oracle.ref_gpu_path import lookupffn_reference_gpu

    def time_ms(fn, reps):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    ours = step().float()
    ffn = model.encoder.layer[0].FFN
    h = torch.randn(B, S, cfg.hidden_size, generator=torch.Generator(device=device).manual_seed(5), device=device)
    with torch.inference_mode():
        ours_ffn_ms = time_ms(lambda: ffn(h), 10)
        ref_ffn_ms = time_ms(lambda: lookupffn_reference_gpu(ffn, h, fht, gat), 5)
        y_ours, y_ref = ffn(h), lookupffn_reference_gpu(ffn, h, fht, gat)
        ffn_err = float((y_ours - y_ref).abs().max() / y_ours.abs().max())
        # hash codes of this layer against the reference's GPU evaluation, with the disagreements binned by the
        # magnitude of the coordinate (fp64 evaluation of the projection) that caused them
        from oracle import parity as PAR
        from oracle.ref_gpu_path import code_score_reference_gpu, projection_reference_gpu

        T, rows = ffn.num_table, ffn.table_size
        k = int(np.log2(rows))
        h2 = h.reshape(-1, cfg.hidden_size)
        ln = (ffn.LayerNorm.weight, ffn.LayerNorm.bias, ffn.LayerNorm.eps)
        pw, pb = ffn.hash.projection.weight, ffn.hash.projection.bias
        # ours: the inference path, LayerNorm inside the hash kernel; reference: torch LayerNorm, einsum, its own
        # Hadamard kernel; fp64: the same formulas in double from a double LayerNorm
        z_ours = ffn.hash.project(h2, layer_norm=ln)
        z_ref = projection_reference_gpu(ffn.LayerNorm(h2), pw, pb, T * k, fht)
        hn64 = torch.nn.functional.layer_norm(h2.double(), (cfg.hidden_size,), ln[0].double(), ln[1].double(), ln[2])
        z64 = PAR.projection_fp64_torch(hn64, pw, pb, T * k)
        parity = PAR.sign_mismatch_report(z_ours.cpu().numpy(), z_ref.cpu().numpy(), z64.cpu().numpy())
        code_ours = ffn.hash(h2, layer_norm=ln)[0] - (torch.arange(T, device=device, dtype=torch.int32) * rows)[None]
        code_ref = code_score_reference_gpu(z_ref.reshape(-1, T, k))[0]
        differ = code_ours != code_ref
        clean = ~differ.any(dim=-1)
        yo, yr = y_ours.reshape(-1, y_ours.shape[-1]), y_ref.reshape(-1, y_ref.shape[-1])
        parity.update({"hash_codes_checked": int(code_ref.numel()), "hash_code_mismatches": int(differ.sum()),
                       "tokens": int(clean.numel()), "tokens_without_a_differing_code": int(clean.sum()),
                       "ffn_output_max_rel_err_on_those_tokens":
                           float((yo[clean] - yr[clean]).abs().max() / yr[clean].abs().max()) if bool(clean.any()) else None})
        del hn64
        del z64, z_ours, z_ref
    patched = []
    try:
        for layer in model.encoder.layer:
            m = layer.FFN
            m.forward = (lambda hs, residual=None, m=m:
                         lookupffn_reference_gpu(m, hs, fht, gat) if residual is None
                         else lookupffn_reference_gpu(m, hs, fht, gat) + residual)
            patched.append(m)
        ref_out = step().float()
        ref_ms = time_ms(step, 5)
    finally:
        for m in patched:
            del m.forward
    err = float((ref_out - ours).abs().max() / ours.abs().max())
    return {"what": "same encoder, FFN evaluated the reference's way on this GPU (torch.einsum + the reference's "
                    "Hadamard and gather CUDA kernels + elementwise torch)",
            "seq_per_s": B / (ref_ms * 1e-3), "ms_per_step": ref_ms,
            "ffn_layer_ms": {"reference_style": ref_ffn_ms, "ours": ours_ffn_ms},
            "max_abs_diff_over_max_abs": {"ffn_layer": ffn_err, "encoder_output": err},
            "note": "the two maxima run over all tokens, including those whose hash code differs from the reference's on a "
                    "coordinate with |v| < 1e-6 (the LayerNorm inside the hash kernel rounds differently from torch's): "
                    "such a token reads another table row, which moves its output by a few per cent of the output "
                    "scale.  parity_sample counts them and gives the agreement on all other tokens.",
            "parity_sample": parity}


def run_encoder(args, rank, world, local):
    """Benchmark configuration 2: RoBERTa-small prenorm encoder inference with every FFN a LookupFFN (4 layers, hidden
    512, 8 heads, seq 512, batch 32 per GPU, T=256, k=8, fp32 tables, reference BH4 projection).  seq/s."""
    from argparse import Namespace

    from lookupffn_b200.encoder import Lookup

    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    cfg = Namespace(vocab_size=50265, type_vocab_size=1, pad_token_id=1, num_hidden_layers=4, num_attention_heads=8,
                    attention_head_size=64, layer_norm_eps=1e-5, hidden_size=512, hidden_dropout_prob=0.1,
                    attention_probs_dropout_prob=0.1, max_position_embeddings=512, projection_type=args.projection,
                    block_size=64, ffn_num_table=256, ffn_table_size=256)
    torch.manual_seed(1234)
    model = Lookup(cfg).to(device).eval()
    B, S = 32, 512
    g = torch.Generator().manual_seed(99 + rank)
    ids_host = torch.randint(5, cfg.vocab_size, (B, S), generator=g)
    ids_host[:, 0] = 0
    ids_host = ids_host.pin_memory()
    ids = ids_host.to(device)
    tt = torch.zeros(B, S, dtype=torch.long, device=device)
    pos = torch.arange(S, device=device)[None].repeat(B, 1)
    mask = torch.ones(B, S, device=device)
    out_host = torch.empty(B, S, cfg.hidden_size).pin_memory()

    amp = {"on": False}

    def step():
        with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16, enabled=amp["on"]):
            return model(ids, tt, pos, mask)[0]

    def e2e_step():
        ids.copy_(ids_host, non_blocking=True)
        out_host.copy_(step(), non_blocking=True)

    def timed(fn):
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
        return e0.elapsed_time(e1)

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    ms = timed(step)
    clocks = sampler.result()
    e2e_step()
    e2e_ms = timed(e2e_step)
    # the same model with the attention / linear layers around the FFN under bf16 autocast (the reference runs its
    # encoder under 16-bit mixed precision, cfgs/roberta/small-512/*.py: trainer.precision = 16); the LookupFFN
    # kernels and tables stay fp32.  Reported beside the fp32 number, never instead of it.
    amp["on"] = True
    for _ in range(3):
        step()
    amp_ms = timed(step)
    amp["on"] = False
    comparator = None
    if world == 1 and not args.no_cpu_baseline:
        comparator = encoder_gpu_comparator(model, step, B, S, cfg, device)
    if world > 1:
        t = torch.tensor([ms, e2e_ms, amp_ms], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, e2e_ms, amp_ms = (float(v) for v in t.tolist())
    if rank != 0:
        return None
    return {
        "metric": "roberta_small_lookupffn_encoder_inference", "value": world * B * args.steps / (ms * 1e-3),
        "unit": "seq/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c2: RoBERTa-small prenorm encoder inference, 4 layers, hidden 512, 8 heads, seq 512, "
                               "batch 32 per GPU, vocab 50265, LookupFFN T=256 k=8 d_out=512 fp32 tables, "
                               f"projection {args.projection}, random-init weights",
                   "l2": "inputs larger than L2: 4 x 134 MB of tables per step"},
        "tokens_per_s": world * B * S * args.steps / (ms * 1e-3),
        "with_bf16_autocast_around_the_ffn": {"value": world * B * args.steps / (amp_ms * 1e-3), "unit": "seq/s",
                                              "ms_per_step": amp_ms / args.steps},
        "e2e": {"value": world * B * args.steps / (e2e_ms * 1e-3), "unit": "seq/s", "h2d_bytes_per_step": B * S * 8,
                "d2h_bytes_per_step": B * S * cfg.hidden_size * 4, "api": "lookupffn_b200.encoder.Lookup.forward"},
        "gpu_launches": 2 * cfg.num_hidden_layers * args.steps, "clocks": clocks, "gpu_comparator": comparator,
    }


# ---- the reference's CPU path, on this box's host cores ---------------------------------------------------
def load_ref_modules():
    """The reference's own CPU extensions compiled (unmodified) into oracle/_ref, or None."""
    import importlib.util

    from oracle import build as obuild

    mods = {}
    for name in ("ccs_cpu", "gather_add_cpu"):
        path = obuild.ref_module_path(name)
        if not os.path.exists(path):
            return None
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods


def gpu_comparator(idx, wgt, tables, y, gather_ms):
    """Part of the baseline leg (N = 1, outside the timed region): the reference's own CUDA gather kernel, compiled
    unmodified for sm_100a into oracle/_ref, on the benchmark's indices, weights and tables on the same GPU.
    16-bit tables go through its fp16 kernel (fp16 storage and fp16 accumulation), fp32 through its fp32 kernel."""
    from oracle import build as obuild

    mod = obuild.load_ref_module("gather_add")
    if mod is None:
        return None
    N, d = y.shape
    I = idx.shape[1]
    if I % 2 or d % 64:
        return {"unavailable": "the reference kernel needs an even list length and a row size that is a multiple of 64"}
    if tables.dtype == torch.float32:
        fn, name, src, wt = mod.weighted_vector_gather_add_fp32, "weighted_vector_gather_add_fp32", tables, wgt
    else:
        fn, name = mod.weighted_vector_gather_add_fp16, "weighted_vector_gather_add_fp16"
        src, wt = tables.to(torch.float16), wgt.to(torch.float16)
    out = torch.zeros((N, d), dtype=src.dtype, device=y.device)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    fn(idx, src, wt, out)  # warm-up; launches on the default stream, which is the current stream here
    ev[0].record()
    for _ in range(3):
        fn(idx, src, wt, out)
    ev[1].record()
    torch.cuda.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / 3
    scale = float(y.float().abs().max())
    err = float((out.float() - y.float()).abs().max()) / max(scale, 1e-30)
    return {"kernel": f"reference {name} (gather/cuda/extension, unmodified, sm_100a)", "ms_per_launch": ms,
            "ours_ms_per_launch": gather_ms, "ratio": ms / gather_ms, "max_abs_diff_over_max_abs": err,
            "note": "same indices, weights and tables; bias is zero in this workload"}


def parity_sample(args, x, signs, tables, idx, wgt, y, hs):
    """Part of the CPU-baseline leg: the oracle re-computes the first `cpu_tokens` tokens of the benchmark's own
    inputs and the GPU results for those tokens are compared with it.  Codes are expected to agree bit for bit;
    any mismatch is counted, with the share whose projected coordinate is below 1e-6 in magnitude."""
    from oracle import oracle as O

    w = WORKLOADS[args.workload]
    n = min(args.cpu_tokens, x.shape[0])
    T, k = w["T"], w["k"]
    bf16 = x.dtype == torch.bfloat16

    def host(t):
        t = t[:n] if t.shape[0] == x.shape[0] else t
        if t.dtype == torch.bfloat16:
            return t.view(torch.int16).cpu().numpy().view(np.uint16)
        return t.cpu().numpy()

    xs = host(x)
    x32 = O.bf16_bits_to_f32(xs) if bf16 else xs
    z = O.project(x32, signs.cpu().numpy(), T * k, had_scale=hs, mix_a=1.0, mix_b=0.0)
    wm = {"score": O.WEIGHT_SCORE, "ones": O.WEIGHT_ONES}[w["weight_mode"]]
    bo = {"msb": O.MSB_FIRST, "lsb": O.LSB_FIRST}[w["bit_order"]]
    idx_ref, w_ref = O.code_weights(z, T, k, bit_order=bo, weight_mode=wm)
    idx_gpu, w_gpu = host(idx), host(wgt)
    bad = idx_gpu != idx_ref
    tiny = 0
    if bad.any():
        zmin = np.abs(z.reshape(n, T, k)).min(-1)
        tiny = int((zmin[bad] < 1e-6).sum())
    y_ref = O.gather(idx_ref, w_gpu, host(tables), out_bf16=bf16)
    y_gpu = host(y)
    if bf16:
        y_ref, y_gpu = O.bf16_bits_to_f32(y_ref), O.bf16_bits_to_f32(y_gpu)
    return {"tokens": int(n), "hash_codes_checked": int(idx_ref.size), "hash_code_mismatches": int(bad.sum()),
            "mismatches_with_abs_v_below_1e-6": tiny,
            "weights_max_rel_err": float(np.abs(w_gpu - w_ref).max() / np.abs(w_ref).max()),
            "output_max_rel_err": float(np.abs(y_gpu - y_ref).max() / np.abs(y_ref).max()),
            "outputs_bit_identical_given_gpu_weights": bool(np.array_equal(y_gpu, y_ref))}


def cpu_path(args, budget_s):
    """Times the layer forward on the host: projection = CPU restatement (the reference's CPU BH4 needs
    libxsmm, which is not available), code+score and gather = the reference's own C++ extensions when
    oracle/_ref holds them, else the oracle port.  Sample: `cpu_tokens` tokens of the same workload,
    fp32 copies of the tables (the reference's CPU kernels are fp32 only)."""
    from oracle import oracle as O

    w = WORKLOADS[args.workload]
    Ns = args.cpu_tokens
    T, k, D = w["T"], w["k"], padded_dim(w["d_in"])
    R = max(1, -(-T * k // D))
    rng = np.random.RandomState(7)
    x = rng.randn(Ns, w["d_in"]).astype(np.float32)
    tables = (0.02 * rng.randn(T << k, w["d_out"])).astype(np.float32)
    signs = (2.0 * rng.randint(0, 2, size=(R, 2, D, 1, 1)) - 1.0).astype(np.float32)
    cores = os.cpu_count()
    torch.set_num_threads(cores)
    O.set_threads(cores)
    ref = load_ref_modules()
    kind = "reference" if ref is not None else "port"
    hs = float(1.0 / np.sqrt(D))
    offsets = (torch.arange(T, dtype=torch.int32) << k)[None]
    tt = torch.from_numpy(tables)

    def one():
        z = O.project(x, signs, T * k, had_scale=hs, mix_a=1.0, mix_b=0.0)
        if ref is not None:
            zt = torch.from_numpy(z).reshape(Ns, T, k)
            codes = torch.empty(Ns, T, dtype=torch.int32)
            scores = torch.empty(Ns, T, dtype=torch.float32)
            ref["ccs_cpu"].compute_code_score(zt, codes, scores)
            return ref["gather_add_cpu"].weighted_vector_gather_add_avx2_par(codes + offsets, tt, scores)
        idx, wg = O.code_weights(z, T, k)
        return O.gather(idx, wg, tables)

    one()
    times = []
    t_all = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_all < budget_s and len(times) < 50):
        t0 = time.perf_counter()
        one()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": Ns / med, "unit": "tokens/s", "cores": cores, "kind": kind,
            "sample": f"{Ns} tokens of workload {args.workload} (fp32 tables), median of {len(times)} passes; "
                      f"projection = C restatement, code+score and gather = "
                      f"{'reference C++ extensions (oracle/_ref)' if ref is not None else 'oracle port'}",
            "ms_per_pass": med * 1e3}


def reference_cpu_own_shape(local):
    """The reference's CPU inference path on the one shape its CPU kernels are written for (bh4/cpu/kernel.py:57-62,
    gather/cpu/kernel.py:73-76: 64 x 512 tokens, hidden 512, 128 tables of 256 rows, 64 x 64 blocks) -- its three C++
    extensions compiled unmodified (the BH4 one against a stand-in libxsmm header: plain-loop GEMM) -- timed on
    this box's host cores beside this library's layer forward on the same shape on the GPU."""
    from lookupffn_b200 import ops
    from oracle import build as obuild

    mods = {n: obuild.load_ref_module(n) for n in ("sbdht_cpu", "ccs_cpu", "gather_add_cpu")}
    if any(m is None for m in mods.values()):
        return None
    N, D, BS, T, k, d = 64 * 512, 512, 64, 128, 8, 512
    R = T * k // D
    g = torch.Generator().manual_seed(11)
    x = torch.randn(N, D, generator=g)
    w = torch.randn(R, 4, D // BS, BS, BS, generator=g) / float(np.sqrt(BS * D))
    tables = 0.02 * torch.randn(T << k, d, generator=g)
    offsets = (torch.arange(T, dtype=torch.int32) << k)[None]
    cores = os.cpu_count()
    torch.set_num_threads(cores)
    # the extension announces itself on the C++ side's stdout; this program's stdout carries one JSON line only
    sys.stdout.flush()
    saved = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    try:
        os.dup2(devnull, 1)
        mods["sbdht_cpu"].setup_xsmm_kernel_float_avx2(BS, BS, BS, D, BS, D)
    finally:
        os.dup2(saved, 1)
        os.close(saved)
        os.close(devnull)

    def one():
        outs = []
        for r in range(R):  # bh4/cpu/kernel.py:45-52
            xc = x.clone()
            mods["sbdht_cpu"].sbdht(xc, w[r])
            outs.append(xc)
        z = 0.7 * torch.cat(outs, dim=-1) + (1 - 0.7) * x.repeat(1, R)  # lookup.py:36-37 (bias is zero at init)
        codes = torch.empty(N, T, dtype=torch.int32)
        scores = torch.empty(N, T, dtype=torch.float32)
        mods["ccs_cpu"].compute_code_score(z.reshape(N, T, k), codes, scores)
        return mods["gather_add_cpu"].weighted_vector_gather_add_avx2_par(codes + offsets, tables, scores)

    one()
    times = []
    for _ in range(3):
        t0 = time.perf_counter()
        one()
        times.append(time.perf_counter() - t0)
    cpu_s = statistics.median(times)
    # the same layer on the GPU: CPU convention of the projection (x . W per block, H / D)
    device = torch.device("cuda", local)
    xd, wd, td = x.to(device), w.to(device), tables.to(device)
    desc = ops.make_hash_desc(D, wd, None, T, k, transpose_w=True, had_scale=1.0 / D, mix_a=0.7, mix_b=1 - 0.7)
    for _ in range(3):
        ops.layer_fwd(xd, desc, td)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        y = ops.layer_fwd(xd, desc, td)
    e1.record()
    torch.cuda.synchronize()
    gpu_s = e0.elapsed_time(e1) * 1e-3 / 10
    return {"shape": f"N={N}, hidden {D}, T={T}, k={k}, d_out={d}, bh4 64x64, fp32: the only shape the reference's CPU "
                     "kernels accept", "reference_cpu_tokens_per_s": N / cpu_s, "reference_cpu_ms": cpu_s * 1e3,
            "cores": cores, "sample": "whole shape, median of 3 passes; BH4 GEMM = stand-in for libxsmm (plain loops)",
            "this_library_gpu_tokens_per_s": N / gpu_s, "this_library_gpu_ms": gpu_s * 1e3}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    w = dict(WORKLOADS[args.workload])
    if args.tokens:
        w["N"] = args.tokens
    per_step = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    base = None
    vals = []
    for i in range(args.warmup + args.steps):
        base = cpu_path(args, per_step)
        if i >= args.warmup:
            vals.append(base["value"])
    v = statistics.median(vals)
    base = dict(base, value=v)
    return {
        "impl": "reference", "metric": "lookupffn_layer_forward_throughput", "value": v, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": args.cpu_tokens / v * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(layer_config(args, w, world),
                       reference_arm=f"the reference's CPU path on {base['cores']} host cores; each step is a bounded sample "
                                     f"of {args.cpu_tokens} tokens of this workload with fp32 tables (its CPU kernels are "
                                     "fp32 only)"),
        "cpu_baseline": base,
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS) + ["c2enc", "c4", "train"])
    ap.add_argument("--projection", default="bh4", choices=["bh4", "sign_hadamard", "dense"],
                    help="projection of the c2enc workload (bh4 = the reference configs)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-chunk", type=int, default=4736,
                    help="tokens per chunk of the host-buffer call; 4736 = two resident waves of the gather kernel "
                         "(148 SMs x 16 warps each); the call itself halves the first two and the last two chunks")
    ap.add_argument("--cpu-tokens", type=int, default=4096)
    ap.add_argument("--shard", default="tokens", choices=["tokens", "tables"],
                    help="tokens: each rank its own tokens, tables replicated (default); tables: tables split by T, "
                         "partial sums reduce-scattered")
    ap.add_argument("--rs-chunk", type=int, default=32768, help="tokens per reduce-scatter chunk (--shard tables)")
    ap.add_argument("--rs", default="nccl", choices=["nccl", "fused", "fused-store", "copy"],
                    help="--shard tables: combine partial sums with NCCL reduce-scatter, or inside the gather kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--table-sharded-ks", default="",
                    help="comma-separated config-5 workloads of the table-sharded record (default: c5k8, plus c5k12 and "
                         "c5k6 at 8 GPUs)")
    ap.add_argument("--no-table-sharded", action="store_true",
                    help="skip the short table-sharded run appended to the line when more than one GPU runs")
    ap.add_argument("--no-encoder", action="store_true", help="skip the short config-2 encoder run appended at N=1")
    ap.add_argument("--tokens", type=int, default=0, help="override tokens per GPU (profiling on a small case)")
    ap.add_argument("--no-e2e", action="store_true", help="device path only, short report (for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        out = run_reference(args, rank, world)
        if out is not None:
            print(json.dumps(out), flush=True)
        return 0

    if world > 1 or args.shard == "tables":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29512")
        torch.cuda.set_device(local)
        torch.distributed.init_process_group("nccl", rank=rank, world_size=world,
                                             device_id=torch.device("cuda", local))
    if args.workload in ("c2enc", "c4", "train"):
        out = {"c2enc": run_encoder, "c4": run_train_gather, "train": run_train_layer}[args.workload](args, rank, world, local)
        if out is not None:
            print(json.dumps(out), flush=True)
        if world > 1:
            torch.distributed.destroy_process_group()
        return 0
    if args.shard == "tables":
        out = run_table_sharded(args, rank, world, local)
        if out is not None:
            print(json.dumps(out), flush=True)
        torch.distributed.destroy_process_group()
        return 0
    out = run_ours(args, rank, world, local)
    if world > 1 and args.workload == "c3" and not args.tokens and not args.no_table_sharded:
        # the other multi-GPU mode (tables sharded, reduce-scatter over NVLink), a short run appended to the line
        torch.cuda.empty_cache()
        try:
            ts = table_sharded_record(args, rank, world, local)
        except Exception as e:  # the headline line is printed regardless
            ts = {"error": repr(e)}
        if out is not None:
            out["table_sharded"] = ts
    if out is not None:
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_path(args, 15.0)
            if args.workload == "c3" and not args.tokens:
                out["cpu_baseline"]["reference_cpu_path_on_its_own_shape"] = reference_cpu_own_shape(local)
        if world == 1 and args.workload == "c3" and not args.tokens and not args.no_encoder:
            # the second half of the headline metric: RoBERTa-small encoder inference (config 2), a short run
            enc_args = argparse.Namespace(**vars(args))
            enc_args.steps, enc_args.warmup = 10, 3
            enc = run_encoder(enc_args, rank, world, local)
            out["roberta_small_encoder"] = {"value": enc["value"], "unit": enc["unit"], "ms_per_step": enc["ms_per_step"],
                                            "e2e": enc["e2e"]["value"], "steps": 10, "config": enc["config"]["workload"],
                                            "with_bf16_autocast_around_the_ffn":
                                                enc["with_bf16_autocast_around_the_ffn"]["value"],
                                            "gpu_comparator": enc["gpu_comparator"]}
            # and a short run of benchmark configuration 4 (training-mode gather, forward + backward) beside the
            # reference's own CUDA kernels on the same tensors
            torch.cuda.empty_cache()
            c4_args = argparse.Namespace(**vars(args))
            c4_args.steps, c4_args.warmup = 3, 3
            c4 = run_train_gather(c4_args, rank, world, local)
            out["training_gather_c4"] = {k: c4[k] for k in ("value", "unit", "ms_per_step", "kernels_ms",
                                                            "algorithmic_GBps", "gpu_comparator", "steps")}
            out["training_gather_c4"]["config"] = c4["config"]["workload"]
            torch.cuda.empty_cache()
            out["training_step_reference_layer_shape"] = run_train_layer(c4_args, rank, world, local)
        print(json.dumps(out), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
