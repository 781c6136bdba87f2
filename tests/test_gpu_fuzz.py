"""Seeded random-shape sweep of every kernel against the CPU oracle (through the C ABI): ragged sizes, odd
index counts, every code length 1..16, every weight mode, both bit orders, both weight layouts, bf16 and fp32
storage, table sub-ranges.  Bars as in test_gpu_parity.py: projections, codes and gather outputs bit-exact,
weights 1e-5, weight gradient 1e-4, reduction table gradient 1e-5, sorted table gradient bit-exact."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def t2n(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.cpu().numpy()


@pytest.mark.parametrize("seed", [1, 2])
def test_random_shapes_against_oracle(seed):
    from lookupffn_b200 import _lib as L
    from lookupffn_b200 import ops

    dev = torch.device("cuda:0")
    rng = np.random.RandomState(seed)
    failures = []

    def bf(bits):
        return torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.bfloat16)

    def check(name, cond, info):
        if not cond:
            failures.append((name, info))

    # ---- gather forward, weight gradient, reduction table gradient
    for _ in range(40):
        bf16 = rng.rand() < 0.5
        d = int(rng.choice([4, 8, 12, 64, 100, 512, 768, 1000, 1024, 1536, 2048, 3072, 4100])) * (2 if bf16 else 1)
        if bf16:
            d = (d // 8) * 8 or 8
        N, I, S = int(rng.randint(1, 200)), int(rng.randint(0, 300)), int(rng.randint(1, 3000))
        idx = rng.randint(0, S, size=(N, I)).astype(np.int32)
        w = rng.randn(N, I).astype(np.float32)
        tab = (0.02 * rng.randn(S, d)).astype(np.float32)
        bias = rng.randn(d).astype(np.float32)
        if bf16:
            tref = O.f32_to_bf16_bits(tab)
            tt = bf(tref)
        else:
            tref, tt = tab, torch.from_numpy(tab).to(dev)
        ti, tw, tbias = (torch.from_numpy(a).to(dev) for a in (idx, w, bias))
        y = ops.weighted_vector_gather_add(ti, tt, tw, bias=tbias)
        check("gather", np.array_equal(t2n(y), O.gather(idx, w, tref, bias=bias, out_bf16=bf16)), (N, I, S, d, bf16))
        if I > 0:
            dy = rng.randn(N, d).astype(np.float32)
            tg = torch.from_numpy(dy).to(dev)
            dw, ref = t2n(ops.indexed_inner_product(ti, tg, tt)), O.gather_bwd_weights(idx, dy, tref)
            check("dw", np.abs(dw - ref).max() <= 1e-4 * max(np.abs(ref).max(), 1e-20), (N, I, S, d, bf16))
            dt, ref = t2n(ops.weighted_vector_scatter_add(ti, tg, tw, S)), O.gather_bwd_tables(idx, w, dy, S)
            check("dt_red", np.abs(dt - ref).max() <= 1e-5 * max(np.abs(ref).max(), 1e-20), (N, I, S, d))
    # ---- sorted table gradient
    for _ in range(15):
        N, T, m = int(rng.randint(1, 600)), int(rng.randint(1, 12)), int(rng.choice([1, 2, 9]))
        rows, d = int(rng.choice([2, 16, 64, 256, 1024, 4096])), int(rng.choice([4, 64, 768, 1024]))
        idx = (rng.randint(0, rows, size=(N, T, m)) + (np.arange(T) * rows)[None, :, None]).astype(np.int32).reshape(N, T * m)
        w, dy = rng.randn(N, T * m).astype(np.float32), rng.randn(N, d).astype(np.float32)
        out = t2n(ops.weighted_vector_scatter_add(*(torch.from_numpy(a).to(dev) for a in (idx, dy, w)), T * rows,
                                                  structure=(T, m, rows)))
        check("dt_sorted", np.array_equal(out, O.gather_bwd_tables(idx, w, dy, T * rows)), (N, T, m, rows, d))
    # ---- hashing
    for _ in range(50):
        D = int(rng.choice([64, 128, 256, 512, 1024, 2048]))
        d_in = int(rng.randint(D // 2 + 1, D + 1))
        k, T, N = int(rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 12, 16])), int(rng.randint(1, 600)), int(rng.randint(1, 70))
        BS = int(rng.choice([1, 1, 1, 4, 16, 64]))
        if BS > 1 and D > 1024:
            D, d_in = 1024, min(d_in, 1024)
        S, R = int(rng.choice([1, 2, 4])), max(1, -(-T * k // D))
        wm, bo = int(rng.choice([0, 1, 2])), int(rng.choice([0, 1]))
        tw = bool(rng.rand() < 0.5) if BS > 1 else False
        mix = (0.7, 0.3) if rng.rand() < 0.5 else (1.0, 0.0)
        hs = float(rng.choice([1.0, 0.125, 1 / np.sqrt(D)]))
        bf16 = rng.rand() < 0.3
        NB = D // BS
        # diagonals: signs (the reference's use) or, one time in three, arbitrary floats (every product rounded)
        wt = ((2.0 * rng.randint(0, 2, size=(R, S, NB, BS, BS)) - 1.0) * (rng.rand(R, S, NB, BS, BS) + 0.5 if rng.rand() < 0.33 else 1.0)
              if BS == 1 else rng.randn(R, S, NB, BS, BS) / np.sqrt(BS * D) * 3).astype(np.float32)
        bias = (0.05 * rng.randn(T * k)).astype(np.float32) if rng.rand() < 0.7 else None
        x = rng.randn(N, d_in).astype(np.float32)
        if bf16:
            xb = O.f32_to_bf16_bits(x)
            xt, xr = bf(xb), O.bf16_bits_to_f32(xb)
        else:
            xt, xr = torch.from_numpy(x).to(dev), x
        info = (N, d_in, D, BS, S, T, k, wm, bo, tw, mix, hs, bf16, bias is not None)
        z_ref = O.project(xr, wt, T * k, transpose_w=tw, had_scale=hs, mix_a=mix[0], mix_b=mix[1], bias=bias)
        idx_ref, w_ref = O.code_weights(z_ref, T, k, bit_order=bo, weight_mode=wm, tau=0.5)
        desc = ops.make_hash_desc(d_in, torch.from_numpy(wt).to(dev), None if bias is None else torch.from_numpy(bias).to(dev),
                                  T, k, transpose_w=tw, had_scale=float(np.float32(hs)), mix_a=mix[0], mix_b=mix[1],
                                  bit_order=bo, weight_mode=wm, tau=0.5)
        tb_ = int(rng.randint(0, T))
        tc_ = int(rng.randint(1, T - tb_ + 1))
        idx, wg, z = ops.hash_fwd(xt, desc, t_begin=tb_, t_count=tc_, want_z=True)
        m = k + 1 if wm == 2 else 1
        check("hash z", np.array_equal(t2n(z), z_ref[:, tb_ * k:(tb_ + tc_) * k]), info)
        check("hash idx", np.array_equal(t2n(idx), idx_ref[:, tb_ * m:(tb_ + tc_) * m] - tb_ * (1 << k)), info)
        wr = w_ref[:, tb_ * m:(tb_ + tc_) * m]
        check("hash w", np.abs(t2n(wg) - wr).max() <= 1e-5 * max(np.abs(wr).max(), 1e-20), info)
        # the same request without z takes other kernels (codes straight from registers, mix folded into the code
        # step): same codes, same weights
        idx2, wg2, _ = ops.hash_fwd(xt, desc, t_begin=tb_, t_count=tc_)
        check("hash idx (no z)", np.array_equal(t2n(idx2), t2n(idx)), info)
        check("hash w (no z)", np.abs(t2n(wg2) - wr).max() <= 1e-5 * max(np.abs(wr).max(), 1e-20), info)
    assert L.device_status(dev) == 0
    assert not failures, failures[:5]
