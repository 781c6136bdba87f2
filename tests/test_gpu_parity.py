"""Parity of the CUDA kernels (called through the C ABI of liblookupffn.so) with the CPU oracle
and the reference-generated golden vectors.  Bars: hash codes / row indices bit-exact; projected
coordinates z bit-exact (same butterfly order and fmaf chains); gather outputs bit-exact for fp32
and bf16 storage (one fmaf chain per column); weights (expf) within 1e-5 relative; gradient of the
weights within 1e-4 relative (different reduction order); sorted table gradient bit-exact, vector-
reduction table gradient within 1e-5 relative."""
from argparse import Namespace

import numpy as np
import pytest
import torch

from oracle import oracle as O
from oracle import parity as PAR

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from lookupffn_b200 import _lib

    _lib.lib()  # fail here, loudly, if the CUDA library was not built
    return torch.device("cuda:0")


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)


def t2n(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def bf16_tensor(bits, dev):
    return torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.bfloat16)


# ---- Hadamard ------------------------------------------------------------------------------------
@pytest.mark.parametrize("D", [32, 64, 128, 256, 512, 1024, 2048])
def test_fwht_bit_exact(dev, D):
    from lookupffn_b200 import ops

    rng = np.random.RandomState(D)
    for N in (1, 13, 300):
        x = rng.randn(N, D).astype(np.float32)
        y = ops.hadamard(torch.from_numpy(x).to(dev))
        np.testing.assert_array_equal(t2n(y), O.fwht(x))
    x = rng.randn(9, D).astype(np.float32)
    y = ops.hadamard(torch.from_numpy(x).to(dev), scale=0.125)
    np.testing.assert_array_equal(t2n(y), O.fwht(x, 0.125))
    # bf16 storage: widen exactly, transform in fp32, round once
    xb = O.f32_to_bf16_bits(x)
    yb = ops.hadamard(bf16_tensor(xb, dev))
    np.testing.assert_array_equal(t2n(yb), O.f32_to_bf16_bits(O.fwht(O.bf16_bits_to_f32(xb))))


def test_fwht_matches_reference_golden(dev, golden):
    from lookupffn_b200 import ops

    for D in (64, 256, 1024):
        y = ops.hadamard(torch.from_numpy(golden[f"had_{D}_x"]).to(dev))
        assert rel_err(t2n(y), golden[f"had_{D}_y"]) < 1e-5  # reference = fp32 matmul with H


# ---- hashing ---------------------------------------------------------------------------------------
def make_proj(rng, D, BS, S, R, signs):
    NB = D // BS
    if signs:
        return (2.0 * rng.randint(0, 2, size=(R, S, NB, BS, BS)) - 1.0).astype(np.float32)
    return (rng.randn(R, S, NB, BS, BS) / np.sqrt(BS * D)).astype(np.float32)


HASH_CASES = [
    # N, d_in, D, BS, S, T, k, weight_mode, bit_order, had_scale, mix
    (37, 100, 128, 1, 2, 50, 6, O.WEIGHT_SCORE, O.MSB_FIRST, 1.0, (0.7, 0.3)),      # tables straddle rotations
    (64, 128, 128, 1, 2, 64, 8, O.WEIGHT_ONES, O.LSB_FIRST, 2.0 ** -7, (1.0, 0.0)),  # sign-diagonal, LSB, ones
    (33, 512, 512, 1, 2, 128, 8, O.WEIGHT_ONES, O.LSB_FIRST, 1.0 / np.sqrt(512), (1.0, 0.0)),  # benchmark config 1
    (20, 768, 1024, 1, 2, 512, 8, O.WEIGHT_SCORE, O.MSB_FIRST, 1.0 / 32, (1.0, 0.0)),  # benchmark config 3
    (9, 768, 1024, 1, 2, 100, 10, O.WEIGHT_SCORE, O.MSB_FIRST, 1.0, (0.7, 0.3)),
    (9, 300, 512, 1, 4, 90, 12, O.WEIGHT_SCORE, O.LSB_FIRST, 1.0, (0.7, 0.3)),
    (5, 64, 64, 1, 2, 40, 1, O.WEIGHT_SCORE, O.MSB_FIRST, 1.0, (0.7, 0.3)),
    (5, 200, 256, 1, 2, 30, 16, O.WEIGHT_ONES, O.MSB_FIRST, 1.0, (0.7, 0.3)),
    (7, 1500, 2048, 1, 2, 300, 8, O.WEIGHT_SCORE, O.MSB_FIRST, 1.0, (0.7, 0.3)),
    (40, 100, 128, 1, 2, 30, 8, O.WEIGHT_SOFT_FLIP, O.MSB_FIRST, 1.0 / 8, (1.0, 0.0)),  # benchmark config 4 weights
    (11, 100, 128, 1, 2, 21, 6, O.WEIGHT_SOFT_FLIP, O.LSB_FIRST, 1.0 / 8, (1.0, 0.0)),
    # block-diagonal projection (the reference's BH4)
    (70, 512, 512, 64, 4, 128, 8, O.WEIGHT_SCORE, O.MSB_FIRST, 1.0, (0.7, 0.3)),    # reference config t128
    (33, 768, 1024, 64, 4, 160, 8, O.WEIGHT_SCORE, O.MSB_FIRST, 1.0, (0.7, 0.3)),
    (40, 100, 128, 64, 4, 50, 6, O.WEIGHT_SCORE, O.MSB_FIRST, 1.0, (0.7, 0.3)),
    (10, 60, 64, 16, 4, 20, 8, O.WEIGHT_ONES, O.LSB_FIRST, 1.0, (0.7, 0.3)),
    (10, 250, 256, 128, 2, 40, 10, O.WEIGHT_SCORE, O.MSB_FIRST, 1.0, (0.7, 0.3)),
    (6, 256, 256, 4, 4, 64, 8, O.WEIGHT_SOFT_FLIP, O.MSB_FIRST, 1.0, (0.7, 0.3)),
]


@pytest.mark.parametrize("case", HASH_CASES, ids=[f"c{i}" for i in range(len(HASH_CASES))])
@pytest.mark.parametrize("transpose_w", [False, True])
def test_hash_fwd_matches_oracle(dev, case, transpose_w):
    from lookupffn_b200 import ops

    N, d_in, D, BS, S, T, k, wm, bo, hs, mix = case
    if BS == 1 and transpose_w:
        pytest.skip("a diagonal has no transpose")
    rng = np.random.RandomState(N * 1000 + T)
    R = max(1, -(-T * k // D))
    w = make_proj(rng, D, BS, S, R, signs=(BS == 1))
    bias = (0.05 * rng.randn(T * k)).astype(np.float32)
    x = rng.randn(N, d_in).astype(np.float32)
    z_ref = O.project(x, w, T * k, transpose_w=transpose_w, had_scale=hs, mix_a=mix[0], mix_b=mix[1], bias=bias)
    idx_ref, w_ref = O.code_weights(z_ref, T, k, bit_order=bo, weight_mode=wm, tau=0.5)

    wt, bt = torch.from_numpy(w).to(dev), torch.from_numpy(bias).to(dev)
    desc = ops.make_hash_desc(d_in, wt, bt, T, k, transpose_w=transpose_w, had_scale=float(np.float32(hs)),
                              mix_a=mix[0], mix_b=mix[1], bit_order=bo, weight_mode=wm, tau=0.5)
    idx, wgt, z = ops.hash_fwd(torch.from_numpy(x).to(dev), desc, want_z=True)
    np.testing.assert_array_equal(t2n(z), z_ref)           # projected coordinates: bit-exact
    np.testing.assert_array_equal(t2n(idx), idx_ref)       # codes + offsets: bit-exact
    assert rel_err(t2n(wgt), w_ref) < 1e-5                 # weights: expf accuracy
    # a sub-range of tables (what a table-sharded rank computes) equals the slice of the whole
    m = k + 1 if wm == O.WEIGHT_SOFT_FLIP else 1
    tb, tc = T // 3, T - T // 3 - 1
    idx_s, w_s, z_s = ops.hash_fwd(torch.from_numpy(x).to(dev), desc, t_begin=tb, t_count=tc, want_z=True)
    np.testing.assert_array_equal(t2n(z_s), z_ref[:, tb * k:(tb + tc) * k])
    np.testing.assert_array_equal(t2n(idx_s), idx_ref[:, tb * m:(tb + tc) * m] - tb * (1 << k))
    np.testing.assert_array_equal(t2n(w_s), t2n(wgt)[:, tb * m:(tb + tc) * m])


BLOCK64_CASES = [
    # N, d_in, D, T, k, weight_mode: the 64 x 64 fast kernel without z_out, many work units per CTA
    (6500, 512, 512, 192, 8, O.WEIGHT_SCORE),      # input tile resident, mix folded into the code step, 3 rotations
    (5000, 500, 512, 150, 6, O.WEIGHT_SCORE),      # k does not divide D: carry rows, whole tiles per CTA
    (300, 256, 256, 100, 8, O.WEIGHT_ONES),        # 256-thread variant, 4 rotations
    (4200, 768, 1024, 256, 8, O.WEIGHT_SCORE),     # D = 1024: no resident tile, two passes per stage
    (700, 512, 512, 24, 8, O.WEIGHT_SOFT_FLIP),    # k + 1 candidates per table (scalar stores)
]


@pytest.mark.parametrize("case", BLOCK64_CASES, ids=[f"b{i}" for i in range(len(BLOCK64_CASES))])
def test_hash_block64_without_z_matches_oracle(dev, case):
    """The paths of the 64 x 64 kernel that only run when z itself is not asked for, on enough tokens that every
    CTA walks several (tile, rotation) units and its weight-chunk ring wraps many times."""
    from lookupffn_b200 import _lib, ops

    N, d_in, D, T, k, wm = case
    rng = np.random.RandomState(N + T)
    R = max(1, -(-T * k // D))
    w = make_proj(rng, D, 64, 4, R, signs=False)
    bias = (0.05 * rng.randn(T * k)).astype(np.float32)
    x = rng.randn(N, d_in).astype(np.float32)
    z_ref = O.project(x, w, T * k, transpose_w=True, had_scale=1.0, mix_a=0.7, mix_b=0.3, bias=bias)
    idx_ref, w_ref = O.code_weights(z_ref, T, k, bit_order=O.MSB_FIRST, weight_mode=wm, tau=0.5)
    desc = ops.make_hash_desc(d_in, torch.from_numpy(w).to(dev), torch.from_numpy(bias).to(dev), T, k, transpose_w=True,
                              mix_a=0.7, mix_b=0.3, weight_mode=wm, tau=0.5)
    xd = torch.from_numpy(x).to(dev)
    idx, wgt, _ = ops.hash_fwd(xd, desc)
    np.testing.assert_array_equal(t2n(idx), idx_ref)
    assert rel_err(t2n(wgt), w_ref) < 1e-5
    # a table sub-range starting inside a rotation
    m = k + 1 if wm == O.WEIGHT_SOFT_FLIP else 1
    tb, tc = T // 3 + 1, T - T // 3 - 2
    idx_s, w_s, _ = ops.hash_fwd(xd, desc, t_begin=tb, t_count=tc)
    np.testing.assert_array_equal(t2n(idx_s), idx_ref[:, tb * m:(tb + tc) * m] - tb * (1 << k))
    np.testing.assert_array_equal(t2n(w_s), t2n(wgt)[:, tb * m:(tb + tc) * m])
    assert _lib.device_status(dev) & _lib.STATUS_TIMEOUT == 0


@pytest.mark.parametrize("D,k,mix_a", [(256, 4, 1.0), (512, 8, 1.0), (1024, 8, 0.7), (1024, 6, 1.0), (512, 16, 0.9)])
def test_hash_diagonal_with_general_weights(dev, D, k, mix_a):
    """A diagonal projection whose entries are arbitrary floats, not signs, with a scale that is no power of two and
    a bias: every product is rounded before it is added (no contraction into a fused multiply-add anywhere), so z
    and the codes equal the oracle bit for bit, with z (vector layout) and without (transposing layout)."""
    from lookupffn_b200 import ops

    rng = np.random.RandomState(D + k)
    N, d_in, T = 300, D - 3, (2 * D) // k
    R = max(1, -(-T * k // D))
    w = rng.randn(R, 2, D, 1, 1).astype(np.float32)
    bias = (0.05 * rng.randn(T * k)).astype(np.float32)
    x = rng.randn(N, d_in).astype(np.float32)
    hs = float(np.float32(1.0 / np.sqrt(D) * 0.9))
    z_ref = O.project(x, w, T * k, had_scale=hs, mix_a=mix_a, mix_b=0.0, bias=bias)
    idx_ref, w_ref = O.code_weights(z_ref, T, k)
    desc = ops.make_hash_desc(d_in, torch.from_numpy(w).to(dev), torch.from_numpy(bias).to(dev), T, k, had_scale=hs,
                              mix_a=mix_a, mix_b=0.0)
    xd = torch.from_numpy(x).to(dev)
    idx, wgt, _ = ops.hash_fwd(xd, desc)
    np.testing.assert_array_equal(t2n(idx), idx_ref)
    assert rel_err(t2n(wgt), w_ref) < 1e-5
    idx2, wgt2, z = ops.hash_fwd(xd, desc, want_z=True)
    np.testing.assert_array_equal(t2n(z), z_ref)
    np.testing.assert_array_equal(t2n(idx2), idx_ref)


@pytest.mark.parametrize("D,k", [(1024, 8), (512, 8), (256, 8), (1024, 16), (512, 16)])
def test_hash_soft_flip_candidates_without_z(dev, D, k):
    """k + 1 candidates per table from the transposing kernel (whole rotations leave through per-warp staging buffers
    as 16-byte stores; partial ranges and unaligned rows take the scalar stores): codes exact, weights 1e-5."""
    from lookupffn_b200 import ops

    rng = np.random.RandomState(D + k)
    N, d_in = 77, D - 5
    T = (3 * D) // k            # three rotations
    w = make_proj(rng, D, 1, 2, 3, signs=True)
    bias = (0.05 * rng.randn(T * k)).astype(np.float32)
    x = rng.randn(N, d_in).astype(np.float32)
    hs = float(np.float32(1.0 / np.sqrt(D)))
    z_ref = O.project(x, w, T * k, had_scale=hs, mix_a=1.0, mix_b=0.0, bias=bias)
    idx_ref, w_ref = O.code_weights(z_ref, T, k, weight_mode=O.WEIGHT_SOFT_FLIP, tau=0.5)
    desc = ops.make_hash_desc(d_in, torch.from_numpy(w).to(dev), torch.from_numpy(bias).to(dev), T, k, had_scale=hs,
                              mix_a=1.0, mix_b=0.0, weight_mode=O.WEIGHT_SOFT_FLIP, tau=0.5)
    xd = torch.from_numpy(x).to(dev)
    m = k + 1
    idx, wgt, _ = ops.hash_fwd(xd, desc)
    np.testing.assert_array_equal(t2n(idx), idx_ref)
    assert rel_err(t2n(wgt), w_ref) < 1e-5
    for tb, tc in ((1, T - 2), (D // k, D // k), (4, T - 4)):  # ragged ends, exactly the middle rotation, aligned start
        idx_s, w_s, _ = ops.hash_fwd(xd, desc, t_begin=tb, t_count=tc)
        np.testing.assert_array_equal(t2n(idx_s), idx_ref[:, tb * m:(tb + tc) * m] - tb * (1 << k))
        np.testing.assert_array_equal(t2n(w_s), t2n(wgt)[:, tb * m:(tb + tc) * m])


def test_hash_bf16_input(dev):
    from lookupffn_b200 import ops

    rng = np.random.RandomState(5)
    N, d_in, D, T, k = 50, 768, 1024, 512, 8
    w = make_proj(rng, D, 1, 2, 4, signs=True)
    xb = O.f32_to_bf16_bits(rng.randn(N, d_in).astype(np.float32))
    z_ref = O.project(O.bf16_bits_to_f32(xb), w, T * k, had_scale=1 / 32, mix_a=1.0, mix_b=0.0)
    idx_ref, w_ref = O.code_weights(z_ref, T, k)
    desc = ops.make_hash_desc(d_in, torch.from_numpy(w).to(dev), None, T, k, had_scale=1 / 32, mix_a=1.0, mix_b=0.0)
    idx, wgt, z = ops.hash_fwd(bf16_tensor(xb, dev), desc, want_z=True)
    np.testing.assert_array_equal(t2n(z), z_ref)
    np.testing.assert_array_equal(t2n(idx), idx_ref)
    assert rel_err(t2n(wgt), w_ref) < 1e-5


@pytest.mark.parametrize("tag,T,k", [("k8", 12, 8), ("k6", 10, 6), ("k10", 5, 10), ("k1", 4, 1)])
def test_code_weights_matches_reference_golden(dev, golden, tag, T, k):
    from lookupffn_b200 import ops

    z = torch.from_numpy(golden[f"ccs_{tag}_z"]).to(dev)
    code, score = ops.compute_code_score(z)
    np.testing.assert_array_equal(t2n(code), golden[f"ccs_{tag}_code_torch"])
    np.testing.assert_array_equal(t2n(code), golden[f"ccs_{tag}_code_cpp"])
    assert rel_err(t2n(score), golden[f"ccs_{tag}_score_cpp"]) < 1e-5


def test_code_edge_values(dev):
    from lookupffn_b200 import ops

    z = torch.tensor([[[0.0, -0.0, float("nan"), 1e-45, -1e-45, float("inf"), -float("inf"), 3.0]]], device=dev)
    code, _ = ops.compute_code_score(z, weight_mode=O.WEIGHT_ONES)
    assert int(code[0, 0]) == 0b00010101
    code, _ = ops.compute_code_score(z, weight_mode=O.WEIGHT_ONES, bit_order=O.LSB_FIRST)
    assert int(code[0, 0]) == 0b10101000


def test_bh4_matches_reference_golden(dev, golden):
    from lookupffn_b200 import ops
    from lookupffn_b200.lookup import BH4

    for tag in ("a", "b", "c", "d"):
        in_dim, out_dim, BS, D, R = [int(v) for v in golden[f"bh4_{tag}_meta"]]
        x = golden[f"bh4_{tag}_x"]
        w = torch.from_numpy(golden[f"bh4_{tag}_w"]).to(dev)
        xp = np.zeros((x.shape[0], D), dtype=np.float32)
        xp[:, :in_dim] = x
        P = ops.bh4(torch.from_numpy(xp).to(dev), w)
        assert rel_err(t2n(P), golden[f"bh4_{tag}_P"]) < 2e-5   # reference = torch einsum + matmul with H
        mod = BH4(in_dim, out_dim, BS).to(dev)
        with torch.no_grad():
            mod.weight.copy_(w)
            mod.bias.copy_(torch.from_numpy(golden[f"bh4_{tag}_bias"]))
        z = t2n(mod(torch.from_numpy(x).to(dev)))
        zr = golden[f"bh4_{tag}_z"]
        assert rel_err(z, zr) < 2e-5
        # signs against the reference's own evaluation: only coordinates with |v| < 1e-6 (fp64 v) may differ
        z64 = PAR.projection_fp64_torch(torch.from_numpy(x).to(dev), w, mod.bias.detach(), out_dim).cpu().numpy()
        PAR.assert_codes_match_up_to_tiny_coordinates(z, zr, z64)
    # no bounded wait inside the block kernel (weight chunks arriving by bulk copy) ran out
    from lookupffn_b200 import _lib
    assert _lib.device_status(dev) & _lib.STATUS_TIMEOUT == 0


def test_cpu_bh4_convention_matches_reference_cpu_extension(dev):
    """transpose_w=1 with had_scale=1/D is the projection of the reference's CPU extension
    (bh4/cpu/torch_extension.cpp:123-196); vectors from that extension itself (tests/golden/sbdht_golden.npz).
    Both block kernels are exercised: the 64 x 64 fast path ([i][o] weights as given) and the generic one."""
    import os

    from lookupffn_b200 import ops

    g = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sbdht_golden.npz")))
    x, w, out = g["sbdht_x"], g["sbdht_w"], g["sbdht_out"]
    D = x.shape[1]
    xd, wd = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    z = ops.bh4(xd, wd, transpose_w=True, had_scale=1.0 / D)
    assert rel_err(t2n(z), out) < 2e-6
    np.testing.assert_array_equal(t2n(z), O.project(x, w, out.shape[1], transpose_w=True, had_scale=1.0 / D,
                                                    mix_a=1.0, mix_b=0.0))
    # the same function through the other weight layout: W^T handed over with transpose_w=0 (generic kernel)
    z2 = ops.bh4(xd, wd.transpose(-1, -2).contiguous(), transpose_w=False, had_scale=1.0 / D)
    np.testing.assert_array_equal(t2n(z2), t2n(z))
    f = ops.hadamard(torch.from_numpy(g["fwht_x"]).to(dev), scale=1.0 / D)
    assert rel_err(t2n(f), g["fwht_out"]) < 1e-6


# ---- gather forward ----------------------------------------------------------------------------------
GATHER_CASES = [
    # N, I, S, d
    (1, 1, 5, 4), (7, 3, 50, 16), (33, 18, 333, 64), (64, 128, 32768, 512), (20, 512, 4096, 768),
    (5, 37, 1000, 1024), (3, 64, 500, 1536), (4, 10, 100, 2052), (6, 70, 900, 4096), (17, 0, 9, 64),
    (40, 4608, 2000, 768),
]


@pytest.mark.parametrize("N,I,S,d", GATHER_CASES)
def test_gather_fwd_fp32_bit_exact(dev, N, I, S, d):
    from lookupffn_b200 import ops

    rng = np.random.RandomState(N + I + d)
    idx = rng.randint(0, S, size=(N, I)).astype(np.int32)
    w = rng.randn(N, I).astype(np.float32)
    tab = (0.02 * rng.randn(S, d)).astype(np.float32)
    bias = rng.randn(d).astype(np.float32)
    ti, tw, tt, tb = (torch.from_numpy(a).to(dev) for a in (idx, w, tab, bias))
    np.testing.assert_array_equal(t2n(ops.weighted_vector_gather_add(ti, tt, tw)), O.gather(idx, w, tab))
    np.testing.assert_array_equal(t2n(ops.weighted_vector_gather_add(ti, tt, tw, bias=tb)),
                                  O.gather(idx, w, tab, bias=bias))
    out_b = ops.weighted_vector_gather_add(ti, tt, tw, bias=tb, out_dtype=torch.bfloat16)
    np.testing.assert_array_equal(t2n(out_b), O.gather(idx, w, tab, bias=bias, out_bf16=True))


@pytest.mark.parametrize("N,I,S,d", [c for c in GATHER_CASES if c[3] % 8 == 0])
def test_gather_fwd_bf16_bit_exact(dev, N, I, S, d):
    from lookupffn_b200 import ops

    rng = np.random.RandomState(N + I + d + 1)
    idx = rng.randint(0, S, size=(N, I)).astype(np.int32)
    w = rng.randn(N, I).astype(np.float32)
    tab = O.f32_to_bf16_bits((0.02 * rng.randn(S, d)).astype(np.float32))
    bias = rng.randn(d).astype(np.float32)
    ti, tw, tb = (torch.from_numpy(a).to(dev) for a in (idx, w, bias))
    tt = bf16_tensor(tab, dev)
    out = ops.weighted_vector_gather_add(ti, tt, tw, bias=tb)
    assert out.dtype == torch.bfloat16
    np.testing.assert_array_equal(t2n(out), O.gather(idx, w, tab, bias=bias, out_bf16=True))
    out32 = ops.weighted_vector_gather_add(ti, tt, tw, out_dtype=torch.float32)
    np.testing.assert_array_equal(t2n(out32), O.gather(idx, w, tab))


def test_gather_matches_reference_golden(dev, golden):
    from lookupffn_b200 import ops

    for tag in ("a", "b"):
        ti, tw, tt = (torch.from_numpy(golden[f"gat_{tag}_{n}"]).to(dev) for n in ("idx", "w", "tables"))
        out = t2n(ops.weighted_vector_gather_add(ti, tt, tw))
        assert rel_err(out, golden[f"gat_{tag}_out_scalar"]) < 1e-6
        assert rel_err(out, golden[f"gat_{tag}_out_torch"]) < 1e-6


def test_gather_out_of_range_index_is_skipped_and_flagged(dev):
    from lookupffn_b200 import _lib, ops

    rng = np.random.RandomState(3)
    N, I, S, d = 9, 12, 40, 64
    idx = rng.randint(0, S, size=(N, I)).astype(np.int32)
    idx[2, 5] = S
    idx[4, 0] = -1
    w = rng.randn(N, I).astype(np.float32)
    tab = rng.randn(S, d).astype(np.float32)
    _lib.device_status(dev)
    out = ops.weighted_vector_gather_add(*(torch.from_numpy(a).to(dev) for a in (idx, tab, w)))
    ref, bad = O.gather(idx, w, tab, return_bad=True)
    assert bad == 2
    np.testing.assert_array_equal(t2n(out), ref)
    assert _lib.device_status(dev) & _lib.STATUS_INDEX_RANGE
    assert _lib.device_status(dev) == 0  # reading clears it


# ---- gather backward --------------------------------------------------------------------------------------
BWD_CASES = [(1, 1, 5, 4), (32, 8, 300, 64), (19, 33, 777, 768), (8, 64, 100, 1024), (5, 40, 64, 1536), (6, 90, 64, 3072)]


@pytest.mark.parametrize("N,I,S,d", BWD_CASES)
def test_gather_bwd_weights(dev, N, I, S, d):
    from lookupffn_b200 import ops

    rng = np.random.RandomState(N + I)
    idx = rng.randint(0, S, size=(N, I)).astype(np.int32)
    tab = (0.02 * rng.randn(S, d)).astype(np.float32)
    dy = rng.randn(N, d).astype(np.float32)
    ti, tt, tg = (torch.from_numpy(a).to(dev) for a in (idx, tab, dy))
    assert rel_err(t2n(ops.indexed_inner_product(ti, tg, tt)), O.gather_bwd_weights(idx, dy, tab)) < 1e-4
    if d % 8 == 0:
        tb = O.f32_to_bf16_bits(tab)
        assert rel_err(t2n(ops.indexed_inner_product(ti, tg, bf16_tensor(tb, dev))),
                       O.gather_bwd_weights(idx, dy, tb)) < 1e-4


@pytest.mark.parametrize("N,I,S,d", BWD_CASES)
def test_gather_bwd_tables_any_index_list(dev, N, I, S, d):
    from lookupffn_b200 import ops

    rng = np.random.RandomState(N + I + 7)
    idx = rng.randint(0, S, size=(N, I)).astype(np.int32)
    idx[0, :] = min(3, S - 1)  # many terms on one row
    w = rng.randn(N, I).astype(np.float32)
    dy = rng.randn(N, d).astype(np.float32)
    ti, tw, tg = (torch.from_numpy(a).to(dev) for a in (idx, w, dy))
    out = ops.weighted_vector_scatter_add(ti, tg, tw, S)
    assert rel_err(t2n(out), O.gather_bwd_tables(idx, w, dy, S)) < 1e-5


@pytest.mark.parametrize("N,T,m,rows,d", [(1, 1, 1, 2, 4), (50, 6, 1, 256, 64), (300, 5, 9, 256, 768),
                                           (700, 3, 1, 64, 512), (64, 4, 7, 4096, 128), (2000, 2, 1, 16, 1024),
                                           (5000, 2, 3, 2048, 64), (33, 3, 2, 2049, 32),
                                           # enough gradient rows that the segmented gather runs in column tiles
                                           # (tiles of 96 + 96 + 64 vectors at d = 1024; 64 + 64 + 64 at d = 768)
                                           (12000, 2, 1, 16, 1024), (14001, 1, 2, 64, 768)])
def test_gather_bwd_tables_sorted_bit_exact_and_deterministic(dev, N, T, m, rows, d):
    from lookupffn_b200 import ops

    rng = np.random.RandomState(N + T)
    idx = (rng.randint(0, rows, size=(N, T, m)) + (np.arange(T) * rows)[None, :, None]).astype(np.int32).reshape(N, T * m)
    w = rng.randn(N, T * m).astype(np.float32)
    dy = rng.randn(N, d).astype(np.float32)
    ti, tw, tg = (torch.from_numpy(a).to(dev) for a in (idx, w, dy))
    out1 = t2n(ops.weighted_vector_scatter_add(ti, tg, tw, T * rows, structure=(T, m, rows)))
    out2 = t2n(ops.weighted_vector_scatter_add(ti, tg, tw, T * rows, structure=(T, m, rows)))
    np.testing.assert_array_equal(out1, out2)
    np.testing.assert_array_equal(out1, O.gather_bwd_tables(idx, w, dy, T * rows))


def test_gather_backward_matches_reference_golden(dev, golden):
    from lookupffn_b200 import ops

    ti, tw, tt, tg = (torch.from_numpy(golden[f"bwd_{n}"]).to(dev) for n in ("idx", "w", "tables", "dy"))
    tt.requires_grad_(True)
    tw.requires_grad_(True)
    out = ops.weighted_gather_add(ti, tt, tw)
    out.backward(tg)
    assert rel_err(t2n(out.detach()), golden["bwd_out"]) < 1e-6
    assert rel_err(t2n(tw.grad), golden["bwd_dw"]) < 1e-5
    assert rel_err(t2n(tt.grad), golden["bwd_dtables"]) < 1e-5


# ---- the module ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["bh4", "dense"])
def test_module_matches_reference_golden(dev, golden, tag):
    from lookupffn_b200 import LookupFFN

    sd = {k[len(f"mod_{tag}_param_"):]: torch.from_numpy(v) for k, v in golden.items()
          if k.startswith(f"mod_{tag}_param_")}
    T, rows, d_out = sd["tables"].shape
    cfg = Namespace(hidden_size=sd["LayerNorm.weight"].numel(), ffn_num_table=T, ffn_table_size=rows,
                    layer_norm_eps=1e-5, projection_type=tag, block_size=64)
    mod = LookupFFN(cfg, d_out)
    mod.load_state_dict(sd, strict=True)
    mod = mod.to(dev).eval()
    x = torch.from_numpy(golden[f"mod_{tag}_x"]).to(dev)
    with torch.no_grad():
        y = mod(x)
        u = mod.LayerNorm(x.reshape(-1, x.shape[-1]))
        idx, w = mod.hash(u)
    assert y.shape == golden[f"mod_{tag}_y"].shape  # leading dims kept (lookup.py:112-118)
    code = t2n(idx) - (np.arange(T) * rows)[None].astype(np.int32)
    ref_code = golden[f"mod_{tag}_code"]
    # LayerNorm and (dense) the projection run in torch on the GPU: a code may differ from the reference's only
    # when one of its coordinates has |v| < 1e-6; tokens without a differing code must match in weights and output
    zr = golden[f"mod_{tag}_z"].reshape(-1, T, int(np.log2(rows)))
    flipped = code != ref_code
    assert np.abs(zr[flipped]).min(axis=-1).max(initial=0.0) < PAR.V_EPS
    clean = ~flipped.any(axis=-1)
    assert clean.sum() >= 0.9 * clean.size
    assert rel_err(t2n(w)[clean], golden[f"mod_{tag}_score"].reshape(-1, T)[clean]) < 1e-4
    assert rel_err(t2n(y).reshape(-1, d_out)[clean], golden[f"mod_{tag}_y"].reshape(-1, d_out)[clean]) < 1e-4


def test_module_backward_tables_and_bias(dev):
    from lookupffn_b200 import LookupFFN

    torch.manual_seed(0)
    cfg = Namespace(hidden_size=96, ffn_num_table=12, ffn_table_size=64, layer_norm_eps=1e-5,
                    projection_type="bh4", block_size=32)
    mod = LookupFFN(cfg, 64).to(dev).train()
    x = torch.randn(4, 10, 96, device=dev)
    y = mod(x)
    g = torch.randn_like(y)
    y.backward(g)
    with torch.no_grad():
        u = mod.LayerNorm(x.reshape(-1, 96))
        idx, w = mod.hash(u)
    ref = O.gather_bwd_tables(t2n(idx), t2n(w), t2n(g.reshape(-1, 64)), 12 * 64)
    np.testing.assert_array_equal(t2n(mod.tables.grad).reshape(12 * 64, 64), ref)
    assert rel_err(t2n(mod.bias.grad), t2n(g.reshape(-1, 64).sum(0))) < 1e-5


# ---- full-size properties (benchmark config 3) -------------------------------------------------------------------
def test_full_size_forward_properties(dev):
    from lookupffn_b200 import ops

    N, d_in, D, T, k, d_out = 65536, 768, 1024, 512, 8, 768
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(N, d_in, generator=g, device=dev).to(torch.bfloat16)
    tables = (0.02 * torch.randn(T << k, d_out, generator=g, device=dev)).to(torch.bfloat16)
    signs = (2 * torch.randint(0, 2, (4, 2, D, 1, 1), generator=g, device=dev) - 1).float()
    desc = ops.make_hash_desc(d_in, signs, None, T, k, had_scale=1 / 32, mix_a=1.0, mix_b=0.0)
    idx, w, _ = ops.hash_fwd(x, desc)
    y = ops.weighted_vector_gather_add(idx, tables, w)
    # a random sample of tokens against the oracle, end to end (codes exact, outputs bit-exact given equal weights)
    sel = torch.randperm(N, generator=torch.Generator().manual_seed(2))[:64]
    xs = t2n(x[sel.to(dev)])
    z_ref = O.project(O.bf16_bits_to_f32(xs), t2n(signs), T * k, had_scale=1 / 32, mix_a=1.0, mix_b=0.0)
    idx_ref, w_ref = O.code_weights(z_ref, T, k)
    np.testing.assert_array_equal(t2n(idx[sel.to(dev)]), idx_ref)
    assert rel_err(t2n(w[sel.to(dev)]), w_ref) < 1e-5
    y_ref = O.gather(idx_ref, t2n(w[sel.to(dev)]), t2n(tables), out_bf16=True)
    np.testing.assert_array_equal(t2n(y[sel.to(dev)]), y_ref)
    # codes are in range and use every row of every table about equally
    codes = idx - (torch.arange(T, device=dev, dtype=torch.int32) << k)[None]
    assert int(codes.min()) >= 0 and int(codes.max()) < (1 << k)
    # permutation equivariance: permuting tokens permutes outputs, bit for bit
    perm = torch.randperm(N, generator=g, device=dev)
    y_p = ops.weighted_vector_gather_add(idx[perm].contiguous(), tables, w[perm].contiguous())
    assert torch.equal(y_p.view(torch.int16), y[perm].view(torch.int16))
    # scaling weights by a power of two scales fp32 outputs exactly
    y32 = ops.weighted_vector_gather_add(idx, tables, w, out_dtype=torch.float32)
    y32_2 = ops.weighted_vector_gather_add(idx, tables, w * 4.0, out_dtype=torch.float32)
    assert torch.equal(y32 * 4.0, y32_2)
    # additivity over a split of the tables: the two halves' partial sums add up to the whole within rounding
    h = (T // 2)
    ya = ops.weighted_vector_gather_add(idx[:, :h].contiguous(), tables, w[:, :h].contiguous(), out_dtype=torch.float32)
    yb = ops.weighted_vector_gather_add(idx[:, h:].contiguous(), tables, w[:, h:].contiguous(), out_dtype=torch.float32)
    err = (ya + yb - y32).abs().max() / y32.abs().max()
    assert float(err) < 1e-5


# ---- gradients through the whole layer --------------------------------------------------------------------------
def _torch_reference_layer(mod, x, idx):
    """fp64 PyTorch restatement of the layer for gradient checks (lookup.py:29-39,98-129, bh4/kernel.py:23-36,
    compute_code_score/kernel.py:51-53).  The discrete row indices come from the CUDA forward: codes carry no
    gradient, and reusing them keeps a coordinate at rounding level from picking another row."""
    from scipy.linalg import hadamard as sylvester

    p = mod.hash.projection
    T, k = mod.hash.num_table, mod.hash.code_length
    u = torch.nn.functional.layer_norm(x.double(), (x.shape[-1],), mod.LayerNorm.weight.double(),
                                       mod.LayerNorm.bias.double(), mod.LayerNorm.eps)
    N = u.shape[0]
    if isinstance(p, torch.nn.Linear):
        z = u @ p.weight.double().t() + p.bias.double()
    else:
        D, BS, R = p.padded_in_dim, p.block_size, p.num_repeat
        H = torch.tensor(sylvester(D), dtype=torch.float64, device=x.device)
        up = torch.nn.functional.pad(u, (0, D - u.shape[1]))
        outs = []
        for r in range(R):
            y = up
            for j in range(p.weight.shape[1]):
                y = torch.einsum("bni,noi->bno", y.reshape(N, D // BS, BS), p.weight[r, j].double()).reshape(N, D)
                y = (y @ H) * p.had_scale
            outs.append(y)
        z = p.mix[0] * torch.cat(outs, -1) + p.mix[1] * up.repeat(1, R)
        z = z[:, :T * k] + p.bias.double()
    a = z.reshape(N, T, k).abs()
    score = a.sum(-1) / torch.prod(1 + torch.exp(-2 * a), dim=-1)
    rows = mod.tables.double().reshape(-1, mod.tables.shape[-1])[idx.long()]     # [N, T, d]
    return (rows * score[:, :, None]).sum(1) + mod.bias.double()


@pytest.mark.parametrize("ptype,block", [("bh4", 64), ("bh4", 16), ("dense", 64), ("sign_hadamard", 1)])
def test_layer_gradients_match_torch_reference(dev, ptype, block):
    from lookupffn_b200 import LookupFFN

    torch.manual_seed(3)
    hidden = 256 if block == 64 else 96
    cfg = Namespace(hidden_size=hidden, ffn_num_table=40, ffn_table_size=64, layer_norm_eps=1e-5,
                    projection_type=ptype, block_size=block)
    mod = LookupFFN(cfg, 64).to(dev).train()
    with torch.no_grad():
        mod.hash.projection.bias.normal_(0, 0.05)
        if ptype == "bh4":
            mod.hash.projection.weight.mul_(4.0)  # z of order 1, so that the score's exponentials matter
    x = torch.randn(50, hidden, device=dev, requires_grad=True)
    y = mod(x)
    g = torch.randn_like(y)
    y.backward(g)
    got = {n: q.grad.clone() for n, q in mod.named_parameters() if q.grad is not None}
    got["x"] = x.grad.clone()
    with torch.no_grad():
        idx, _ = mod.hash(mod.LayerNorm(x))
    for q in mod.parameters():
        q.grad = None
    x2 = x.detach().clone().requires_grad_(True)
    y_ref = _torch_reference_layer(mod, x2, idx)
    assert rel_err(t2n(y.detach()), y_ref.detach().cpu().numpy()) < 1e-4
    y_ref.backward(g.double())
    want = {n: q.grad for n, q in mod.named_parameters() if q.grad is not None}
    want["x"] = x2.grad
    assert set(got) == set(want)
    for n in want:
        # north-star bar for gradients with fp32 tables: 1e-3 relative
        assert rel_err(t2n(got[n].float()), want[n].float().cpu().numpy()) < 1e-3, n


def test_encoder_matches_reference_golden(dev, golden):
    """The reference's Lookup encoder (2 layers) run on CPU by the reference code vs this package's encoder
    with the same weights on the GPU.  A coordinate at rounding level may select another table row for a token,
    so the bar is per token: at least 95 % of the token rows agree to 1e-3 of the output scale."""
    from tests.test_abi import _encoder_config
    from lookupffn_b200.encoder import Lookup

    sd = {k[len("enc_param_"):]: torch.from_numpy(v) for k, v in golden.items() if k.startswith("enc_param_")}
    enc = Lookup(_encoder_config())
    enc.load_state_dict(sd, strict=True)
    enc = enc.to(dev).eval()
    ids = torch.from_numpy(golden["enc_ids"]).to(dev)
    mask = torch.from_numpy(golden["enc_mask"]).to(dev)
    B, S = ids.shape
    with torch.no_grad():
        out, extra = enc(ids, torch.zeros_like(ids), torch.arange(S, device=dev)[None].repeat(B, 1), mask)
    assert extra == {}
    ref = golden["enc_out"]
    err = np.abs(t2n(out) - ref).max(axis=-1) / np.abs(ref).max()
    valid = golden["enc_mask"] > 0   # padded positions attend to nothing meaningful in either implementation
    assert (err[valid] < 1e-3).mean() >= 0.95, err


@pytest.mark.parametrize("mode", ["score", "soft_flip", "ones"])
@pytest.mark.parametrize("k", [1, 6, 8, 12])
def test_code_weights_bwd_matches_autograd(dev, mode, k):
    """dz from the CUDA kernel vs torch autograd of an fp64 restatement of the weight formulas
    (compute_code_score/kernel.py:51-53; soft-flip as specified for the benchmark's config 4)."""
    from lookupffn_b200 import ops

    torch.manual_seed(k)
    N, T, tau = 37, 9, 0.5
    z = torch.randn(N, T, k, device=dev)
    z[0, 0, 0] = 0.0
    wm = {"score": O.WEIGHT_SCORE, "soft_flip": O.WEIGHT_SOFT_FLIP, "ones": O.WEIGHT_ONES}[mode]
    m = k + 1 if mode == "soft_flip" else 1
    dw = torch.randn(N, T * m, device=dev)
    dz = ops.code_weights_bwd(z, dw, wm, tau)
    zd = z.double().requires_grad_(True)
    a = zd.abs()
    if mode == "score":
        w = (a.sum(-1) / torch.prod(1 + torch.exp(-2 * a), -1)).reshape(N, T)
    elif mode == "ones":
        w = torch.ones(N, T, dtype=torch.float64, device=dev) + 0 * a.sum(-1)
    else:
        s = torch.sigmoid(a / tau)
        cols = [torch.prod(s, -1)]
        for j in range(k):
            f = s.clone()
            f[..., j] = 1 - s[..., j]
            cols.append(torch.prod(f, -1))
        w = torch.stack(cols, -1).reshape(N, T * m)
    (w * dw.double()).sum().backward()
    assert rel_err(t2n(dz), zd.grad.float().cpu().numpy()) < 1e-5 or float(zd.grad.abs().max()) == 0.0
    if mode == "ones":
        assert float(dz.abs().max()) == 0.0


# ---- the whole-layer entry point (lffn_layer_fwd) --------------------------------------------------------------------
FUSED_CASES = [
    # N, d_in, D, T, d_out, bf16, weight_mode, bit_order, (t_begin, t_count)
    (77, 768, 1024, 512, 768, True, O.WEIGHT_SCORE, O.MSB_FIRST, None),      # benchmark config 3
    (50, 512, 512, 128, 512, False, O.WEIGHT_ONES, O.LSB_FIRST, None),       # benchmark config 1
    (33, 400, 512, 200, 512, True, O.WEIGHT_SCORE, O.MSB_FIRST, None),       # T*k not a multiple of D; VPL 2
    (20, 1000, 1024, 300, 1024, True, O.WEIGHT_SCORE, O.LSB_FIRST, (64, 170)),  # a rank's share of the tables
    (9, 512, 512, 96, 768, False, O.WEIGHT_SCORE, O.MSB_FIRST, (32, 64)),    # VPL 6
    (9, 512, 512, 64, 1024, False, O.WEIGHT_SCORE, O.MSB_FIRST, None),       # VPL 8
    (12, 100, 128, 40, 64, False, O.WEIGHT_SCORE, O.MSB_FIRST, None),        # small D: the scalar-layout hash kernel
    (12, 512, 512, 64, 512, False, O.WEIGHT_SCORE, O.MSB_FIRST, (10, 40)),   # table range not aligned to anything
]


@pytest.mark.parametrize("case", FUSED_CASES, ids=[f"f{i}" for i in range(len(FUSED_CASES))])
def test_layer_fwd_matches_oracle_and_separate_calls(dev, case):
    from lookupffn_b200 import ops

    N, d_in, D, T, d_out, bf16, wm, bo, rng_t = case
    k = 8
    rng = np.random.RandomState(N + T)
    R = max(1, -(-T * k // D))
    signs = make_proj(rng, D, 1, 2, R, signs=True)
    pbias = (0.05 * rng.randn(T * k)).astype(np.float32)
    obias = rng.randn(d_out).astype(np.float32)
    x = rng.randn(N, d_in).astype(np.float32)
    tab = (0.02 * rng.randn(T << k, d_out)).astype(np.float32)
    tb, tc = (0, T) if rng_t is None else rng_t
    hs = 1.0 / 32
    if bf16:
        xb, tabb = O.f32_to_bf16_bits(x), O.f32_to_bf16_bits(tab)
        xt, tt = bf16_tensor(xb, dev), bf16_tensor(tabb, dev)
        x_ref, tab_ref = O.bf16_bits_to_f32(xb), tabb
    else:
        xt, tt = torch.from_numpy(x).to(dev), torch.from_numpy(tab).to(dev)
        x_ref, tab_ref = x, tab
    desc = ops.make_hash_desc(d_in, torch.from_numpy(signs).to(dev), torch.from_numpy(pbias).to(dev), T, k,
                              had_scale=hs, mix_a=1.0, mix_b=0.0, bit_order=bo, weight_mode=wm)
    local = tt[tb << k:(tb + tc) << k].contiguous()
    y = ops.layer_fwd(xt, desc, local, bias=torch.from_numpy(obias).to(dev), t_begin=tb, t_count=tc)
    # lffn_hash_fwd + lffn_gather_fwd called separately on the same inputs: bit-identical
    idx, w, _ = ops.hash_fwd(xt, desc, t_begin=tb, t_count=tc)
    y2 = ops.weighted_vector_gather_add(idx, local, w, bias=torch.from_numpy(obias).to(dev))
    np.testing.assert_array_equal(t2n(y), t2n(y2))
    # the oracle, with the GPU's weights (expf differs in the last bits between libm and CUDA)
    z_ref = O.project(x_ref, signs, T * k, had_scale=hs, mix_a=1.0, mix_b=0.0, bias=pbias)
    idx_ref, _ = O.code_weights(z_ref[:, tb * k:(tb + tc) * k], tc, k, bit_order=bo, weight_mode=wm)
    np.testing.assert_array_equal(t2n(idx), idx_ref)
    y_ref = O.gather(idx_ref, t2n(w), tab_ref[tb << k:(tb + tc) << k], bias=obias, out_bf16=bf16)
    np.testing.assert_array_equal(t2n(y), y_ref)


# ---- edge cases ----------------------------------------------------------------------------------------------------
def test_empty_inputs(dev):
    from lookupffn_b200 import ops

    signs = torch.ones(1, 2, 256, 1, 1, device=dev)
    desc = ops.make_hash_desc(200, signs, None, 32, 8)
    idx, w, z = ops.hash_fwd(torch.zeros(0, 200, device=dev), desc, want_z=True)
    assert idx.shape == (0, 32) and w.shape == (0, 32) and z.shape == (0, 256)
    tab = torch.randn(64, 16, device=dev)
    out = ops.weighted_vector_gather_add(torch.zeros(0, 4, dtype=torch.int32, device=dev), tab, torch.zeros(0, 4, device=dev))
    assert out.shape == (0, 16)
    # an empty index list gives the bias (or zeros)
    b = torch.arange(16, device=dev, dtype=torch.float32)
    out = ops.weighted_vector_gather_add(torch.zeros(3, 0, dtype=torch.int32, device=dev), tab, torch.zeros(3, 0, device=dev), bias=b)
    assert torch.equal(out, b[None].repeat(3, 1))
    dt = ops.weighted_vector_scatter_add(torch.zeros(0, 4, dtype=torch.int32, device=dev), torch.zeros(0, 16, device=dev),
                                         torch.zeros(0, 4, device=dev), 64)
    assert dt.shape == (64, 16) and float(dt.abs().max()) == 0.0
    dt = ops.weighted_vector_scatter_add(torch.zeros(0, 4, dtype=torch.int32, device=dev), torch.zeros(0, 16, device=dev),
                                         torch.zeros(0, 4, device=dev), 64, structure=(4, 1, 16))
    assert float(dt.abs().max()) == 0.0
    assert ops.hadamard(torch.zeros(0, 64, device=dev)).shape == (0, 64)


def test_module_bf16_tables_and_leading_dims(dev):
    from lookupffn_b200 import LookupFFN

    torch.manual_seed(1)
    cfg = Namespace(hidden_size=768, ffn_num_table=64, ffn_table_size=256, layer_norm_eps=1e-5,
                    projection_type="sign_hadamard", block_size=1, lookup_table_dtype=torch.bfloat16)
    mod = LookupFFN(cfg, 768).to(dev).eval()
    x = torch.randn(2, 3, 5, 768, device=dev)
    with torch.no_grad():
        y = mod(x)
        # the module's inference path: LayerNorm inside the hash kernel
        idx, w = mod.hash(x.reshape(-1, 768), layer_norm=(mod.LayerNorm.weight, mod.LayerNorm.bias, 1e-5))
    assert y.shape == (2, 3, 5, 768) and y.dtype == torch.bfloat16
    ref = O.gather(t2n(idx), t2n(w), t2n(mod.tables.detach().reshape(-1, 768)), bias=t2n(mod.bias.detach()),
                   out_bf16=True)
    np.testing.assert_array_equal(t2n(y.reshape(-1, 768)), ref)
    # codes from the oracle's LayerNorm (accumulated in double) and projection: equal wherever no coordinate is tiny
    p = mod.hash.projection
    u = O.layernorm(t2n(x.reshape(-1, 768)), t2n(mod.LayerNorm.weight.detach()), t2n(mod.LayerNorm.bias.detach()), 1e-5)
    z_ref = O.project(u, t2n(p.weight.detach()), 64 * 8, had_scale=float(np.float32(p.had_scale)), mix_a=1.0,
                      mix_b=0.0, bias=t2n(p.bias.detach()))
    idx_ref, _ = O.code_weights(z_ref, 64, 8)
    clean = ~(np.abs(z_ref) < PAR.V_EPS).reshape(-1, 64, 8).any(axis=-1)
    np.testing.assert_array_equal(t2n(idx)[clean], idx_ref[clean])


def test_sliced_index_lists_are_bit_exact(dev):
    """A table set beyond 256 MB with a long index list takes the sliced path of the forward gather and of the
    weight gradient (one launch per slice of the list, fp32 partial sums resumed): results must not change."""
    from lookupffn_b200 import ops

    rng = np.random.RandomState(11)
    N, T, m, rows, d = 24, 176, 9, 512, 768          # 176 * 512 rows * 768 * 4 B = 277 MB, I = 1584
    S, I = T * rows, T * m
    idx = (rng.randint(0, rows, size=(N, T, m)) + (np.arange(T) * rows)[None, :, None]).astype(np.int32).reshape(N, I)
    w = rng.randn(N, I).astype(np.float32)
    dy = rng.randn(N, d).astype(np.float32)
    bias = rng.randn(d).astype(np.float32)
    tab = torch.empty(S, d, device=dev).normal_(0, 0.02, generator=torch.Generator(device=dev).manual_seed(3))
    ti, tw, tg, tb = (torch.from_numpy(a).to(dev) for a in (idx, w, dy, bias))
    y = ops.weighted_vector_gather_add(ti, tab, tw, bias=tb)
    dw = ops.indexed_inner_product(ti, tg, tab)
    tabn = t2n(tab)
    np.testing.assert_array_equal(t2n(y), O.gather(idx, w, tabn, bias=bias))
    assert rel_err(t2n(dw), O.gather_bwd_weights(idx, dy, tabn)) < 1e-4


def test_layer_fwd_host_buffers_match_device_path(dev):
    """lffn_layer_fwd_host: pinned host x in, pinned host y out, chunked over internal streams; must equal the
    device-buffer path bit for bit, including a ragged last chunk and a second call that reuses the workspace."""
    import ctypes as C

    from lookupffn_b200 import _lib as L
    from lookupffn_b200 import ops

    lib = L.lib()
    g = torch.Generator(device=dev).manual_seed(8)
    N, d_in, D, T, k, d_out = 1000, 768, 1024, 96, 8, 768
    R = -(-T * k // D)
    x = torch.randn(N, d_in, generator=g, device=dev).to(torch.bfloat16)
    tables = (0.02 * torch.randn(T << k, d_out, generator=g, device=dev)).to(torch.bfloat16)
    signs = (2 * torch.randint(0, 2, (R, 2, D, 1, 1), generator=g, device=dev) - 1).float()
    bias = torch.randn(d_out, generator=g, device=dev)
    desc = ops.make_hash_desc(d_in, signs, None, T, k, had_scale=1 / 32, mix_a=1.0, mix_b=0.0)
    y_dev = ops.layer_fwd(x, desc, tables, bias=bias)
    chunk = 192  # 1000 = 5 * 192 + 40
    nbytes = lib.lffn_layer_fwd_host_ws_bytes(C.byref(desc), L.BF16, L.BF16, d_out, chunk)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    x_host = x.cpu().pin_memory()
    for _ in range(2):
        y_host = torch.zeros(N, d_out, dtype=torch.bfloat16).pin_memory()
        with torch.cuda.device(dev):
            L.check(lib.lffn_layer_fwd_host(C.byref(desc), L.ptr(x_host), L.BF16, N, L.ptr(tables), L.BF16, d_out,
                                            L.ptr(bias), L.ptr(y_host), L.BF16, L.ptr(ws), nbytes, chunk, L.stream_ptr(dev)))
        assert torch.equal(y_host.view(torch.int16), y_dev.cpu().view(torch.int16))
    # a workspace that is too small is refused with the needed size in the message
    rc = lib.lffn_layer_fwd_host(C.byref(desc), L.ptr(x_host), L.BF16, N, L.ptr(tables), L.BF16, d_out, L.ptr(bias),
                                 L.ptr(y_host), L.BF16, L.ptr(ws), nbytes // 2, chunk, L.stream_ptr(dev))
    assert rc == -5 and b"workspace" in lib.lffn_last_error_string()


def test_full_size_training_gather_adjoint_identities(dev):
    """Benchmark config 4 at full size (N=16384, T=512, k=8, m=9 candidates, d=768, fp32): the forward and the
    two gradients are tied by size-independent identities, since y is linear in the weights and in the tables:
        <y, dy> = sum_{n,i} w[n,i] * dw[n,i] = <dtables, tables>,
    and the sorted table gradient must reproduce bit for bit on a second run."""
    from lookupffn_b200 import ops

    N, T, k, d = 16384, 512, 8, 768
    m, rows = k + 1, 1 << k
    g = torch.Generator(device=dev).manual_seed(6)
    x = torch.randn(N, d, generator=g, device=dev)
    signs = (2 * torch.randint(0, 2, (4, 2, 1024, 1, 1), generator=g, device=dev) - 1).float()
    tables = 0.02 * torch.randn(T * rows, d, generator=g, device=dev)
    dy = torch.randn(N, d, generator=g, device=dev)
    desc = ops.make_hash_desc(d, signs, None, T, k, had_scale=1 / 32, mix_a=1.0, mix_b=0.0,
                              weight_mode=O.WEIGHT_SOFT_FLIP, tau=0.5)
    idx, w, _ = ops.hash_fwd(x, desc)
    assert idx.shape == (N, T * m)
    # the k+1 candidates of a table are the hard code and its k single-bit flips; their weights sum to <= 1
    cand = (idx.view(N, T, m) - (torch.arange(T, device=dev, dtype=torch.int32) * rows)[None, :, None])
    flips = cand[:, :, 1:] ^ cand[:, :, :1]
    assert bool(((flips & (flips - 1)) == 0).all()) and bool((flips > 0).all())
    assert float(w.view(N, T, m).sum(-1).max()) <= 1.0 + 1e-5
    y = ops.weighted_vector_gather_add(idx, tables, w)
    dw = ops.indexed_inner_product(idx, dy, tables)
    dt = ops.weighted_vector_scatter_add(idx, dy, w, T * rows, structure=(T, m, rows))
    dt2 = ops.weighted_vector_scatter_add(idx, dy, w, T * rows, structure=(T, m, rows))
    assert torch.equal(dt, dt2)
    a = float((y.double() * dy.double()).sum())
    b = float((w.double() * dw.double()).sum())
    c = float((dt.double() * tables.double()).sum())
    scale = float((y.double().abs() * dy.double().abs()).sum())
    assert abs(a - b) < 1e-5 * scale and abs(a - c) < 1e-5 * scale
    # a sample of tokens against the oracle
    sel = torch.arange(0, N, N // 16, device=dev)
    y_ref = O.gather(t2n(idx[sel]), t2n(w[sel]), t2n(tables))
    np.testing.assert_array_equal(t2n(y[sel]), y_ref)
