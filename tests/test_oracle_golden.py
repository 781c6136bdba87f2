"""Pins the CPU oracle (oracle/lffn_oracle.c) to vectors produced by the reference's own
code (tests/golden/make_golden.py).  Codes must agree exactly; where the reference result
comes from a differently ordered float reduction (torch matmul/einsum/sum) the comparison
carries the tolerance written beside it."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import parity as PAR


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)


@pytest.mark.parametrize("tag,T,k", [("k8", 12, 8), ("k6", 10, 6), ("k10", 5, 10), ("k1", 4, 1)])
def test_code_score_matches_reference(golden, tag, T, k):
    z = golden[f"ccs_{tag}_z"]
    idx, w = O.code_weights(z, T, k, bit_order=O.MSB_FIRST, weight_mode=O.WEIGHT_SCORE, add_offsets=False)
    # bit-exact codes against both reference implementations (torch formula and the C++ extension)
    np.testing.assert_array_equal(idx, golden[f"ccs_{tag}_code_torch"])
    np.testing.assert_array_equal(idx, golden[f"ccs_{tag}_code_cpp"])
    # scores: same formula, serial accumulation as the C++ extension; 1e-5 covers expf differences
    assert rel_err(w, golden[f"ccs_{tag}_score_cpp"]) < 1e-5
    assert rel_err(w, golden[f"ccs_{tag}_score_torch"]) < 1e-5


def test_code_edge_values(golden):
    # 0, -0, and NaN give bit 0 (strict >): compute_code_score/kernel.py:47, torch_extension.cc:35
    z = np.array([[0.0, -0.0, np.nan, 1e-45, -1e-45, np.inf, -np.inf, 3.0]], dtype=np.float32)
    idx, _ = O.code_weights(z, 1, 8, bit_order=O.MSB_FIRST, weight_mode=O.WEIGHT_ONES, add_offsets=False)
    assert idx[0, 0] == 0b00010101
    idx, _ = O.code_weights(z, 1, 8, bit_order=O.LSB_FIRST, weight_mode=O.WEIGHT_ONES, add_offsets=False)
    assert idx[0, 0] == 0b10101000


def test_lsb_is_bit_reversal_of_msb(golden):
    z = golden["ccs_k6_z"]
    a, _ = O.code_weights(z, 10, 6, bit_order=O.MSB_FIRST, add_offsets=False)
    b, _ = O.code_weights(z, 10, 6, bit_order=O.LSB_FIRST, add_offsets=False)
    rev = np.array([int(format(c, "06b")[::-1], 2) for c in range(64)])
    np.testing.assert_array_equal(rev[a], b)


@pytest.mark.parametrize("D", [64, 256, 1024])
def test_fwht_matches_reference_matmul(golden, D):
    x = golden[f"had_{D}_x"]
    # reference = X @ scipy.linalg.hadamard(D) in fp32; different summation order -> 1e-5 of the max
    assert rel_err(O.fwht(x), golden[f"had_{D}_y"]) < 1e-5


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_bh4_projection_matches_reference(golden, tag):
    in_dim, out_dim, BS, D, R = [int(v) for v in golden[f"bh4_{tag}_meta"]]
    x, w, bias = golden[f"bh4_{tag}_x"], golden[f"bh4_{tag}_w"], golden[f"bh4_{tag}_bias"]
    assert w.shape == (R, 4, D // BS, BS, BS)
    # raw bh4_cuda output (no mix, no slice, no bias)
    P = O.project(x, w, R * D, mix_a=1.0, mix_b=0.0)
    assert rel_err(P, golden[f"bh4_{tag}_P"]) < 2e-5
    # BH4._forward: 0.7 * P + 0.3 * tile(x_pad), slice, + bias
    z = O.project(x, w, out_dim, bias=bias)
    zr = golden[f"bh4_{tag}_z"]
    assert rel_err(z, zr) < 2e-5
    # sign bits may differ from the reference's einsum/matmul evaluation only on coordinates with |v| < 1e-6
    # (v judged on an fp64 evaluation); the disagreements are counted
    import torch

    z64 = PAR.projection_fp64_torch(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(bias), out_dim).numpy()
    PAR.assert_codes_match_up_to_tiny_coordinates(z, zr, z64)


def test_gather_matches_reference(golden):
    for tag in ("a", "b"):
        idx, w, tab = golden[f"gat_{tag}_idx"], golden[f"gat_{tag}_w"], golden[f"gat_{tag}_tables"]
        out = O.gather(idx, w, tab)
        assert rel_err(out, golden[f"gat_{tag}_out_scalar"]) < 1e-6
        assert rel_err(out, golden[f"gat_{tag}_out_torch"]) < 1e-6
    assert rel_err(O.gather(golden["gat_a_idx"], golden["gat_a_w"], golden["gat_a_tables"]),
                   golden["gat_a_out_avx2"]) < 1e-6


def test_gather_backward_matches_reference(golden):
    idx, w, tab, dy = golden["bwd_idx"], golden["bwd_w"], golden["bwd_tables"], golden["bwd_dy"]
    assert rel_err(O.gather(idx, w, tab), golden["bwd_out"]) < 1e-6
    dw = O.gather_bwd_weights(idx, dy, tab)
    assert rel_err(dw, golden["bwd_dw"]) < 1e-5
    assert rel_err(dw, golden["bwd_dw_autograd"]) < 1e-5
    dt = O.gather_bwd_tables(idx, w, dy, tab.shape[0])
    assert rel_err(dt, golden["bwd_dtables"]) < 1e-5
    assert rel_err(dt, golden["bwd_dtables_autograd"]) < 1e-5


def test_bf16_round_trip():
    rng = np.random.RandomState(0)
    a = rng.randn(1000).astype(np.float32)
    import torch

    ref = torch.from_numpy(a).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    np.testing.assert_array_equal(O.f32_to_bf16_bits(a), ref)
    np.testing.assert_array_equal(O.bf16_bits_to_f32(ref), torch.from_numpy(a).to(torch.bfloat16).float().numpy())
    # gather with bf16 tables == gather with the same values widened to fp32 (exact widening)
    tab = rng.randn(50, 16).astype(np.float32)
    tb = O.f32_to_bf16_bits(tab)
    idx = rng.randint(0, 50, size=(7, 6)).astype(np.int32)
    w = rng.randn(7, 6).astype(np.float32)
    np.testing.assert_array_equal(O.gather(idx, w, tb), O.gather(idx, w, O.bf16_bits_to_f32(tb)))
    ob = O.gather(idx, w, tb, out_bf16=True)
    np.testing.assert_array_equal(ob, O.f32_to_bf16_bits(O.gather(idx, w, tb)))


@pytest.mark.parametrize("tag", ["dense", "bh4"])
def test_whole_module_matches_reference(golden, tag):
    P = {k[len(f"mod_{tag}_param_"):]: v for k, v in golden.items() if k.startswith(f"mod_{tag}_param_")}
    assert set(P) == {"LayerNorm.weight", "LayerNorm.bias", "hash.projection.weight", "hash.projection.bias",
                      "tables", "bias"}
    x = golden[f"mod_{tag}_x"]
    x2 = x.reshape(-1, x.shape[-1])
    T, rows, d_out = P["tables"].shape
    k = int(np.log2(rows))
    u = O.layernorm(x2, P["LayerNorm.weight"], P["LayerNorm.bias"], 1e-5)
    assert rel_err(u, golden[f"mod_{tag}_u"]) < 1e-5
    if tag == "dense":
        z = O.project_dense(u, P["hash.projection.weight"], P["hash.projection.bias"])
    else:
        z = O.project(u, P["hash.projection.weight"], T * k, bias=P["hash.projection.bias"])
    zr = golden[f"mod_{tag}_z"]
    assert rel_err(z, zr) < 2e-5
    # from the reference's own z the codes and scores must match exactly / to expf accuracy
    idx, w = O.code_weights(zr, T, k, add_offsets=False)
    np.testing.assert_array_equal(idx, golden[f"mod_{tag}_code"])
    assert rel_err(w, golden[f"mod_{tag}_score"]) < 1e-5
    # the oracle's own pipeline: codes may differ only on coordinates with |v| < 1e-6; tokens without such a
    # coordinate must give the reference's codes exactly and its output to 1e-4
    idx2, w2 = O.code_weights(z, T, k, add_offsets=False)
    _, diff = PAR.assert_codes_match_up_to_tiny_coordinates(z, zr)
    clean = ~diff.any(axis=-1)
    assert clean.sum() >= 0.9 * clean.size
    np.testing.assert_array_equal(idx2[clean], golden[f"mod_{tag}_code"][clean])
    off = (np.arange(T) * rows)[None].astype(np.int32)
    y = O.gather(idx2 + off, w2, P["tables"].reshape(T * rows, d_out), bias=P["bias"])
    assert rel_err(y[clean], golden[f"mod_{tag}_y"].reshape(-1, d_out)[clean]) < 1e-4
    if tag == "bh4":
        y2 = O.layer_fwd(x2, P["hash.projection.weight"], P["tables"], T, k,
                         ln=(P["LayerNorm.weight"], P["LayerNorm.bias"], 1e-5),
                         proj_bias=P["hash.projection.bias"], bias=P["bias"])
        off = (np.arange(T) * rows)[None].astype(np.int32)
        np.testing.assert_array_equal(
            y2, O.gather(idx2 + off, w2, P["tables"].reshape(T * rows, d_out), bias=P["bias"]))


def test_cpu_bh4_convention_matches_reference_cpu_extension():
    """The reference's CPU inference path computes the projection with x . W per block and H / D
    (bh4/cpu/torch_extension.cpp:123-196), not the x . W^T and unnormalised H of its CUDA/training path.  The
    oracle reaches it with transpose_w=True, had_scale=1/D; tests/golden/sbdht_golden.npz holds outputs of the
    reference's own CPU extension (built against a stand-in libxsmm header, make_sbdht_golden.py)."""
    import os

    g = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sbdht_golden.npz")))
    x, w, out = g["sbdht_x"], g["sbdht_w"], g["sbdht_out"]
    D = x.shape[1]
    z = O.project(x, w, out.shape[1], transpose_w=True, had_scale=1.0 / D, mix_a=1.0, mix_b=0.0)
    assert rel_err(z, out) < 2e-6          # summation order of the 64-term products and of the butterflies differs
    other = O.project(x, w, out.shape[1], transpose_w=False, had_scale=1.0 / D, mix_a=1.0, mix_b=0.0)
    assert rel_err(other, out) > 0.5       # the CUDA convention is a different function of the same weights
    assert rel_err(O.fwht(g["fwht_x"], 1.0 / D), g["fwht_out"]) < 1e-6


def test_sign_mismatch_report_bins_by_magnitude():
    z_ref = np.array([[0.5, -2e-7, 3e-8, -4e-6, 0.2, -0.3]], dtype=np.float32)
    z = z_ref.copy()
    z[0, 1] = 1e-7      # flipped, |v| = 2e-7: exempt
    z[0, 2] = -1e-8     # flipped, |v| = 3e-8: exempt
    z[0, 3] = 1e-6      # flipped, |v| = 4e-6: not exempt
    rep = PAR.sign_mismatch_report(z, z_ref)
    assert rep["coordinates_checked"] == 6 and rep["sign_mismatches"] == 3
    assert rep["mismatches_with_abs_v_below_1e-6"] == 2 and rep["mismatches_with_abs_v_at_or_above_1e-6"] == 1
    assert rep["mismatches_by_abs_v"] == {"[0, 1e-07)": 1, "[1e-07, 1e-06)": 1, "[1e-06, 1e-05)": 1, "[1e-05, 0.0001)": 0,
                                          "[0.0001, inf)": 0}
    with pytest.raises(AssertionError):
        PAR.assert_codes_match_up_to_tiny_coordinates(z, z_ref)
    z[0, 3] = z_ref[0, 3]
    rep2, mask = PAR.assert_codes_match_up_to_tiny_coordinates(z, z_ref)
    assert mask.sum() == 2 and rep2["largest_abs_v_of_a_mismatch"] < 1e-6
