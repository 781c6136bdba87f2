"""Counting hash-code disagreements by the magnitude of the coordinate that caused them.

TEST AND COMPARATOR INFRASTRUCTURE: used by tests and by the benchmark's baseline leg; the product never calls it.

The bar for hash codes: bit-exact against the reference's own evaluation on the same inputs, except for
coordinates v of the projection with |v| < 1e-6, which are counted and reported.  Here v is judged on an fp64
evaluation of the projection where one is available (it is the value both fp32 evaluations approximate), else on
the reference's fp32 value.  The projection z is of unit scale (its rms is 0.65-0.8 on every input used here, the
module's own initialisation: weights randn / sqrt(BS * D), LayerNorm output), so 1e-6 is an absolute bound on z.
"""
import math

import numpy as np

V_EPS = 1e-6
HIST_EDGES = (0.0, 1e-7, 1e-6, 1e-5, 1e-4, float("inf"))  # five bins of |v|


def sign_mismatch_report(z, z_ref, v=None):
    """z, z_ref: the two fp32 evaluations of the projection (any shape, same shape); v: the values whose magnitude
    decides whether a disagreement is exempt (fp64 evaluation), default z_ref.  Returns a dict of plain numbers."""
    z = np.asarray(z)
    z_ref = np.asarray(z_ref)
    v = np.abs(np.asarray(z_ref if v is None else v, dtype=np.float64))
    bad = (z > 0) != (z_ref > 0)
    a = v[bad]
    hist = {f"[{lo:g}, {hi:g})": int(((a >= lo) & (a < hi)).sum()) for lo, hi in zip(HIST_EDGES[:-1], HIST_EDGES[1:])}
    return {"coordinates_checked": int(z.size), "sign_mismatches": int(bad.sum()),
            "mismatches_with_abs_v_below_1e-6": int((a < V_EPS).sum()),
            "mismatches_with_abs_v_at_or_above_1e-6": int((a >= V_EPS).sum()),
            "largest_abs_v_of_a_mismatch": float(a.max()) if a.size else 0.0,
            "mismatches_by_abs_v": hist, "z_rms": float(np.sqrt(np.mean(np.square(z_ref, dtype=np.float64))))}


def assert_codes_match_up_to_tiny_coordinates(z, z_ref, v=None):
    """Asserts the bar and returns (report, mask of coordinates whose signs disagree)."""
    rep = sign_mismatch_report(z, z_ref, v)
    assert rep["mismatches_with_abs_v_at_or_above_1e-6"] == 0, rep
    return rep, (np.asarray(z) > 0) != (np.asarray(z_ref) > 0)


def projection_fp64_torch(x, weight, bias, out_dim, decay=0.7, had_scale=1.0):
    """fp64 evaluation of the reference projection (lookup.py:29-39, bh4/kernel.py:23-36) with torch, on whatever
    device x lives on: per rotation and stage the block-diagonal product ("bni,noi->bno") and a product with the
    Sylvester matrix.  The mix coefficients are the fp32 values the fp32 paths use, widened."""
    import torch

    N, d_in = x.shape
    R, S, NB, BS, _ = weight.shape
    D = NB * BS
    xd = torch.zeros(N, D, dtype=torch.float64, device=x.device)
    xd[:, :d_in] = x.double()
    H = torch.ones(1, 1, dtype=torch.float64, device=x.device)
    for _ in range(int(math.log2(D))):
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    w = weight.double()
    outs = []
    for r in range(R):
        y = xd
        for s in range(S):
            y = torch.einsum("bni,noi->bno", y.reshape(N, NB, BS), w[r, s]).reshape(N, D) @ H
            if had_scale != 1.0:
                y = y * float(np.float32(had_scale))
        outs.append(y)
    a, b = float(np.float32(decay)), float(np.float32(1 - decay))
    z = a * torch.cat(outs, -1) + b * xd.repeat(1, R)
    z = z[:, :out_dim]
    return z if bias is None else z + bias.double()
