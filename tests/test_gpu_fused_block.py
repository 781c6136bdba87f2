"""The feed-forward block of an encoder layer as two kernels: LayerNorm inside the hash kernel's load
(lffn_hash_fwd_ln), bias and residual inside the gather's epilogue (lffn_gather_fwd_residual), and both through
lffn_layer_fwd_ln_residual and the module.  Checked against the CPU oracle (LayerNorm accumulated in double,
projection, codes, gather) -- codes may differ from the oracle's only on coordinates with |v| < 1e-6, outputs of
tokens without such a coordinate agree to 1e-5 -- and against the unfused path (torch LayerNorm, separate adds)."""
import ctypes as C
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

    _lib.lib()
    return torch.device("cuda:0")


def rel_err(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)


LN_CASES = [
    # N, d_in, D, BS, S, T, k, transpose_w   -> which kernel
    (70, 768, 1024, 1, 2, 512, 8, False),    # diagonal, vector layout (the benchmark's layer shape)
    (45, 200, 256, 1, 2, 60, 6, False),      # diagonal, scalar layout, tables straddle rotations
    (100, 512, 512, 64, 4, 256, 8, True),    # 64 x 64 blocks, input tile resident in shared memory
    (41, 700, 1024, 64, 4, 128, 8, True),    # 64 x 64 blocks, D = 1024: the mix re-reads x from global memory
    (37, 100, 128, 16, 4, 20, 6, False),     # generic block kernel, k does not divide D
]


@pytest.mark.parametrize("case", LN_CASES, ids=[f"ln{i}" for i in range(len(LN_CASES))])
def test_hash_with_layernorm_prologue_matches_oracle(dev, case):
    from lookupffn_b200 import ops

    N, d_in, D, BS, S, T, k, tw = case
    rng = np.random.RandomState(N * 7 + D)
    R = max(1, -(-T * k // D))
    NB = D // BS
    if BS == 1:
        pw = (2.0 * rng.randint(0, 2, size=(R, S, NB, 1, 1)) - 1.0).astype(np.float32)
        hs, mix = float(1.0 / np.sqrt(D)), (1.0, 0.0)
    else:
        pw = (rng.randn(R, S, NB, BS, BS) / np.sqrt(BS * D)).astype(np.float32)
        hs, mix = 1.0, (0.7, 1 - 0.7)
    x = (1.5 * rng.randn(N, d_in) + 0.3).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.randn(d_in)).astype(np.float32)
    beta = (0.05 * rng.randn(d_in)).astype(np.float32)
    pbias = (0.02 * rng.randn(T * k)).astype(np.float32)
    eps = 1e-5
    u = O.layernorm(x, gamma, beta, eps)
    z_ref = O.project(u, pw, T * k, transpose_w=tw, had_scale=hs, mix_a=mix[0], mix_b=mix[1], bias=pbias)
    desc = ops.make_hash_desc(d_in, torch.from_numpy(pw).to(dev), torch.from_numpy(pbias).to(dev), T, k,
                              transpose_w=tw, had_scale=hs, mix_a=mix[0], mix_b=mix[1])
    ln = (torch.from_numpy(gamma).to(dev), torch.from_numpy(beta).to(dev), eps)
    xt = torch.from_numpy(x).to(dev)
    idx, w, z = ops.hash_fwd(xt, desc, want_z=True, layer_norm=ln)
    z = z.cpu().numpy()
    assert rel_err(z, z_ref) < 5e-6
    _, flipped = PAR.assert_codes_match_up_to_tiny_coordinates(z, z_ref)
    # the kernel's own z gives the kernel's codes exactly (same code path as without LayerNorm)
    idx_own, w_own = O.code_weights(z, T, k)
    np.testing.assert_array_equal(idx.cpu().numpy(), idx_own)
    assert rel_err(w.cpu().numpy(), w_own) < 1e-5
    # and equals torch's LayerNorm followed by the plain kernel up to the rounding of the normalisation
    u_t = torch.nn.functional.layer_norm(xt, (d_in,), ln[0], ln[1], eps)
    _, _, z_t = ops.hash_fwd(u_t, desc, want_z=True)
    assert rel_err(z, z_t.cpu().numpy()) < 5e-6
    # codes and weights alone (no z: for the diagonal shapes this is the transposing-layout kernel, whose
    # LayerNorm sums the row in another order): same codes wherever no coordinate is tiny, weights to 1e-5
    idx_c, w_c, _ = ops.hash_fwd(xt, desc, layer_norm=ln)
    clean = ~(np.abs(z_ref) < PAR.V_EPS).reshape(N, T, k).any(axis=-1)
    np.testing.assert_array_equal(idx_c.cpu().numpy()[clean], idx.cpu().numpy()[clean])
    assert rel_err(w_c.cpu().numpy()[clean], w.cpu().numpy()[clean]) < 1e-5
    # without codes (projection only) the same z comes out
    _, _, z_only = ops.hash_fwd(xt, desc, want_z=True, want_codes=False, layer_norm=ln)
    np.testing.assert_array_equal(z_only.cpu().numpy(), z)
    # no bias vector: beta = None
    _, _, z_nb = ops.hash_fwd(xt, desc, want_z=True, layer_norm=(ln[0], None, eps))
    z_nb_ref = O.project(O.layernorm(x, gamma, None, eps), pw, T * k, transpose_w=tw, had_scale=hs, mix_a=mix[0],
                         mix_b=mix[1], bias=pbias)
    assert rel_err(z_nb.cpu().numpy(), z_nb_ref) < 5e-6


@pytest.mark.parametrize("N,I,S,d,bf16", [(33, 18, 333, 64, False), (20, 512, 4096, 768, True), (5, 37, 1000, 1536, False),
                                          (40, 4608, 2000, 768, False), (9, 70, 900, 1024, True)])
def test_gather_residual_epilogue_is_exact(dev, N, I, S, d, bf16):
    from lookupffn_b200 import ops

    rng = np.random.RandomState(N + I)
    idx = rng.randint(0, S, size=(N, I)).astype(np.int32)
    w = rng.randn(N, I).astype(np.float32)
    tab = (0.02 * rng.randn(S, d)).astype(np.float32)
    bias = rng.randn(d).astype(np.float32)
    res = rng.randn(N, d).astype(np.float32)
    it, wt = torch.from_numpy(idx).to(dev), torch.from_numpy(w).to(dev)
    bt = torch.from_numpy(bias).to(dev)
    if bf16:
        tb, rb = O.f32_to_bf16_bits(tab), O.f32_to_bf16_bits(res)
        tt = torch.from_numpy(tb.view(np.int16)).to(dev).view(torch.bfloat16)
        rt = torch.from_numpy(rb.view(np.int16)).to(dev).view(torch.bfloat16)
        acc = O.gather(idx, w, tb, bias=bias)                       # fp32 sums + bias
        want = O.f32_to_bf16_bits(acc + O.bf16_bits_to_f32(rb))     # one more rounded add, then one rounding to bf16
        got = ops.weighted_vector_gather_add(it, tt, wt, bias=bt, residual=rt)
        np.testing.assert_array_equal(got.view(torch.int16).cpu().numpy().view(np.uint16), want)
    else:
        tt, rt = torch.from_numpy(tab).to(dev), torch.from_numpy(res).to(dev)
        want = O.gather(idx, w, tab, bias=bias) + res
        got = ops.weighted_vector_gather_add(it, tt, wt, bias=bt, residual=rt)
        np.testing.assert_array_equal(got.cpu().numpy(), want)
        # in place: the residual buffer is also the output
        from lookupffn_b200 import _lib as L

        buf = rt.clone()
        with torch.cuda.device(dev):
            L.check(L.lib().lffn_gather_fwd_residual(L.ptr(it), L.ptr(wt), L.ptr(tt), 0, L.ptr(buf), 0, N, I, S, d,
                                                     L.ptr(bt), L.ptr(buf), L.stream_ptr(dev)))
        np.testing.assert_array_equal(buf.cpu().numpy(), want)


@pytest.mark.parametrize("ptype,block,hidden", [("bh4", 64, 512), ("sign_hadamard", 1, 768), ("bh4", 16, 96)])
def test_module_fused_block_matches_unfused_and_oracle(dev, ptype, block, hidden):
    """LookupFFN.forward(x, residual=x) in inference = two kernels; against (a) the same module evaluated piece by
    piece (torch LayerNorm, hash, gather, adds) and (b) the CPU oracle's whole-layer forward with LayerNorm."""
    from lookupffn_b200 import LookupFFN

    torch.manual_seed(hidden)
    T, rows = 64, 256
    cfg = Namespace(hidden_size=hidden, ffn_num_table=T, ffn_table_size=rows, layer_norm_eps=1e-5,
                    projection_type=ptype, block_size=block)
    mod = LookupFFN(cfg, hidden).to(dev).eval()
    with torch.no_grad():
        mod.LayerNorm.weight.normal_(1.0, 0.1)
        mod.LayerNorm.bias.normal_(0.0, 0.05)
        mod.hash.projection.bias.normal_(0.0, 0.02)
    x = torch.randn(3, 50, hidden, device=dev)
    with torch.no_grad():
        y = mod(x, residual=x)                                      # fused
        u = mod.LayerNorm(x.reshape(-1, hidden))
        code, score = mod.hash(u)
        pieces = mod.gather(code, score, mod.tables) + x.reshape(-1, hidden)
        code_f, score_f = mod.hash(x.reshape(-1, hidden), layer_norm=(mod.LayerNorm.weight, mod.LayerNorm.bias, 1e-5))
    same = (code_f == code).all(dim=-1).cpu().numpy()
    assert same.sum() >= 0.9 * same.size
    yf = y.reshape(-1, hidden).cpu().numpy()
    assert rel_err(yf[same], pieces.cpu().numpy()[same]) < 1e-5
    # the oracle: same parameters, LayerNorm in double
    p = mod.hash.projection
    wk = p.weight.detach().cpu().numpy()
    y_ref = O.layer_fwd(x.reshape(-1, hidden).cpu().numpy(), wk, mod.tables.detach().cpu().numpy(), T, 8,
                        ln=(mod.LayerNorm.weight.detach().cpu().numpy(), mod.LayerNorm.bias.detach().cpu().numpy(), 1e-5),
                        had_scale=p.had_scale, mix_a=p.mix[0], mix_b=p.mix[1],
                        proj_bias=p.bias.detach().cpu().numpy(), bias=mod.bias.detach().cpu().numpy())
    y_ref = y_ref + x.reshape(-1, hidden).cpu().numpy()
    u_ref = O.layernorm(x.reshape(-1, hidden).cpu().numpy(), mod.LayerNorm.weight.detach().cpu().numpy(),
                        mod.LayerNorm.bias.detach().cpu().numpy(), 1e-5)
    z_ref = O.project(u_ref, wk, T * 8, had_scale=p.had_scale, mix_a=p.mix[0], mix_b=p.mix[1],
                      bias=p.bias.detach().cpu().numpy())
    idx_ref, _ = O.code_weights(z_ref, T, 8)
    clean = (code_f.cpu().numpy() == idx_ref).all(axis=-1)
    assert clean.sum() >= 0.9 * clean.size
    assert rel_err(yf[clean], y_ref[clean]) < 1e-5


def test_layer_fwd_ln_residual_entry_point(dev):
    """The C-ABI call itself, bf16 activations: equals lffn_hash_fwd_ln + lffn_gather_fwd_residual bit for bit."""
    from lookupffn_b200 import _lib as L
    from lookupffn_b200 import ops

    N, d_in, D, T, k, d_out = 300, 768, 1024, 128, 8, 768
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(N, d_in, generator=g, device=dev).bfloat16()
    res = torch.randn(N, d_out, generator=g, device=dev).bfloat16()
    tables = (0.02 * torch.randn(T << k, d_out, generator=g, device=dev)).bfloat16()
    signs = (2 * torch.randint(0, 2, (1, 2, D, 1, 1), generator=g, device=dev) - 1).float()
    gamma = 1 + 0.1 * torch.randn(d_in, generator=g, device=dev)
    beta = 0.05 * torch.randn(d_in, generator=g, device=dev)
    bias = torch.randn(d_out, generator=g, device=dev)
    desc = ops.make_hash_desc(d_in, signs, None, T, k, had_scale=1 / 32, mix_a=1.0, mix_b=0.0)
    out = torch.empty(N, d_out, dtype=torch.bfloat16, device=dev)
    iw = torch.empty(N, T, dtype=torch.int32, device=dev)
    ww = torch.empty(N, T, device=dev)
    with torch.cuda.device(dev):
        L.check(L.lib().lffn_layer_fwd_ln_residual(C.byref(desc), L.ptr(gamma), L.ptr(beta), 1e-5, L.ptr(x), L.BF16, N, 0,
                                                   T, L.ptr(tables), L.BF16, d_out, L.ptr(bias), L.ptr(res), L.ptr(out),
                                                   L.BF16, L.ptr(iw), L.ptr(ww), L.stream_ptr(dev)))
    idx, w, _ = ops.hash_fwd(x, desc, layer_norm=(gamma, beta, 1e-5))
    want = ops.weighted_vector_gather_add(idx, tables, w, bias=bias, residual=res)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    assert torch.equal(iw, idx)
    assert L.device_status(dev) == 0


T_CASES = [
    # N, d_in, D, T, k, weight_mode, bit_order, bias, (t_begin, t_count)
    (65, 768, 1024, 512, 8, O.WEIGHT_SCORE, O.MSB_FIRST, False, None),
    (33, 1000, 1024, 300, 8, O.WEIGHT_SCORE, O.LSB_FIRST, True, (64, 170)),
    (20, 1024, 1024, 100, 16, O.WEIGHT_SCORE, O.MSB_FIRST, True, (3, 90)),
    (17, 500, 512, 250, 4, O.WEIGHT_ONES, O.MSB_FIRST, True, (8, 200)),
    (29, 512, 512, 128, 8, O.WEIGHT_SOFT_FLIP, O.MSB_FIRST, False, None),
    (31, 200, 256, 500, 2, O.WEIGHT_SCORE, O.LSB_FIRST, True, None),
    (9, 256, 256, 700, 1, O.WEIGHT_SCORE, O.MSB_FIRST, False, (1, 650)),
    (40, 300, 512, 40, 16, O.WEIGHT_SOFT_FLIP, O.LSB_FIRST, True, (5, 30)),
    (50, 512, 512, 64, 8, O.WEIGHT_SCORE, O.MSB_FIRST, True, (12, 40)),     # range not a multiple of four tables
    # code lengths that do not divide D / 32: tables straddle lanes and rotations
    (33, 1000, 1024, 700, 6, O.WEIGHT_SCORE, O.MSB_FIRST, True, (100, 400)),
    (21, 1024, 1024, 1365, 6, O.WEIGHT_SCORE, O.MSB_FIRST, False, (1024, 341)),   # a rank's share of a large layer
    (19, 512, 512, 100, 10, O.WEIGHT_SCORE, O.LSB_FIRST, True, None),
    (14, 300, 512, 64, 12, O.WEIGHT_SOFT_FLIP, O.MSB_FIRST, False, (7, 50)),
    (27, 256, 256, 90, 3, O.WEIGHT_ONES, O.MSB_FIRST, True, (1, 88)),
    (11, 768, 1024, 40, 13, O.WEIGHT_SCORE, O.MSB_FIRST, True, None),
]


@pytest.mark.parametrize("case", T_CASES, ids=[f"t{i}" for i in range(len(T_CASES))])
@pytest.mark.parametrize("bf16", [False, True])
def test_transposing_hash_layout_matches_the_other_layouts_and_oracle(dev, case, bf16):
    """Codes-and-weights requests without z run the kernel that changes layout through shared memory in the middle
    of each transform; asking for z as well selects the shuffle kernels.  Same butterfly order, same operation
    order in the weights: indices and weights must be bit-identical, and the indices equal the oracle's."""
    from lookupffn_b200 import ops

    N, d_in, D, T, k, wm, bo, with_bias, rng_t = case
    rng = np.random.RandomState(N + T + k)
    R = max(1, -(-T * k // D))
    pw = (2.0 * rng.randint(0, 2, size=(R, 2, D, 1, 1)) - 1.0).astype(np.float32)
    pbias = (0.05 * rng.randn(T * k)).astype(np.float32) if with_bias else None
    x = rng.randn(N, d_in).astype(np.float32)
    hs = float(1.0 / np.sqrt(D))
    if bf16:
        xb = O.f32_to_bf16_bits(x)
        xt = torch.from_numpy(xb.view(np.int16)).to(dev).view(torch.bfloat16)
        x = O.bf16_bits_to_f32(xb)
    else:
        xt = torch.from_numpy(x).to(dev)
    tb, tc = (0, T) if rng_t is None else rng_t
    desc = ops.make_hash_desc(d_in, torch.from_numpy(pw).to(dev), None if pbias is None else torch.from_numpy(pbias).to(dev),
                              T, k, had_scale=hs, mix_a=1.0, mix_b=0.0, bit_order=bo, weight_mode=wm, tau=0.5)
    idx, w, _ = ops.hash_fwd(xt, desc, t_begin=tb, t_count=tc)                       # transposing layout
    idx2, w2, z = ops.hash_fwd(xt, desc, t_begin=tb, t_count=tc, want_z=True)        # shuffle layouts
    assert torch.equal(idx, idx2)
    assert torch.equal(w.view(torch.int32), w2.view(torch.int32))
    z_ref = O.project(x, pw, T * k, had_scale=hs, mix_a=1.0, mix_b=0.0, bias=pbias)[:, tb * k:(tb + tc) * k]
    np.testing.assert_array_equal(z.cpu().numpy(), z_ref)
    idx_ref, w_ref = O.code_weights(z_ref, tc, k, bit_order=bo, weight_mode=wm, tau=0.5)
    np.testing.assert_array_equal(idx.cpu().numpy(), idx_ref)
    assert rel_err(w.cpu().numpy(), w_ref) < 1e-5


def test_tracing_stage_times_and_nvtx_ranges(dev):
    """Tracing is off by default; with LFFN_TRACE_STAGE_TIMES a whole-layer call leaves the durations of its two
    kernels, and with LFFN_TRACE_NVTX the calls still work (the ranges go to whatever tool is attached, or nowhere)."""
    from lookupffn_b200 import _lib as L
    from lookupffn_b200 import ops

    lib = L.lib()
    h, g = C.c_float(-1), C.c_float(-1)
    N, d_in, D, T, k, d_out = 4096, 512, 512, 128, 8, 512
    gen = torch.Generator(device=dev).manual_seed(2)
    x = torch.randn(N, d_in, generator=gen, device=dev)
    tables = 0.02 * torch.randn(T << k, d_out, generator=gen, device=dev)
    signs = (2 * torch.randint(0, 2, (2, 2, D, 1, 1), generator=gen, device=dev) - 1).float()
    desc = ops.make_hash_desc(d_in, signs, None, T, k, had_scale=1 / 16, mix_a=1.0, mix_b=0.0)
    base = ops.layer_fwd(x, desc, tables)
    try:
        assert lib.lffn_trace_configure(L.TRACE_NVTX | L.TRACE_STAGE_TIMES) == 0
        y = ops.layer_fwd(x, desc, tables)
        with torch.cuda.device(dev):
            L.check(lib.lffn_trace_last_layer_times(C.byref(h), C.byref(g)))
        assert 0 < h.value < 50 and 0 < g.value < 50
        assert torch.equal(y, base)
        assert lib.lffn_trace_configure(8) == -1  # unknown flag
    finally:
        assert lib.lffn_trace_configure(0) == 0
