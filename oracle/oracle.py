"""numpy front end of the CPU oracle (oracle/lffn_oracle.c).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by the smoke test and by the
CPU-baseline legs of bench.py, always as the checker or the baseline -- never
by the lookupffn_b200 package.  Parity of this oracle with the reference is
pinned by tests/test_oracle_golden.py against vectors made by the reference's
own code (tests/golden/make_golden.py).

Array conventions: fp32 unless said otherwise; bf16 arrays are numpy uint16
holding the raw bit patterns.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

MSB_FIRST, LSB_FIRST = 0, 1
WEIGHT_SCORE, WEIGHT_ONES, WEIGHT_SOFT_FLIP = 0, 1, 2

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.ORACLE_SO
        src = os.path.join(_build.HERE, "lffn_oracle.c")
        if (not os.path.exists(path)) or (os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(path)):
            _build.build_oracle(verbose=False)
        _lib = C.CDLL(path)
        _lib.lffn_oracle_gather.restype = C.c_long
        _lib.lffn_oracle_layer_fwd.restype = C.c_long
        _lib.lffn_oracle_num_threads.restype = C.c_int
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads():
    return lib().lffn_oracle_num_threads()


def set_threads(n):
    lib().lffn_oracle_set_threads(C.c_int(n))


def f32_to_bf16_bits(a):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = _f32(a).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)
    return r


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def fwht(x, scale=1.0):
    x = _f32(x)
    N, D = x.shape
    out = np.empty_like(x)
    lib().lffn_oracle_fwht(_p(x), _p(out), C.c_long(N), C.c_int(D), C.c_float(scale))
    return out


def layernorm(x, gamma, beta, eps):
    x = _f32(x)
    N, d = x.shape
    g = None if gamma is None else _f32(gamma)
    b = None if beta is None else _f32(beta)
    out = np.empty_like(x)
    lib().lffn_oracle_layernorm(_p(x), _p(g), _p(b), C.c_float(eps), _p(out), C.c_long(N), C.c_int(d))
    return out


def padded_dim(d_in):
    return 1 << max(0, int(np.ceil(np.log2(d_in))))


def project(x, w, out_dim, transpose_w=False, had_scale=1.0, mix_a=0.7, mix_b=1 - 0.7, bias=None):
    """x [N, d_in]; w [R, S, D/BS, BS, BS] -> z [N, out_dim]."""
    x = _f32(x)
    w = _f32(w)
    N, d_in = x.shape
    R, S, NB, BS, BS2 = w.shape
    assert BS == BS2
    D = NB * BS
    assert D == padded_dim(d_in) or D >= d_in
    assert R * D >= out_dim
    b = None if bias is None else _f32(bias)
    z = np.empty((N, out_dim), dtype=np.float32)
    lib().lffn_oracle_project(_p(x), C.c_long(N), C.c_int(d_in), C.c_int(D), _p(w), C.c_int(BS), C.c_int(S),
                              C.c_int(R), C.c_int(int(transpose_w)), C.c_float(had_scale), C.c_float(mix_a),
                              C.c_float(mix_b), _p(b), C.c_int(out_dim), _p(z))
    return z


def project_dense(x, w, bias):
    x = _f32(x)
    w = _f32(w)
    N, d_in = x.shape
    out_dim = w.shape[0]
    b = None if bias is None else _f32(bias)
    z = np.empty((N, out_dim), dtype=np.float32)
    lib().lffn_oracle_project_dense(_p(x), C.c_long(N), C.c_int(d_in), _p(w), _p(b), C.c_int(out_dim), _p(z))
    return z


def code_weights(z, T, k, bit_order=MSB_FIRST, weight_mode=WEIGHT_SCORE, tau=0.5, add_offsets=True):
    """z [N, T*k] (or [N, T, k]) -> idx int32 [N, T*m], w fp32 [N, T*m]."""
    z = _f32(z).reshape(-1, T * k)
    N = z.shape[0]
    m = k + 1 if weight_mode == WEIGHT_SOFT_FLIP else 1
    idx = np.empty((N, T * m), dtype=np.int32)
    w = np.empty((N, T * m), dtype=np.float32)
    lib().lffn_oracle_code_weights(_p(z), C.c_long(N), C.c_int(T), C.c_int(k), C.c_int(bit_order),
                                   C.c_int(weight_mode), C.c_float(tau), C.c_int(int(add_offsets)), _p(idx), _p(w))
    return idx, w


def _table_arg(tables):
    if tables.dtype == np.uint16:
        return np.ascontiguousarray(tables), 1
    return _f32(tables), 0


def gather(idx, w, tables, bias=None, out_bf16=False, return_bad=False):
    """idx [N, I] int32 (already offset), w [N, I], tables [S, d] fp32 or uint16(bf16)."""
    idx = _i32(idx)
    w = _f32(w)
    tables, tb = _table_arg(tables)
    N, I = idx.shape
    S, d = tables.shape
    b = None if bias is None else _f32(bias)
    out = np.empty((N, d), dtype=np.uint16 if out_bf16 else np.float32)
    bad = lib().lffn_oracle_gather(_p(idx), _p(w), _p(tables), C.c_int(tb), _p(out), C.c_int(int(out_bf16)),
                                   C.c_long(N), C.c_int(I), C.c_long(S), C.c_int(d), _p(b))
    return (out, bad) if return_bad else out


def gather_bwd_weights(idx, dy, tables):
    idx = _i32(idx)
    dy = _f32(dy)
    tables, tb = _table_arg(tables)
    N, I = idx.shape
    S, d = tables.shape
    dw = np.empty((N, I), dtype=np.float32)
    lib().lffn_oracle_gather_bwd_weights(_p(idx), _p(dy), _p(tables), C.c_int(tb), _p(dw), C.c_long(N), C.c_int(I),
                                         C.c_long(S), C.c_int(d))
    return dw


def gather_bwd_tables(idx, w, dy, S):
    idx = _i32(idx)
    w = _f32(w)
    dy = _f32(dy)
    N, I = idx.shape
    d = dy.shape[1]
    dt = np.empty((S, d), dtype=np.float32)
    lib().lffn_oracle_gather_bwd_tables(_p(idx), _p(w), _p(dy), _p(dt), C.c_long(N), C.c_int(I), C.c_long(S),
                                        C.c_int(d))
    return dt


def layer_fwd(x, proj_w, tables, T, k, ln=None, transpose_w=False, had_scale=1.0, mix_a=0.7, mix_b=1 - 0.7,
              proj_bias=None, bit_order=MSB_FIRST, weight_mode=WEIGHT_SCORE, tau=0.5, bias=None, out_bf16=False):
    """Whole layer forward.  ln = (gamma, beta, eps) or None; tables [T, 2^k, d_out] or [T*2^k, d_out]."""
    x = _f32(x)
    proj_w = _f32(proj_w)
    N, d_in = x.shape
    R, S, NB, BS, _ = proj_w.shape
    D = NB * BS
    tables, tb = _table_arg(tables.reshape(-1, tables.shape[-1]))
    d_out = tables.shape[1]
    assert tables.shape[0] == T << k
    g = bta = None
    eps = 0.0
    if ln is not None:
        g, bta, eps = _f32(ln[0]), _f32(ln[1]), float(ln[2])
    pb = None if proj_bias is None else _f32(proj_bias)
    b = None if bias is None else _f32(bias)
    out = np.empty((N, d_out), dtype=np.uint16 if out_bf16 else np.float32)
    lib().lffn_oracle_layer_fwd(_p(x), C.c_long(N), C.c_int(d_in), _p(g), _p(bta), C.c_float(eps),
                                C.c_int(int(ln is not None)), C.c_int(D), _p(proj_w), C.c_int(BS), C.c_int(S),
                                C.c_int(R), C.c_int(int(transpose_w)), C.c_float(had_scale), C.c_float(mix_a),
                                C.c_float(mix_b), _p(pb), C.c_int(T), C.c_int(k), C.c_int(bit_order),
                                C.c_int(weight_mode), C.c_float(tau), _p(tables), C.c_int(tb), C.c_int(d_out), _p(b),
                                _p(out), C.c_int(int(out_bf16)))
    return out
