"""Operator functions of the LookupFFN path, with the reference's names and argument meaning
(src/roberta/models/prenorm_lookup/{bh4,compute_code_score,gather}/kernel.py), each calling the
sm_100a kernels of liblookupffn.so through its C ABI.  CUDA tensors only; a missing library or
a CPU tensor raises.
"""
import ctypes as C
import math

import torch

from . import _lib as L
from ._lib import (BF16, F32, LSB_FIRST, MSB_FIRST, WEIGHT_ONES, WEIGHT_SCORE, WEIGHT_SOFT_FLIP,  # noqa: F401
                   LookupFFNError)


SORTED_MAX_ROWS = 16384  # rows per table the sorted table-gradient kernel keeps counters for (csrc/gather_bwd.cu)


def _contig(t):
    return t if t.is_contiguous() else t.contiguous()


# ---- Hadamard ---------------------------------------------------------------------------------
def hadamard(inp, scale=1.0):
    """inp [N, D] (fp32 or bf16) -> inp @ H_D * scale, H the unnormalised Sylvester matrix.
    Reference: hadamard(inp) (bh4/fast_hadamard_transform/kernel.py:78-89)."""
    L.require_cuda(inp)
    assert inp.dim() == 2
    inp = _contig(inp)
    N, D = inp.shape
    out = torch.empty_like(inp)
    with torch.cuda.device(inp.device):
        L.check(L.lib().lffn_fwht(L.ptr(inp), L.ptr(out), N, D, L.dtype_code(inp.dtype), float(scale),
                                  L.stream_ptr(inp.device)))
    return out


class _Hadamard(torch.autograd.Function):
    """The transform is its own transpose: backward = the same transform
    (bh4/fast_hadamard_transform/kernel.py:47-54)."""

    @staticmethod
    def forward(ctx, inp, scale):
        ctx.scale = scale
        return hadamard(inp, scale)

    @staticmethod
    def backward(ctx, g):
        return hadamard(g.contiguous(), ctx.scale), None


def fast_hadamard_transform(X, scale=1.0):
    return _Hadamard.apply(X, scale)


# ---- hashing ------------------------------------------------------------------------------------
def make_hash_desc(d_in, proj_w, proj_bias, T, k, transpose_w=False, had_scale=1.0, mix_a=0.7, mix_b=1 - 0.7,
                   bit_order=MSB_FIRST, weight_mode=WEIGHT_SCORE, tau=0.5):
    """proj_w [R, S, D/BS, BS, BS] fp32 CUDA tensor.  The descriptor holds raw pointers and keeps a
    reference to the tensors so that they outlive it."""
    L.require_cuda(proj_w, proj_bias)
    assert proj_w.dtype == torch.float32 and proj_w.is_contiguous() and proj_w.dim() == 5
    R, S, NB, BS, BS2 = proj_w.shape
    assert BS == BS2
    if proj_bias is not None:
        assert proj_bias.dtype == torch.float32 and proj_bias.is_contiguous() and proj_bias.numel() == T * k
    desc = L.HashDesc(d_in=d_in, D=NB * BS, BS=BS, S=S, R=R, transpose_w=int(transpose_w), had_scale=had_scale,
                      mix_a=mix_a, mix_b=mix_b, T=T, k=k, bit_order=bit_order, weight_mode=weight_mode, tau=tau,
                      proj_w=proj_w.data_ptr(), proj_bias=0 if proj_bias is None else proj_bias.data_ptr())
    desc._keepalive = (proj_w, proj_bias)  # the struct holds raw pointers; pin the tensors to its lifetime
    return desc


def hash_fwd(x, desc, t_begin=0, t_count=None, want_z=False, want_codes=True, layer_norm=None):
    """x [N, d_in] -> (idx int32 [N, t_count*m] with table offsets, w fp32 [N, t_count*m], z or None).
    Reference: Hashing.forward (lookup.py:64-77) + the offsets of LookupFFN.gather (lookup.py:126).
    layer_norm = (weight, bias, eps): the module's LayerNorm (lookup.py:99) applied inside the kernel's load."""
    L.require_cuda(x)
    if x.dtype == torch.float16:  # the reference trains under fp16 autocast; the kernels read fp32 or bf16
        x = x.float()
    x = _contig(x)
    N = x.shape[0]
    t_count = desc.T - t_begin if t_count is None else t_count
    m = desc.k + 1 if desc.weight_mode == WEIGHT_SOFT_FLIP else 1
    idx = w = z = None
    if want_codes:
        idx = torch.empty((N, t_count * m), dtype=torch.int32, device=x.device)
        w = torch.empty((N, t_count * m), dtype=torch.float32, device=x.device)
    if want_z:
        z = torch.empty((N, t_count * desc.k), dtype=torch.float32, device=x.device)
    g = b = None
    eps = 0.0
    if layer_norm is not None:
        g, b, eps = layer_norm
        g = _contig(g.detach().float())
        b = None if b is None else _contig(b.detach().float())
        L.require_cuda(g, b)
    with torch.cuda.device(x.device):
        L.check(L.lib().lffn_hash_fwd_ln(C.byref(desc), L.ptr(g), L.ptr(b), float(eps), L.ptr(x),
                                         L.dtype_code(x.dtype), N, t_begin, t_count, L.ptr(idx), L.ptr(w), L.ptr(z),
                                         L.stream_ptr(x.device)))
    return idx, w, z


def layer_fwd(x, desc, tables, bias=None, t_begin=0, t_count=None, out_dtype=None):
    """Hash -> gather -> + bias for tables [t_begin, t_begin+t_count) through lffn_layer_fwd: one fused kernel when
    the shape allows it, otherwise the hash and gather kernels with workspaces allocated here.
    Reference: LookupFFN._forward after LayerNorm (lookup.py:101-110)."""
    L.require_cuda(x, tables, bias)
    x, tables = _contig(x), _contig(tables)
    N = x.shape[0]
    t_count = desc.T - t_begin if t_count is None else t_count
    m = desc.k + 1 if desc.weight_mode == WEIGHT_SOFT_FLIP else 1
    d_out = tables.shape[1]
    out_dtype = tables.dtype if out_dtype is None else out_dtype
    out = torch.empty((N, d_out), dtype=out_dtype, device=x.device)
    idx = torch.empty((N, t_count * m), dtype=torch.int32, device=x.device)
    w = torch.empty((N, t_count * m), dtype=torch.float32, device=x.device)
    if bias is not None:
        bias = _contig(bias.float())
    with torch.cuda.device(x.device):
        L.check(L.lib().lffn_layer_fwd(C.byref(desc), L.ptr(x), L.dtype_code(x.dtype), N, t_begin, t_count, L.ptr(tables),
                                       L.dtype_code(tables.dtype), d_out, L.ptr(bias), L.ptr(out),
                                       L.dtype_code(out_dtype), L.ptr(idx), L.ptr(w), L.stream_ptr(x.device)))
    return out


def bh4(x, w, training=False, transpose_w=False, had_scale=1.0):
    """x [N, D] (D a power of two), w [R, S, D/BS, BS, BS] -> [N, R*D]: R repeats of S x (block-diagonal
    multiply, Hadamard).  Reference: bh4(x, w, training) (bh4/kernel.py:10-36), CUDA semantics."""
    L.require_cuda(x, w)
    R, S, NB, BS, _ = w.shape
    D = NB * BS
    assert x.shape[1] == D
    desc = make_hash_desc(D, _contig(w.float()), None, R * D, 1, transpose_w=transpose_w, had_scale=had_scale,
                          mix_a=1.0, mix_b=0.0, weight_mode=WEIGHT_ONES)
    _, _, z = hash_fwd(x, desc, want_z=True, want_codes=False)
    return z


def compute_code_score(hash_scores, training=False, bit_order=MSB_FIRST, weight_mode=WEIGHT_SCORE, tau=0.5,
                       add_offsets=False):
    """hash_scores [N, T, k] fp32 -> (code int32 [N, T*m], score fp32 [N, T*m]).
    Reference: compute_code_score(hash_scores, training) (compute_code_score/kernel.py:22-55)."""
    L.require_cuda(hash_scores)
    assert hash_scores.dim() == 3 and hash_scores.dtype == torch.float32
    z = _contig(hash_scores)
    N, T, k = z.shape
    m = k + 1 if weight_mode == WEIGHT_SOFT_FLIP else 1
    code = torch.empty((N, T * m), dtype=torch.int32, device=z.device)
    score = torch.empty((N, T * m), dtype=torch.float32, device=z.device)
    with torch.cuda.device(z.device):
        L.check(L.lib().lffn_code_weights(L.ptr(z), N, T, k, bit_order, weight_mode, float(tau), int(add_offsets),
                                          L.ptr(code), L.ptr(score), L.stream_ptr(z.device)))
    return code, score


def code_weights_bwd(z, dw, weight_mode=WEIGHT_SCORE, tau=0.5):
    """dz [N, T, k] from dw [N, T*m]: the gradient autograd derives from compute_code_score_torch
    (compute_code_score/kernel.py:43-55)."""
    L.require_cuda(z, dw)
    z, dw = _contig(z), _contig(dw.float())
    N, T, k = z.shape
    dz = torch.empty_like(z)
    with torch.cuda.device(z.device):
        L.check(L.lib().lffn_code_weights_bwd(L.ptr(z), L.ptr(dw), N, T, k, weight_mode, float(tau), L.ptr(dz),
                                              L.stream_ptr(z.device)))
    return dz


class CodeScore(torch.autograd.Function):
    """z [N, T, k] -> (row indices with table offsets, weights); the weights are differentiable in z."""

    @staticmethod
    def forward(ctx, z, bit_order, weight_mode, tau):
        z = _contig(z.float())
        idx, w = compute_code_score(z, bit_order=bit_order, weight_mode=weight_mode, tau=tau, add_offsets=True)
        ctx.save_for_backward(z)
        ctx.weight_mode, ctx.tau = weight_mode, tau
        ctx.mark_non_differentiable(idx)
        return idx, w

    @staticmethod
    def backward(ctx, _didx, dw):
        (z,) = ctx.saved_tensors
        return code_weights_bwd(z, dw, ctx.weight_mode, ctx.tau), None, None, None


# Stage inputs kept by the training forward for the backward pass (what the reference's autograd keeps for its einsum
# chain): up to this many bytes per call; above it the backward pass recomputes them.
PROJECTION_SAVE_LIMIT_BYTES = 2 << 30


def proj_fwd_train(x, kernel_weight, bias, out_dim, had_scale, mix_a, mix_b):
    """z = BH4(x) [N, out_dim] through lffn_proj_fwd_train, plus the stage inputs for proj_bwd (64 x 64 blocks)."""
    N = x.shape[0]
    desc = make_hash_desc(x.shape[1], kernel_weight, bias, out_dim, 1, transpose_w=True, had_scale=had_scale,
                          mix_a=mix_a, mix_b=mix_b, weight_mode=WEIGHT_ONES)
    lib = L.lib()
    nbytes = lib.lffn_proj_acts_bytes(C.byref(desc), N)
    acts = torch.empty(nbytes // 4, dtype=torch.float32, device=x.device)
    z = torch.empty((N, out_dim), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        L.check(lib.lffn_proj_fwd_train(C.byref(desc), L.ptr(x), L.dtype_code(x.dtype), N, L.ptr(z), L.ptr(acts), nbytes,
                                        L.stream_ptr(x.device)))
    return z, acts


def proj_bwd(x, weight, kernel_weight, out_dim, dz, had_scale, mix_a, mix_b, need_dw=True, need_dbias=True, acts=None):
    """Backward of z = BH4(x) for 64 x 64 blocks through lffn_proj_bwd: returns (du [N, D], dweight in the parameter's
    layout or None, dbias or None).  weight [R, S, NB, 64(o), 64(i)] is the parameter, kernel_weight its [.., i, o]
    copy that the forward fast path streams, acts the stage inputs from proj_fwd_train (None: recomputed)."""
    R, S, NB, BS, _ = weight.shape
    D = NB * BS
    N = x.shape[0]
    dev = x.device
    desc = make_hash_desc(x.shape[1], kernel_weight, None, out_dim, 1, transpose_w=True, had_scale=had_scale,
                          mix_a=mix_a, mix_b=mix_b, weight_mode=WEIGHT_ONES)
    w_oi = _contig(weight.detach().float())
    dz = _contig(dz.float())
    du = torch.empty((N, D), dtype=torch.float32, device=dev)
    dw = torch.empty(weight.shape, dtype=torch.float32, device=dev) if need_dw else None
    dbias = torch.empty(out_dim, dtype=torch.float32, device=dev) if need_dbias else None
    lib = L.lib()
    nbytes = lib.lffn_proj_bwd_ws_bytes(C.byref(desc), N)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        L.check(lib.lffn_proj_bwd(C.byref(desc), L.ptr(w_oi), L.ptr(x), L.dtype_code(x.dtype), N, L.ptr(dz), L.ptr(du),
                                  L.ptr(dw), L.ptr(dbias), L.ptr(acts), L.ptr(ws), nbytes, L.stream_ptr(dev)))
    return du, dw, dbias


LAYERNORM_BWD_SIZES = (256, 512, 768, 1024)


def layernorm_bwd(x, du, gamma, eps):
    """Gradients of u = LayerNorm(x) * gamma + beta (torch.nn.LayerNorm over the last dimension) through
    lffn_layernorm_bwd: returns (dx [N, d], dgamma [d], dbeta [d]), fp32, deterministic."""
    L.require_cuda(x, du, gamma)
    d = x.shape[-1]
    x2, du2 = _contig(x.reshape(-1, d).float()), _contig(du.reshape(-1, d).float())
    g = _contig(gamma.detach().float())
    N, dev = x2.shape[0], x2.device
    dx = torch.empty_like(x2)
    dgamma = torch.empty(d, dtype=torch.float32, device=dev)
    dbeta = torch.empty(d, dtype=torch.float32, device=dev)
    lib = L.lib()
    nbytes = lib.lffn_layernorm_bwd_ws_bytes(d)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        L.check(lib.lffn_layernorm_bwd(L.ptr(x2), L.ptr(du2), L.ptr(g), N, d, float(eps), L.ptr(dx), L.ptr(dgamma),
                                       L.ptr(dbeta), L.ptr(ws), nbytes, L.stream_ptr(dev)))
    return dx.reshape(x.shape), dgamma, dbeta


class LayerNormFn(torch.autograd.Function):
    """The layer's LayerNorm for training: torch's forward kernel, this library's backward (lffn_layernorm_bwd), which
    recomputes the row statistics from x instead of keeping them."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        ctx.save_for_backward(x, weight)
        ctx.eps = eps
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)

    @staticmethod
    def backward(ctx, du):
        x, weight = ctx.saved_tensors
        dx, dgamma, dbeta = layernorm_bwd(x, du, weight, ctx.eps)
        return dx.to(x.dtype), dgamma.to(weight.dtype), dbeta.to(weight.dtype), None


def layer_norm(x, ln):
    """ln(x) for an nn.LayerNorm `ln`; with this library's backward kernel when x is an fp32 CUDA tensor of a covered
    width and gradients are being recorded, torch's module otherwise."""
    if (torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.float32 and ln.elementwise_affine and ln.bias is not None
            and x.shape[-1] in LAYERNORM_BWD_SIZES and (x.requires_grad or ln.weight.requires_grad)):
        return LayerNormFn.apply(x, ln.weight, ln.bias, ln.eps)
    return ln(x)


class Projection(torch.autograd.Function):
    """z = BH4(x): forward by the fused hash kernel (projection only).  Backward for the reference's shape (64 x 64
    blocks, D a multiple of 256) is lffn_proj_bwd: the stage inputs are recomputed and the chain walked in reverse by
    this library's own kernels.  Other block sizes walk the same chain with the Hadamard kernel and torch.einsum for
    the block-diagonal factors, as the reference's autograd does (bh4/kernel.py:23-36)."""

    @staticmethod
    def forward(ctx, x, weight, bias, had_scale, mix_a, mix_b, kernel_weight, kernel_transposed):
        R, S, NB, BS, _ = weight.shape
        D = NB * BS
        out_dim = bias.numel()
        desc = make_hash_desc(x.shape[1], kernel_weight, _contig(bias.detach().float()), out_dim, 1,
                              transpose_w=kernel_transposed, had_scale=had_scale, mix_a=mix_a, mix_b=mix_b,
                              weight_mode=WEIGHT_ONES)
        if x.dtype == torch.float16:
            x = x.float()
        x = _contig(x)
        fast = BS == 64 and D % 256 == 0 and D <= 1024 and kernel_transposed
        acts = None
        if fast and R * S * (-(-x.shape[0] // 32)) * D * 32 * 4 <= PROJECTION_SAVE_LIMIT_BYTES:
            z, acts = proj_fwd_train(x, kernel_weight, _contig(bias.detach().float()), out_dim, had_scale, mix_a, mix_b)
        else:
            _, _, z = hash_fwd(x, desc, want_z=True, want_codes=False)
        ctx.save_for_backward(x, weight, kernel_weight if fast else None, acts)
        ctx.meta = (D, BS, S, R, out_dim, had_scale, mix_a, mix_b, fast)
        return z

    @staticmethod
    def backward(ctx, dz):
        x, weight, kernel_weight, acts = ctx.saved_tensors
        D, BS, S, R, out_dim, had_scale, mix_a, mix_b, fast = ctx.meta
        N, d_in = x.shape
        if fast:
            du, dweight, dbias = proj_bwd(x, weight, kernel_weight, out_dim, dz, had_scale, mix_a, mix_b,
                                          need_dw=ctx.needs_input_grad[1], need_dbias=ctx.needs_input_grad[2], acts=acts)
            dx = du[:, :d_in].to(x.dtype) if ctx.needs_input_grad[0] else None
            if dweight is not None:
                dweight = dweight.to(weight.dtype)
            return dx, dweight, dbias, None, None, None, None, None
        NB = D // BS
        dz = _contig(dz.float())
        dbias = dz.sum(0) if ctx.needs_input_grad[2] else None
        dzp = dz if out_dim == R * D else torch.nn.functional.pad(dz, (0, R * D - out_dim))
        u = x.float()
        if d_in < D:
            u = torch.nn.functional.pad(u, (0, D - d_in))
        du = (mix_b * dzp.reshape(N, R, D).sum(1)) if mix_b != 0 else torch.zeros(N, D, device=x.device)
        need_w = ctx.needs_input_grad[1]
        dweight = torch.zeros_like(weight, dtype=torch.float32) if need_w else None
        w = weight.detach().float()
        for r in range(R):
            ys = []
            y = u
            for j in range(S):  # recompute the inputs of every stage
                ys.append(y)
                if BS == 1:
                    t = y * w[r, j].reshape(D)
                else:
                    t = torch.einsum("bni,noi->bno", y.reshape(N, NB, BS), w[r, j]).reshape(N, D)
                y = hadamard(_contig(t), had_scale) if j < S - 1 else None
            g = _contig(mix_a * dzp[:, r * D:(r + 1) * D])
            for j in range(S - 1, -1, -1):
                g = hadamard(g, had_scale)
                if BS == 1:
                    if need_w:
                        dweight[r, j] = (g * ys[j]).sum(0).reshape(NB, 1, 1)
                    g = _contig(g * w[r, j].reshape(D))
                else:
                    g3 = g.reshape(N, NB, BS)
                    if need_w:
                        dweight[r, j] = torch.einsum("bno,bni->noi", g3, ys[j].reshape(N, NB, BS))
                    g = _contig(torch.einsum("bno,noi->bni", g3, w[r, j]).reshape(N, D))
            du = du + g
        dx = du[:, :d_in].to(x.dtype) if ctx.needs_input_grad[0] else None
        if need_w:
            dweight = dweight.to(weight.dtype)
        return dx, dweight, dbias, None, None, None, None, None


# ---- gather and its backward ------------------------------------------------------------------------
def _check_gather_args(indexes, source, weights):
    # the reference's asserts (gather/cuda/kernel.py:28-43) minus its `index_size % 2` and
    # `vector_dim % 64` limits, which these kernels do not have
    L.require_cuda(indexes, source, weights)
    assert indexes.dtype == torch.int32, indexes.dtype
    assert source.dtype in (torch.float32, torch.bfloat16), source.dtype
    assert weights.dtype == torch.float32, weights.dtype
    assert indexes.dim() == 2 and source.dim() == 2 and weights.dim() == 2
    assert weights.shape == indexes.shape


def weighted_vector_gather_add(indexes, source, weights, bias=None, out_dtype=None, residual=None):
    """outputs[b] = sum_i weights[b, i] * source[indexes[b, i]] (+ bias) (+ residual[b]).
    Reference: weighted_vector_gather_add(indexes, source, weights) (gather/cuda/kernel.py:22-70); the bias add
    of lookup.py:108 and the residual add of layer.py:75-78 ride in the kernel's epilogue when given."""
    _check_gather_args(indexes, source, weights)
    indexes, source, weights = _contig(indexes), _contig(source), _contig(weights)
    N, I = indexes.shape
    S, d = source.shape
    out_dtype = source.dtype if out_dtype is None else out_dtype
    out = torch.empty((N, d), dtype=out_dtype, device=source.device)
    if bias is not None:
        bias = _contig(bias.float())
    if residual is not None:
        L.require_cuda(residual)
        residual = _contig(residual.reshape(N, d).to(out_dtype))
    with torch.cuda.device(source.device):
        L.check(L.lib().lffn_gather_fwd_residual(L.ptr(indexes), L.ptr(weights), L.ptr(source),
                                                 L.dtype_code(source.dtype), L.ptr(out), L.dtype_code(out_dtype), N, I,
                                                 S, d, L.ptr(bias), L.ptr(residual), L.stream_ptr(source.device)))
    return out


def indexed_inner_product(indexes, source_1, source_2):
    """outputs[b, i] = <source_1[b], source_2[indexes[b, i]]>, source_1 fp32 [N, d].
    Reference: indexed_inner_product (gather/cuda/kernel.py:72-122)."""
    L.require_cuda(indexes, source_1, source_2)
    assert indexes.dtype == torch.int32 and source_1.dtype == torch.float32
    indexes, source_1, source_2 = _contig(indexes), _contig(source_1), _contig(source_2)
    N, I = indexes.shape
    S, d = source_2.shape
    assert source_1.shape == (N, d)
    out = torch.empty((N, I), dtype=torch.float32, device=source_2.device)
    with torch.cuda.device(source_2.device):
        L.check(L.lib().lffn_gather_bwd_weights(L.ptr(indexes), L.ptr(source_1), L.ptr(source_2),
                                                L.dtype_code(source_2.dtype), L.ptr(out), N, I, S, d,
                                                L.stream_ptr(source_2.device)))
    return out


def weighted_vector_scatter_add(indexes, source, weights, output_size, structure=None):
    """outputs[indexes[b, i]] += weights[b, i] * source[b]; outputs fp32 [output_size, d].
    Reference: weighted_vector_scatter_add (gather/cuda/kernel.py:124-173).
    structure=(T, m, rows) declares the layer's index structure (entry (b, t*m+c) lies in table t of
    `rows` rows) and selects the deterministic sorted kernel; None accepts any index list.  Shapes the sorted
    kernel does not cover (more than SORTED_MAX_ROWS rows per table, or 2^31 entries and more) go to the
    general kernel, as the reference's scatter-add handles any table size."""
    L.require_cuda(indexes, source, weights)
    assert indexes.dtype == torch.int32 and source.dtype == torch.float32 and weights.dtype == torch.float32
    indexes, source, weights = _contig(indexes), _contig(source), _contig(weights)
    N, I = indexes.shape
    d = source.shape[1]
    out = torch.empty((output_size, d), dtype=torch.float32, device=source.device)
    lib = L.lib()
    with torch.cuda.device(source.device):
        if structure is not None:
            T, m, rows = structure
            assert T * m == I and T * rows == output_size
            if rows > SORTED_MAX_ROWS or N * I >= 2 ** 31:
                structure = None
        if structure is None:
            L.check(lib.lffn_gather_bwd_tables(L.ptr(indexes), L.ptr(weights), L.ptr(source), L.ptr(out), N, I,
                                               output_size, d, L.stream_ptr(source.device)))
        else:
            nbytes = lib.lffn_gather_bwd_tables_sorted_scratch_bytes(N, T, m, rows)
            scratch = torch.empty(nbytes, dtype=torch.uint8, device=source.device)
            L.check(lib.lffn_gather_bwd_tables_sorted(L.ptr(indexes), L.ptr(weights), L.ptr(source), L.ptr(out), N, T,
                                                      m, rows, d, L.ptr(scratch), nbytes,
                                                      L.stream_ptr(source.device)))
    return out


class WeightedVectorGatherAdd(torch.autograd.Function):
    """Reference: WeightedVectorGatherAdd (gather/cuda/kernel.py:175-202): saves (indexes, source,
    weights); backward returns (None, grad_source, grad_weights)."""

    @staticmethod
    def forward(ctx, indexes, source, weights, structure=None, bias=None):
        """bias (optional, [d]): the `outputs + self.bias` of lookup.py:108 in the kernel's epilogue; its gradient
        is the column sum of grad_outputs (lffn_bias_grad)."""
        indexes, source, weights = _contig(indexes), _contig(source), _contig(weights)
        ctx.save_for_backward(indexes, source, weights)
        ctx.structure = structure
        ctx.bias_dtype = None if bias is None else bias.dtype
        return weighted_vector_gather_add(indexes, source, weights, bias=bias)

    @staticmethod
    def backward(ctx, grad_outputs):
        indexes, source, weights = ctx.saved_tensors
        g = _contig(grad_outputs.float())
        grad_source = grad_weights = grad_bias = None
        if ctx.needs_input_grad[2]:
            grad_weights = indexed_inner_product(indexes, g, source)
        if ctx.needs_input_grad[1]:
            grad_source = weighted_vector_scatter_add(indexes, g, weights, source.shape[0], ctx.structure)
            grad_source = grad_source.to(source.dtype)
        if ctx.bias_dtype is not None and ctx.needs_input_grad[4]:
            grad_bias = bias_grad(g).to(ctx.bias_dtype)
        return None, grad_source, grad_weights, None, grad_bias


def bias_grad(dy):
    """Column sums of dy [N, d] (fp32) through lffn_bias_grad: deterministic."""
    L.require_cuda(dy)
    dy = _contig(dy.reshape(-1, dy.shape[-1]).float())
    N, d = dy.shape
    out = torch.empty(d, dtype=torch.float32, device=dy.device)
    lib = L.lib()
    nbytes = lib.lffn_bias_grad_ws_bytes(d)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dy.device)
    with torch.cuda.device(dy.device):
        L.check(lib.lffn_bias_grad(L.ptr(dy), N, d, L.ptr(out), L.ptr(ws), nbytes, L.stream_ptr(dy.device)))
    return out


def weighted_gather_add(indexes, source, weights, structure=None, bias=None):
    return WeightedVectorGatherAdd.apply(indexes, source, weights, structure, bias)


def gather(indices, weights, tables, training=False, structure=None, bias=None):
    """Reference: gather(indices, weights, tables, training) (gather/kernel.py:11-25).  `indices`
    already carry the table offsets; tables is [S, d]; bias (optional) is added in the kernel."""
    return weighted_gather_add(indices, tables, weights, structure, bias)


def padded_dim(d_in):
    return int(2 ** math.ceil(math.log2(d_in)))
