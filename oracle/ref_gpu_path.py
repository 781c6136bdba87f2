"""The reference's GPU evaluation of a LookupFFN layer, restated around the reference's own CUDA kernels.

TEST AND COMPARATOR INFRASTRUCTURE: used by tests and by the benchmark's baseline leg as the GPU comparator; the
product never calls it.

The reference's Python cannot travel to the GPU machine, its compiled CUDA extensions (oracle/_ref) can.  This
file restates the few lines of Python that sit between them, following the reference line by line:

  projection     lookup.py:29-39 (pad, 0.7 * bh4 + 0.3 * x.repeat, slice, + bias) and bh4/kernel.py:23-36
                 (per rotation and stage: torch.einsum("bni,noi->bno") then the Hadamard kernel)
  code + score   compute_code_score/kernel.py:43-55 (elementwise torch on the GPU)
  gather         lookup.py:101-129 (offsets, flatten tables, gather kernel, + bias)

`fht` is the reference's fast_hadamard_transform_kernel module, `gat` its gather_add module.
"""
import math

import torch


def bh4_reference_gpu(x, weight, fht):
    """x [N, D] fp32, weight [R, 4, NB, BS, BS] -> [N, R * D] (bh4/kernel.py:23-36)."""
    N, D = x.shape
    R, S, NB, BS, _ = weight.shape
    outs = []
    for r in range(R):
        y = x
        for s in range(S):
            y = torch.einsum("bni,noi->bno", y.reshape(N, NB, BS), weight[r, s]).reshape(N, D)
            y = fht.fast_hadamard_transform(y.contiguous())
        outs.append(y)
    return torch.cat(outs, dim=-1)


def projection_reference_gpu(x, weight, bias, out_dim, fht, decay=0.7):
    """lookup.py:29-39."""
    N, d_in = x.shape
    D = int(2 ** math.ceil(math.log2(d_in)))
    R = weight.shape[0]
    if D > d_in:
        x = torch.cat([x, torch.zeros(N, D - d_in, dtype=x.dtype, device=x.device)], dim=-1)
    z = decay * bh4_reference_gpu(x, weight, fht) + (1 - decay) * x.repeat(1, R)
    return z[:, :out_dim] + bias


def code_score_reference_gpu(z):
    """z [N, T, k] -> (int32 codes MSB first, fp32 scores) (compute_code_score/kernel.py:43-55)."""
    k = z.shape[-1]
    bits = (z > 0).int()
    place = 2 ** torch.arange(k - 1, -1, -1, device=z.device, dtype=torch.int32)
    code = (bits * place).sum(dim=-1).int()
    a = torch.abs(z)
    score = a.sum(dim=-1) / (1 + torch.exp(-2 * a)).prod(dim=-1)
    return code, score


def lookupffn_reference_gpu(mod, hidden_states, fht, gat):
    """forward of a LookupFFN-shaped module (parameters LayerNorm, hash.projection.{weight,bias}, tables, bias) the
    way the reference evaluates it on a GPU (lookup.py:101-129)."""
    shape = hidden_states.shape[:-1]
    h = hidden_states.reshape(-1, hidden_states.shape[-1])
    h = mod.LayerNorm(h)
    T, rows, d = mod.tables.shape
    k = int(math.log2(rows))
    z = projection_reference_gpu(h.float(), mod.hash.projection.weight, mod.hash.projection.bias, T * k, fht)
    code, score = code_score_reference_gpu(z.reshape(-1, T, k))
    code = (code + torch.arange(T, device=code.device, dtype=torch.int32)[None, :] * rows).contiguous()
    out = torch.zeros(h.shape[0], d, dtype=torch.float32, device=h.device)
    gat.weighted_vector_gather_add_fp32(code, mod.tables.reshape(T * rows, d), score.contiguous(), out)
    return (out + mod.bias).reshape(*shape, d)


def reference_autograd_functions(fht, gat):
    """The reference's two autograd wrappers around its CUDA kernels, restated: the Hadamard transform whose backward
    is the same transform (bh4/fast_hadamard_transform/kernel.py:47-54) and the weighted gather-add whose backward
    is its inner-product and scatter-add kernels (gather/cuda/kernel.py:175-202, fp32 branches of :110-118 and
    :159-170).  Returns (hadamard, gather) callables."""

    class Hadamard(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            return fht.fast_hadamard_transform(x.contiguous())

        @staticmethod
        def backward(ctx, g):
            return fht.fast_hadamard_transform(g.contiguous())

    class Gather(torch.autograd.Function):
        @staticmethod
        def forward(ctx, indexes, source, weights):
            indexes, source, weights = indexes.contiguous(), source.contiguous(), weights.contiguous()
            ctx.save_for_backward(indexes, source, weights)
            out = torch.zeros(indexes.shape[0], source.shape[1], dtype=torch.float32, device=source.device)
            gat.weighted_vector_gather_add_fp32(indexes, source, weights, out)
            return out

        @staticmethod
        def backward(ctx, grad_outputs):
            grad_outputs = grad_outputs.contiguous()
            indexes, source, weights = ctx.saved_tensors
            grad_weights = torch.zeros(indexes.shape, dtype=torch.float32, device=source.device)
            gat.indexed_inner_product_fp32(indexes, grad_outputs, source, grad_weights)
            grad_source = torch.zeros_like(source)
            gat.weighted_vector_scatter_add_fp32(indexes, grad_outputs, weights, grad_source)
            return None, grad_source, grad_weights

    return Hadamard.apply, Gather.apply


def lookupffn_reference_gpu_training(mod, hidden_states, fht, gat):
    """The differentiable forward of a LookupFFN-shaped module the way the reference trains it on a GPU: autograd
    over nn.LayerNorm, torch.einsum + its Hadamard function per stage (bh4/kernel.py:23-36), the elementwise score
    (compute_code_score/kernel.py:43-55; the code carries no gradient) and its gather function (lookup.py:98-129)."""
    hadamard, gather = reference_autograd_functions(fht, gat)
    shape = hidden_states.shape[:-1]
    h = mod.LayerNorm(hidden_states.reshape(-1, hidden_states.shape[-1]))
    T, rows, d = mod.tables.shape
    k = int(math.log2(rows))
    N, d_in = h.shape
    weight, bias = mod.hash.projection.weight, mod.hash.projection.bias
    R, S, NB, BS, _ = weight.shape
    D = NB * BS
    x = h if D == d_in else torch.cat([h, torch.zeros(N, D - d_in, dtype=h.dtype, device=h.device)], dim=-1)
    outs = []
    for r in range(R):
        y = x
        for s in range(S):
            y = torch.einsum("bni,noi->bno", y.reshape(N, NB, BS), weight[r, s]).reshape(N, D)
            y = hadamard(y)
        outs.append(y)
    z = (0.7 * torch.cat(outs, dim=-1) + (1 - 0.7) * x.repeat(1, R))[:, :T * k] + bias
    zz = z.reshape(N, T, k)
    with torch.no_grad():
        place = 2 ** torch.arange(k - 1, -1, -1, device=z.device, dtype=torch.int32)
        code = ((zz > 0).int() * place).sum(dim=-1).int()
        code = (code + torch.arange(T, device=z.device, dtype=torch.int32)[None, :] * rows).contiguous()
    a = torch.abs(zz)
    score = a.sum(dim=-1) / (1 + torch.exp(-2 * a)).prod(dim=-1)
    out = gather(code, mod.tables.reshape(T * rows, d), score.contiguous())
    return (out + mod.bias).reshape(*shape, d)
