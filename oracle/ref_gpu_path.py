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
