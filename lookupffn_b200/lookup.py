"""LookupFFN: the hashed-lookup-table replacement of a transformer feed-forward block.

Drop-in for the reference's module (src/roberta/models/prenorm_lookup/lookup.py:10-129): same
constructor `LookupFFN(config, output_size)`, same `forward(hidden_states)`, same parameter names
and shapes (`LayerNorm.weight/bias`, `hash.projection.weight/bias`, `tables`, `bias`), so a
reference checkpoint loads with strict=True.  The work is done by the sm_100a kernels of
liblookupffn.so; tensors must live on a CUDA device (there is no CPU path).

Config attributes read (reference names): hidden_size, ffn_num_table, ffn_table_size,
layer_norm_eps, projection_type ("bh4" | "dense" | "sign_hadamard"), block_size.
Optional attributes (defaults = reference behaviour):
  lookup_bit_order    "msb" (reference) | "lsb"
  lookup_weight_mode  "score" (reference) | "ones" | "soft_flip"
  lookup_tau          temperature of soft_flip (0.5)
  lookup_table_dtype  torch.float32 (reference) | torch.bfloat16
"""
import math

import numpy as np
import torch
import torch.nn as nn

from . import ops
from ._lib import MSB_FIRST, LSB_FIRST, WEIGHT_ONES, WEIGHT_SCORE, WEIGHT_SOFT_FLIP

_BIT_ORDER = {"msb": MSB_FIRST, "lsb": LSB_FIRST}
_WEIGHT_MODE = {"score": WEIGHT_SCORE, "ones": WEIGHT_ONES, "soft_flip": WEIGHT_SOFT_FLIP}


class BH4(nn.Module):
    """Block-diagonal x Hadamard projection (reference lookup.py:10-47).  Holds the parameters and
    the description of the projection; the arithmetic runs fused inside the hash kernel."""

    num_stages = 4

    def __init__(self, in_dim, out_dim, block_size, decay_coeff=0.7):
        super().__init__()
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.block_size = block_size
        self.decay_coeff = decay_coeff
        self.padded_in_dim = int(2 ** math.ceil(math.log2(in_dim)))
        self.num_repeat = max(1, int(math.ceil(self.out_dim / self.padded_in_dim)))
        self.num_block = self.padded_in_dim // self.block_size
        coeff = math.sqrt(self.block_size * self.padded_in_dim)
        self.weight = nn.Parameter(
            torch.randn(self.num_repeat, self.num_stages, self.num_block, self.block_size, self.block_size) / coeff)
        self.bias = nn.Parameter(torch.zeros(self.out_dim))
        self.had_scale = 1.0
        self.register_load_state_dict_post_hook(lambda module, _keys: module.refresh_kernel_weight())

    def extra_repr(self):
        return (f"in_dim={self.in_dim}, out_dim={self.out_dim}, block_size={self.block_size}, "
                f"decay_coeff={self.decay_coeff}")

    @property
    def mix(self):
        return self.decay_coeff, 1 - self.decay_coeff

    def kernel_weight(self):
        """(weight tensor, transpose_w flag) to hand to the hash kernel.  The 64 x 64 fast path streams the
        blocks in [i][o] order, so for that shape a transposed copy of the parameter is kept.  It is refreshed when
        the parameter's storage or version counter changes (optimizer step, .to()), after load_state_dict, and on
        every call while the module is in training mode.  An in-place write through `weight.data` in eval mode
        does not move the version counter: call refresh_kernel_weight() after one."""
        w = self.weight.detach()
        if self.block_size != 64 or self.padded_in_dim % 256 != 0:
            return w.contiguous(), False
        key = (w.data_ptr(), w._version, w.device)
        if self.training or getattr(self, "_wt_key", None) != key:
            self._wt = w.transpose(-1, -2).contiguous()
            self._wt_key = key
        return self._wt, True

    def refresh_kernel_weight(self):
        """Drop the cached transposed weights; the next forward rebuilds them from the parameter."""
        self._wt_key = None

    def forward(self, xs):
        """The projection alone, z [..., out_dim] (reference BH4.forward)."""
        shape = xs.shape[:-1]
        x = xs.reshape(-1, xs.shape[-1])
        wk, tw = self.kernel_weight()
        desc = ops.make_hash_desc(self.in_dim, wk, self.bias.detach().contiguous(), self.out_dim, 1, transpose_w=tw,
                                  had_scale=self.had_scale, mix_a=self.mix[0], mix_b=self.mix[1],
                                  weight_mode=WEIGHT_ONES)
        _, _, z = ops.hash_fwd(x, desc, want_z=True, want_codes=False)
        return z.reshape(*shape, self.out_dim)


class SignHadamard(BH4):
    """v = H diag(s2) H diag(s1) x per rotation with fixed random +-1 diagonals and the Hadamard
    matrix normalised by 1/sqrt(D): the BS = 1, two-stage, no-mix case of the same kernel."""

    num_stages = 2

    def __init__(self, in_dim, out_dim, seed=0):
        super().__init__(in_dim, out_dim, block_size=1, decay_coeff=1.0)
        g = torch.Generator().manual_seed(seed)
        signs = (2 * torch.randint(0, 2, self.weight.shape, generator=g) - 1).float()
        self.weight = nn.Parameter(signs, requires_grad=False)
        self.had_scale = 1.0 / math.sqrt(self.padded_in_dim)


class Hashing(nn.Module):
    """Projection to T*k coordinates, then codes and weights (reference lookup.py:49-77)."""

    def __init__(self, config):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_table = config.ffn_num_table
        self.table_size = config.ffn_table_size
        self.code_length = int(math.log2(self.table_size))
        self.total_dim = self.num_table * self.code_length
        self.bit_order = _BIT_ORDER[getattr(config, "lookup_bit_order", "msb")]
        self.weight_mode = _WEIGHT_MODE[getattr(config, "lookup_weight_mode", "score")]
        self.tau = float(getattr(config, "lookup_tau", 0.5))
        if config.projection_type == "bh4":
            self.projection = BH4(self.hidden_size, self.total_dim, block_size=config.block_size)
        elif config.projection_type == "sign_hadamard":
            self.projection = SignHadamard(self.hidden_size, self.total_dim, seed=getattr(config, "lookup_seed", 0))
        elif config.projection_type == "dense":
            self.projection = nn.Linear(self.hidden_size, self.total_dim)
        else:
            raise NotImplementedError

    @property
    def candidates(self):
        return self.code_length + 1 if self.weight_mode == WEIGHT_SOFT_FLIP else 1

    def fuses_layer_norm(self):
        """True when the projection runs in this package's hash kernel, which can apply the LayerNorm in its load."""
        return not isinstance(self.projection, nn.Linear)

    @torch.no_grad()
    def project(self, x, layer_norm=None):
        """The projected coordinates z [N, T*k] alone, through the same kernels as forward (diagnostics: which
        coordinates sit near zero).  layer_norm as in forward."""
        p = self.projection
        if isinstance(p, nn.Linear):
            return p(x).float()
        wk, tw = p.kernel_weight()
        desc = ops.make_hash_desc(self.hidden_size, wk, p.bias.detach().contiguous(), self.num_table,
                                  self.code_length, transpose_w=tw, had_scale=p.had_scale, mix_a=p.mix[0],
                                  mix_b=p.mix[1], bit_order=self.bit_order, weight_mode=self.weight_mode, tau=self.tau)
        return ops.hash_fwd(x, desc, want_z=True, want_codes=False, layer_norm=layer_norm)[2]

    def forward(self, x, t_begin=0, t_count=None, layer_norm=None):
        """x [N, hidden] -> (row indices int32 [N, T*m] with table offsets added, weights fp32 [N, T*m]).
        layer_norm = (weight, bias, eps): x is the un-normalised input and the kernel applies the LayerNorm
        (inference with a bh4 / sign_hadamard projection only)."""
        t_count = self.num_table - t_begin if t_count is None else t_count
        p = self.projection
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or any(q.requires_grad for q in p.parameters()))
        assert layer_norm is None or (self.fuses_layer_norm() and not needs_grad)
        if isinstance(p, nn.Linear):
            z = p(x).float().reshape(x.shape[0], self.num_table, self.code_length)
            z = z[:, t_begin:t_begin + t_count].contiguous()
            if needs_grad:
                return ops.CodeScore.apply(z, self.bit_order, self.weight_mode, self.tau)
            return ops.compute_code_score(z, bit_order=self.bit_order, weight_mode=self.weight_mode, tau=self.tau,
                                          add_offsets=True)
        wk, tw = p.kernel_weight()
        if needs_grad:
            # training: projection and weights as two differentiable steps (z makes one round trip through HBM);
            # inference below runs the single fused kernel
            assert t_begin == 0 and t_count == self.num_table, "training runs on the whole table range"
            z = ops.Projection.apply(x, p.weight, p.bias, p.had_scale, p.mix[0], p.mix[1], wk, tw)
            return ops.CodeScore.apply(z.reshape(x.shape[0], self.num_table, self.code_length), self.bit_order,
                                       self.weight_mode, self.tau)
        desc = ops.make_hash_desc(self.hidden_size, wk, p.bias.detach().contiguous(), self.num_table,
                                  self.code_length, transpose_w=tw, had_scale=p.had_scale, mix_a=p.mix[0],
                                  mix_b=p.mix[1], bit_order=self.bit_order, weight_mode=self.weight_mode, tau=self.tau)
        idx, w, _ = ops.hash_fwd(x, desc, t_begin=t_begin, t_count=t_count, layer_norm=layer_norm)
        return idx, w


class LookupFFN(nn.Module):
    def __init__(self, config, output_size):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.output_size = output_size
        self.LayerNorm = nn.LayerNorm(self.hidden_size, eps=config.layer_norm_eps)
        self.num_table = config.ffn_num_table
        self.table_size = config.ffn_table_size
        assert (2 ** int(math.log2(self.table_size))) == self.table_size
        self.hash = Hashing(config)
        table_dtype = getattr(config, "lookup_table_dtype", torch.float32)
        self.tables = nn.Parameter(
            (0.02 * torch.randn(self.num_table, self.table_size, self.output_size)).to(table_dtype))
        self.bias = nn.Parameter(0.001 * torch.randn(self.output_size))

    def extra_repr(self):
        return (f"hidden_size={self.hidden_size}, num_table={self.num_table}, table_size={self.table_size}, "
                f"output_size={self.output_size}")

    def _inference(self):
        """No gradient can be asked for: the fused two-kernel path applies."""
        return not (torch.is_grad_enabled() and any(p.requires_grad for p in self.parameters()))

    def _forward(self, hidden_states, residual=None):
        if not hidden_states.is_cuda:
            raise RuntimeError("lookupffn_b200.LookupFFN runs on CUDA tensors only (no CPU fallback)")
        if self._inference() and not hidden_states.requires_grad and self.hash.fuses_layer_norm() \
                and hidden_states.dtype in (torch.float32, torch.bfloat16):
            # two kernels: LayerNorm inside the hash kernel's load; bias and residual inside the gather's epilogue
            ln = self.LayerNorm
            code, score = self.hash(hidden_states, layer_norm=(ln.weight, ln.bias, ln.eps))
            T, rows, d = self.tables.shape
            return ops.weighted_vector_gather_add(code, self.tables.reshape(T * rows, d), score, bias=self.bias,
                                                  residual=residual)
        hidden_states = ops.layer_norm(hidden_states, self.LayerNorm)
        code, score = self.hash(hidden_states)
        outputs = self.gather(code, score, self.tables)
        return outputs if residual is None else outputs + residual.reshape(outputs.shape).to(outputs.dtype)

    def forward(self, hidden_states, residual=None):
        """residual (optional, same leading dims, output_size last): added to the result, as the encoder layer
        does (layer.py:75-78: dropout(FFN(x)) + x); in inference the add rides in the gather kernel's epilogue.
        Callers that apply dropout between the two keep doing the add themselves."""
        shape = hidden_states.shape[:-1]
        dim = hidden_states.shape[-1]
        hidden_states = hidden_states.reshape(int(np.prod(shape)), dim)
        outputs = self._forward(hidden_states, residual)
        return outputs.reshape(*shape, self.output_size)

    def gather(self, indexes, weights, tables):
        """indexes already hold code + t * table_size (the kernel adds the offsets of reference
        lookup.py:126).  The bias add of lookup.py:108 is fused into the kernel; in training its gradient is the
        column sum of the output gradient (lffn_bias_grad)."""
        num_table, table_size, vector_dim = tables.shape
        flat = tables.reshape(num_table * table_size, vector_dim)
        m = self.hash.candidates
        if torch.is_grad_enabled() and (flat.requires_grad or weights.requires_grad):
            return ops.gather(indexes, weights, flat, training=self.training, structure=(num_table, m, table_size),
                              bias=self.bias)
        return ops.weighted_vector_gather_add(indexes, flat, weights, bias=self.bias)
