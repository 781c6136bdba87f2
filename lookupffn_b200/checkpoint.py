"""Checkpoint interchange with the reference.

A reference training run stores a PyTorch-Lightning checkpoint whose "state_dict" holds the MLM model
under the prefix "model." (roberta_to_hf_checkpoint.py:102-106), i.e. keys "model.roberta.<encoder key>"
and "model.lm_head.*".  The modules of this package use the reference's parameter names, so loading is a
matter of stripping prefixes; the helpers below also convert tables to bf16 storage and re-order table
rows between the two code bit orders.
"""
import re

import torch


def lightning_state_dict(ckpt):
    """`ckpt`: a path to a .ckpt file, the loaded checkpoint dict, or already a state_dict."""
    if isinstance(ckpt, (str, bytes)) or hasattr(ckpt, "__fspath__"):
        ckpt = torch.load(ckpt, map_location="cpu", weights_only=True)
    return ckpt["state_dict"] if "state_dict" in ckpt else ckpt


def encoder_state_dict(ckpt, prefix="model.roberta."):
    """State dict for lookupffn_b200.encoder.Lookup from a reference checkpoint (heads and other
    sub-modules outside the encoder are dropped)."""
    sd = lightning_state_dict(ckpt)
    out = {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}
    if not out:
        raise KeyError(f"no key starts with {prefix!r}; first keys: {list(sd)[:3]}")
    return out


def layer_state_dict(encoder_sd, layer):
    """State dict of one LookupFFN layer (keys LayerNorm.*, hash.projection.*, tables, bias)."""
    pre = f"encoder.layer.{layer}.FFN."
    out = {k[len(pre):]: v for k, v in encoder_sd.items() if k.startswith(pre)}
    if not out:
        raise KeyError(f"no LookupFFN parameters under {pre!r}")
    return out


def tables_to(sd, dtype=torch.bfloat16):
    """Copy of a state dict with every `tables` tensor converted (fp32 -> bf16 halves table memory; the
    kernels accumulate in fp32 either way)."""
    return {k: (v.to(dtype) if re.search(r"(^|\.)tables$", k) else v) for k, v in sd.items()}


def bit_reverse_permutation(k):
    """perm[c] = c with its k bits reversed."""
    c = torch.arange(1 << k)
    r = torch.zeros_like(c)
    for j in range(k):
        r |= ((c >> j) & 1) << (k - 1 - j)
    return r


def reorder_tables_bit_order(tables):
    """Tables [T, 2^k, d] trained under one code bit order (MSB-first, the reference, or LSB-first), re-ordered
    so that the other order addresses the same rows: new[t, reverse(c)] = old[t, c].  An involution."""
    T, rows, d = tables.shape
    k = rows.bit_length() - 1
    assert 1 << k == rows
    perm = bit_reverse_permutation(k).to(tables.device)
    out = torch.empty_like(tables)
    out[:, perm] = tables
    return out
