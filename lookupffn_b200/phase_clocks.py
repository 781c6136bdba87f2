"""Where hash_block64_kernel (the 64 x 64 block-diagonal hashing kernel) spends its cycles.

    python -m lookupffn_b200.phase_clocks [--shape c2|ref|c3]

Builds a variant of the library with -DLFFN_HB_PHASE_CLOCKS (thread 0 of every CTA adds the clock64 cycles
between phase marks to per-phase counters), runs one launch of the chosen shape and prints each phase's share.
The marks cost a little time themselves: use the shares, take absolute times from the normal build.
The multiply-add and chunk-wait rows are what warp 0 sees; the other warps run the same loop.
"""
import argparse
import ctypes
import os
import sys  # noqa: F401

HERE = os.path.dirname(os.path.abspath(__file__))
VARIANT = os.path.join(HERE, "liblookupffn_phase_clocks.so")
PHASES = ["tile load / carry", "multiply-add loop", "Hadamard passes", "mix pass (when not folded)",
          "codes and weights", "wait for a weight chunk", "write-back + barrier"]
SHAPES = {  # name: (tokens, d_in, tables, code bits, x dtype)
    "c2": (16384, 512, 256, 8, "float32"),
    "ref": (32768, 512, 128, 8, "float32"),
    "c3": (65536, 768, 512, 8, "bfloat16"),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", choices=sorted(SHAPES), default="c2")
    args = ap.parse_args()

    from lookupffn_b200 import _lib, build
    build.build(defines=("LFFN_HB_PHASE_CLOCKS",), output=VARIANT)
    if _lib._lib is not None:
        sys.exit("the library is already loaded in this process")
    _lib.LIB_PATH = VARIANT  # the loader opens this path on first use

    import numpy as np
    import torch
    from lookupffn_b200 import ops

    lib = ctypes.CDLL(VARIANT)  # same handle as the loader's: the counters live in this image
    dev = torch.device("cuda:0")
    N, d_in, T, k, dt = SHAPES[args.shape]
    BS, S = 64, 4
    D = ops.padded_dim(d_in)
    R = max(1, -(-T * k // D))
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(N, d_in, generator=g, device=dev).to(getattr(torch, dt))
    w = (torch.randn(R, S, D // BS, BS, BS, generator=g, device=dev) / np.sqrt(BS * D)).contiguous()
    desc = ops.make_hash_desc(d_in, w, None, T, k, transpose_w=True)
    for _ in range(3):
        ops.hash_fwd(x, desc)
    torch.cuda.synchronize()
    if lib.lffn_debug_hash_block_phases(None, 1) != 0:
        sys.exit("could not reset the phase counters")
    ops.hash_fwd(x, desc)
    torch.cuda.synchronize()
    out = (ctypes.c_ulonglong * 8)()
    if lib.lffn_debug_hash_block_phases(out, 1) != 0:
        sys.exit("could not read the phase counters")
    total = sum(out[:len(PHASES)])
    if total == 0:
        sys.exit("no cycles recorded: this shape did not run hash_block64_kernel")
    n_cta = min(torch.cuda.get_device_properties(dev).multi_processor_count, (N + 31) // 32 * R)
    print(f"shape {args.shape}: N={N} D={D} T={T} k={k} rotations={R}; {total // n_cta} cycles per CTA")
    for name, v in zip(PHASES, out):
        print(f"  {name:32s} {100.0 * v / total:5.1f} %")


if __name__ == "__main__":
    main()
