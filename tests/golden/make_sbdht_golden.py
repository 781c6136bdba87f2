"""Generate tests/golden/sbdht_golden.npz: vectors of the reference's CPU BH4 path, made by the reference's own
code.

    python oracle/build.py                      # builds oracle/_ref/sbdht_cpu*.so from the reference's source
    python tests/golden/make_sbdht_golden.py

Runs src/roberta/models/prenorm_lookup/bh4/cpu/kernel.py of the reference checkout (LFFN_REFERENCE_ROOT, else a
directory named "reference" beside this repository): its module-level set-up call
(setup_xsmm_kernel_float_avx2(64, 64, 64, 512, 64, 512), kernel.py:32-37), its `bh4(x, w)` (kernel.py:45-52 ->
sbdht, torch_extension.cpp:123-196) and its `fwht_` (kernel.py:42-43 -> fwht_cpu_fp32_avx2_,
torch_extension.cpp:66-121).  torch.utils.cpp_extension.load is replaced by a loader that returns the prebuilt
oracle/_ref/sbdht_cpu module, so nothing is JIT-compiled.  The extension's source is the reference's, unmodified;
its one third-party include, <libxsmm.h>, resolves to oracle/standin/libxsmm.h (plain-loop C += A * B,
column-major): the GEMM's summation order is therefore the stand-in's, everything else is the reference's.

Arrays written
  sbdht_x [64, 512], sbdht_w [2, 4, 8, 64, 64] (randn / sqrt(64 * 512), the module's initialisation),
  sbdht_out [64, 1024] = bh4(x, w);  fwht_x [8, 512], fwht_out = fwht_(x) (in place, H / D).
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("LFFN_REFERENCE_ROOT") or os.path.join(os.path.dirname(REPO), "reference")
OUT = os.path.join(HERE, "sbdht_golden.npz")

sys.path.insert(0, REPO)
sys.path.insert(0, REF)
sys.dont_write_bytecode = True

import torch  # noqa: E402
import torch.utils.cpp_extension as cpp_ext  # noqa: E402

from oracle import build as obuild  # noqa: E402


def main():
    def load(name, sources=None, *a, **k):
        spec = importlib.util.spec_from_file_location(name, obuild.ref_module_path(name))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[name] = mod
        return mod

    cpp_ext.load = load
    torch.set_num_threads(4)
    import src.roberta.models.prenorm_lookup.bh4.cpu.kernel as ref_cpu  # runs the set-up call on import

    rng = np.random.RandomState(777)
    D, BS, R = 512, 64, 2
    x = rng.randn(64, D).astype(np.float32)
    w = (rng.randn(R, 4, D // BS, BS, BS) / np.sqrt(BS * D)).astype(np.float32)
    out = ref_cpu.bh4(torch.from_numpy(x.copy()), torch.from_numpy(w.copy()))
    fx = rng.randn(8, D).astype(np.float32)
    ft = torch.from_numpy(fx.copy())
    ref_cpu.fwht_(ft)
    np.savez_compressed(OUT, sbdht_x=x, sbdht_w=w, sbdht_out=out.numpy(), fwht_x=fx, fwht_out=ft.numpy())
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
