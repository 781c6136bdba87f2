"""Compile liblookupffn.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m lookupffn_b200.build [--force] [--verbose]
    python -m lookupffn_b200.build --define LFFN_HB_PHASE_CLOCKS --output /some/path/libvariant.so

The second form compiles a variant with extra -D macros into a library of its own (own object directory; the
default library is left alone); load it with LFFN_LIBRARY_PATH.
"""
import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "liblookupffn.so")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3", "--expt-relaxed-constexpr", "-shared",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def up_to_date(lib=LIB):
    if not os.path.exists(lib):
        return False
    t = os.path.getmtime(lib)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return all(os.path.getmtime(p) <= t for p in deps)


def build(force=False, verbose=False, ptxas_info=False, defines=(), output=None):
    """One `nvcc -c` per source file (in parallel), then one link step."""
    variant = bool(defines) or output is not None
    if variant and output is None:
        raise ValueError("a build with extra macros needs its own output path")
    lib = os.path.abspath(output) if variant else LIB
    if not force and up_to_date(lib):
        return lib
    from concurrent.futures import ThreadPoolExecutor

    nvcc = os.environ.get("NVCC", "nvcc")
    objdir = os.path.join(HERE, "_obj", "variant_" + os.path.basename(lib)) if variant else os.path.join(HERE, "_obj")
    os.makedirs(objdir, exist_ok=True)
    cflags = [f for f in NVCC_FLAGS if f != "-shared"] + (["-Xptxas", "-v"] if ptxas_info else [])
    cflags += ["-D" + d for d in defines]

    def compile_one(src):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc] + cflags + ["-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a"] + objs + ["-o", lib, "-ldl"]
    if verbose:
        print(" ".join(link), flush=True)
    subprocess.check_call(link)
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true")
    ap.add_argument("--define", action="append", default=[], metavar="NAME[=VALUE]")
    ap.add_argument("--output", default=None, help="library path of a variant build")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, ptxas_info=a.ptxas_info, defines=tuple(a.define), output=a.output))
    sys.exit(0)
