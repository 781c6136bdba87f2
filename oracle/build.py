"""Build the CPU oracle (and, when the reference checkout is present, the
reference's own CPU extensions) with plain gcc/g++ commands.

TEST INFRASTRUCTURE: the outputs are loaded only by tests, the smoke test and
the benchmark's CPU-baseline legs.

  python oracle/build.py            # oracle + (if the reference tree exists) oracle/_ref
  python oracle/build.py --no-ref   # oracle only

Outputs
  oracle/liblffn_oracle.so   C restatement (oracle/lffn_oracle.c)
  oracle/_ref/ccs_cpu*.so          reference compute_code_score extension, unmodified source
  oracle/_ref/gather_add_cpu*.so   reference CPU gather extension, unmodified source
  oracle/_ref/sbdht_cpu*.so        reference CPU BH4 extension (block-diagonal x Hadamard), unmodified source, compiled
                                   against the stand-in oracle/standin/libxsmm.h (the real libxsmm is not available)
  oracle/_ref/gather_add*.so       reference CUDA gather extension (fp32 / fp16 kernels), unmodified source, sm_100a
  oracle/_ref/fast_hadamard_transform_kernel*.so   reference CUDA Hadamard extension, unmodified source, sm_100a
The reference sources are compiled where they lie; nothing is copied.  The two CUDA modules are the GPU comparator:
tests check the library's kernels against them on the GPU, the benchmark times them beside its own.
"""
import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liblffn_oracle.so")
REF_OUT = os.path.join(HERE, "_ref")
# where the reference checkout lives: LFFN_REFERENCE_ROOT, else a directory named "reference" beside this repository
REF_ROOT = os.environ.get("LFFN_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
REF_LOOKUP = os.path.join(REF_ROOT, "src", "roberta", "models", "prenorm_lookup")

# AVX2+FMA rather than -march=native: the library is built on one machine and
# run on another.  -ffp-contract=off keeps every rounding where the source puts it.
CFLAGS = ["-O3", "-mavx2", "-mfma", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC", "-shared"]

REF_EXTENSIONS = {
    # module name -> source relative to prenorm_lookup/
    "ccs_cpu": os.path.join("compute_code_score", "torch_extension.cc"),
    "gather_add_cpu": os.path.join("gather", "cpu", "torch_extension.cpp"),
    # the CPU BH4 extension includes <libxsmm.h> (third-party, absent): compiled against oracle/standin/libxsmm.h
    "sbdht_cpu": os.path.join("bh4", "cpu", "torch_extension.cpp"),
}
REF_EXTRA_INCLUDES = {"sbdht_cpu": [os.path.join(HERE, "standin")]}


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False, verbose=True):
    src = os.path.join(HERE, "lffn_oracle.c")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    cmd = ["gcc", "-std=gnu11"] + CFLAGS + [src, "-o", ORACLE_SO, "-lm"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return ORACLE_SO


def ref_module_path(name):
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(REF_OUT, name + suffix)


def load_ref_module(name):
    """Import one of the modules built into oracle/_ref (None when it has not been built)."""
    import importlib.util

    path = ref_module_path(name)
    if not os.path.exists(path):
        return None
    import torch  # noqa: F401  (the extension modules link against libtorch)

    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def build_ref(force=False, verbose=True):
    """Compile the reference's two CPU extensions (pybind11 + ATen modules) with one
    g++ command each.  Returns the list built, or [] when the reference tree is absent."""
    if not os.path.isdir(REF_LOOKUP):
        return []
    import torch
    from torch.utils import cpp_extension

    os.makedirs(REF_OUT, exist_ok=True)
    inc = []
    for p in cpp_extension.include_paths():
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    built = []
    for name, rel in REF_EXTENSIONS.items():
        src = os.path.join(REF_LOOKUP, rel)
        out = ref_module_path(name)
        if not force and _newer(out, [src]):
            built.append(out)
            continue
        cmd = (["g++", "-std=c++17", "-O3", "-mavx2", "-mfma", "-fopenmp", "-fPIC", "-shared", "-w",
                f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
               + inc + [f"-I{d}" for d in REF_EXTRA_INCLUDES.get(name, [])] + [src, "-o", out, f"-L{libdir}", f"-Wl,-rpath,{libdir}",
                        "-ltorch_python", "-ltorch", "-ltorch_cpu", "-lc10", "-lgomp"])
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        built.append(out)
    return built


REF_CUDA_EXTENSIONS = {
    # module name -> (directory relative to prenorm_lookup/, sources)
    "gather_add": (os.path.join("gather", "cuda", "extension"),
                   ["gather_kernel_fp16.cu", "gather_fp16.cu", "gather_kernel_fp32.cu", "gather_fp32.cu",
                    "torch_extension.cpp"]),
    "fast_hadamard_transform_kernel": (os.path.join("bh4", "fast_hadamard_transform", "extension"),
                                       ["cuda_kernel.cu", "cuda_launch.cu", "torch_extension.cpp"]),
}


def build_ref_cuda(force=False, verbose=True):
    """Compile the reference's CUDA extensions for sm_100a: one nvcc / g++ command per source file (the same files
    its own torch.utils.cpp_extension.load call lists), one link step per module.  Objects go to oracle/_ref/obj."""
    if not os.path.isdir(REF_LOOKUP):
        return []
    from concurrent.futures import ThreadPoolExecutor

    import torch
    from torch.utils import cpp_extension

    objdir = os.path.join(REF_OUT, "obj")
    os.makedirs(objdir, exist_ok=True)
    inc = []
    for p in cpp_extension.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    jobs, plan = [], {}
    for name, (rel, files) in REF_CUDA_EXTENSIONS.items():
        srcs = [os.path.join(REF_LOOKUP, rel, f) for f in files]
        out = ref_module_path(name)
        if not force and _newer(out, srcs):
            plan[name] = (out, None)
            continue
        objs = []
        for src in srcs:
            obj = os.path.join(objdir, name + "_" + os.path.basename(src) + ".o")
            defs = [f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H", abi]
            if src.endswith(".cu"):
                cmd = (["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-w",
                        "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"] + defs + inc + ["-c", src, "-o", obj])
            else:
                cmd = (["g++", "-std=c++17", "-O3", "-fPIC", "-w"] + defs + inc
                       + ["-isystem", os.path.join(cuda_home, "include"), "-c", src, "-o", obj])
            jobs.append(cmd)
            objs.append(obj)
        plan[name] = (out, objs)

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(run, jobs))
    built = []
    for name, (out, objs) in plan.items():
        if objs is not None:
            run(["g++", "-shared"] + objs + ["-o", out, f"-L{libdir}", f"-Wl,-rpath,{libdir}",
                                             f"-L{os.path.join(cuda_home, 'lib64')}", "-ltorch_python", "-ltorch",
                                             "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-lcudart"])
        built.append(out)
    return built


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--no-ref", action="store_true")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    build_oracle(force=a.force)
    if not a.no_ref:
        got = build_ref(force=a.force)
        print("reference CPU extensions:", got if got else "reference tree not present, skipped")
        got = build_ref_cuda(force=a.force)
        print("reference CUDA extensions:", got if got else "reference tree not present, skipped")


if __name__ == "__main__":
    sys.exit(main())
