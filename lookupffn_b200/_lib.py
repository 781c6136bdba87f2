"""ctypes binding of liblookupffn.so (include/lookupffn.h).

The library is the only compute path of this package: if it cannot be loaded the import of
any op fails with an error that says how to build it.  There is no CPU or PyTorch fallback.
"""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# LFFN_LIBRARY_PATH selects another build of the same library (e.g. a tuning variant)
LIB_PATH = os.environ.get("LFFN_LIBRARY_PATH") or os.path.join(_HERE, "liblookupffn.so")

F32, BF16 = 0, 1
MSB_FIRST, LSB_FIRST = 0, 1
WEIGHT_SCORE, WEIGHT_ONES, WEIGHT_SOFT_FLIP = 0, 1, 2
STATUS_INDEX_RANGE, STATUS_STRUCTURE, STATUS_TIMEOUT = 1, 2, 4
TRACE_NVTX, TRACE_STAGE_TIMES = 1, 2
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024

ERR_NAMES = {-1: "INVALID_ARG", -2: "UNSUPPORTED", -3: "CUDA", -4: "INDEX_RANGE", -5: "SCRATCH"}


class LookupFFNError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"liblookupffn: {ERR_NAMES.get(code, code)}: {message}")
        self.code = code


class HashDesc(C.Structure):
    """struct lffn_hash_desc"""
    _fields_ = [
        ("d_in", C.c_int32), ("D", C.c_int32), ("BS", C.c_int32), ("S", C.c_int32), ("R", C.c_int32),
        ("transpose_w", C.c_int32), ("had_scale", C.c_float), ("mix_a", C.c_float), ("mix_b", C.c_float),
        ("T", C.c_int32), ("k", C.c_int32), ("bit_order", C.c_int32), ("weight_mode", C.c_int32),
        ("tau", C.c_float), ("proj_w", C.c_void_p), ("proj_bias", C.c_void_p),
    ]


_SIGNATURES = {
    "lffn_version": (C.c_int, []),
    "lffn_last_error_string": (C.c_char_p, []),
    "lffn_trace_configure": (C.c_int, [C.c_uint32]),
    "lffn_trace_last_layer_times": (C.c_int, [C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "lffn_device_status": (C.c_int, [C.POINTER(C.c_uint32), C.c_void_p]),
    "lffn_selftest_bounded_wait": (C.c_int, [C.c_int32, C.c_void_p]),
    "lffn_probe_read": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int32, C.c_int32, C.c_void_p, C.POINTER(C.c_size_t),
                                  C.c_void_p]),
    "lffn_fwht": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_float, C.c_void_p]),
    "lffn_hash_fwd": (C.c_int, [C.POINTER(HashDesc), C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int32,
                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lffn_hash_fwd_ln": (C.c_int, [C.POINTER(HashDesc), C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_int32,
                                   C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lffn_code_weights": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float,
                                    C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lffn_code_weights_bwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_float,
                                        C.c_void_p, C.c_void_p]),
    "lffn_proj_bwd_ws_bytes": (C.c_size_t, [C.POINTER(HashDesc), C.c_int64]),
    "lffn_proj_acts_bytes": (C.c_size_t, [C.POINTER(HashDesc), C.c_int64]),
    "lffn_proj_fwd_train": (C.c_int, [C.POINTER(HashDesc), C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p,
                                      C.c_size_t, C.c_void_p]),
    "lffn_proj_bwd": (C.c_int, [C.POINTER(HashDesc), C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_void_p,
                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "lffn_bias_grad_ws_bytes": (C.c_size_t, [C.c_int32]),
    "lffn_bias_grad": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "lffn_layernorm_bwd_ws_bytes": (C.c_size_t, [C.c_int32]),
    "lffn_layernorm_bwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "lffn_gather_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int64,
                                  C.c_int32, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]),
    "lffn_gather_fwd_residual": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32,
                                           C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p,
                                           C.c_void_p]),
    "lffn_gather_fwd_scatter": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32,
                                          C.c_int64, C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.c_int64, C.c_int32,
                                          C.c_void_p]),
    "lffn_gather_bwd_weights": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int64,
                                          C.c_int32, C.c_int64, C.c_int32, C.c_void_p]),
    "lffn_gather_bwd_tables": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                         C.c_int64, C.c_int32, C.c_void_p]),
    "lffn_gather_bwd_tables_sorted_scratch_bytes": (C.c_size_t, [C.c_int64, C.c_int32, C.c_int32, C.c_int32]),
    "lffn_gather_bwd_tables_sorted": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                                C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p]),
    "lffn_gather_bwd_tables_sorted_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                                       C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "lffn_layer_fwd": (C.c_int, [C.POINTER(HashDesc), C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int32,
                                 C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                 C.c_void_p, C.c_void_p]),
    "lffn_layer_fwd_ln_residual": (C.c_int, [C.POINTER(HashDesc), C.c_void_p, C.c_void_p, C.c_float, C.c_void_p,
                                             C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                                             C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                             C.c_void_p, C.c_void_p]),
    "lffn_layer_fwd_host_ws_bytes": (C.c_size_t, [C.POINTER(HashDesc), C.c_int32, C.c_int32, C.c_int32, C.c_int64]),
    "lffn_layer_fwd_host": (C.c_int, [C.POINTER(HashDesc), C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_int32,
                                      C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_size_t,
                                      C.c_int64, C.c_void_p]),
}

_lib = None


def exported_symbols():
    return sorted(_SIGNATURES)


def lib():
    """Load the library once.  Raises (never falls back) when it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} not found: build it with `python -m lookupffn_b200.build` "
                "(nvcc, sm_100a).  lookupffn_b200 has no CPU or PyTorch fallback.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = the library is older than this binding: rebuild it
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc):
    if rc != 0:
        raise LookupFFNError(rc, lib().lffn_last_error_string().decode())


def dtype_code(t):
    if t == torch.float32:
        return F32
    if t == torch.bfloat16:
        return BF16
    raise TypeError(f"lookupffn_b200 supports float32 and bfloat16 storage, got {t}")


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("lookupffn_b200 runs on CUDA tensors only (no CPU fallback); got a CPU tensor")


def device_status(device=None):
    """Read and clear the device status word (synchronises the current stream)."""
    out = C.c_uint32(0)
    with torch.cuda.device(device):
        check(lib().lffn_device_status(C.byref(out), stream_ptr(device)))
    return out.value
