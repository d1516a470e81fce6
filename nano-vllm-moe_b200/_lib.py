"""ctypes binding of libfp8lin.so (C ABI declared in include/fp8lin.h).

The library is built in-tree by ``build.py`` and loaded from this directory.
Loading never falls back to anything else: if the shared object is missing the
first call raises ``RuntimeError`` telling the user to build it.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p, POINTER
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libfp8lin.so"

W8A16 = 0
W8A8_STATIC = 1
WS_HEADER_BYTES = 65536

OK, ERR_NULL, ERR_SHAPE, ERR_ALIGN, ERR_WORKSPACE, ERR_ARCH, ERR_LAUNCH, ERR_DEVICE, ERR_ARG = range(9)

# every symbol include/fp8lin.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "fp8lin_version": (c_int, []),
    "fp8lin_last_error": (c_char_p, []),
    "fp8lin_launch_count": (ctypes.c_ulonglong, []),
    "fp8lin_packed_bytes": (c_size_t, [c_int64, c_int64]),
    "fp8lin_prepack_weight": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "fp8lin_pack_weight_nk": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "fp8lin_workspace_bytes": (c_size_t, [c_int, c_int64, c_int64, c_int64]),
    "fp8lin_w8a16": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                             c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "fp8lin_w8a8": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                            c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "fp8lin_w8a8_preq": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                 c_void_p, c_size_t, c_void_p]),
    "fp8lin_rmsnorm_quant": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, ctypes.c_float, c_void_p, c_void_p, c_void_p,
                                     c_int64, c_int64, c_int64, c_void_p]),
    "fp8lin_w8a8_scatter": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, POINTER(c_void_p),
                                    c_int64, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "fp8lin_w8a8_reduce_scatter": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, POINTER(c_void_p),
                                           c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "fp8lin_sum_slots_gather": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, POINTER(c_void_p), c_int64, c_int64, c_int64,
                                        c_int64, c_void_p]),
    "fp8lin_quantize_weight": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "fp8lin_abs_max": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "fp8lin_mlp_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64]),
    "fp8lin_mlp_w8a8": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "fp8lin_mlp_w8a8_preq": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "fp8lin_sum_slots": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "fp8lin_linear_static_scratch": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "fp8lin_quantize_activation": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "fp8lin_moe_route": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "fp8lin_debug_wait_timeout": (c_int, [c_void_p, c_int64, c_void_p]),
    "fp8lin_moe_align": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fp8lin_moe_workspace_bytes": (c_size_t, [c_int64, c_int, c_int64, c_int64]),
    "fp8lin_moe_experts_w8a8": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p,
                                        c_int64, c_void_p, c_size_t, c_void_p]),
    "fp8lin_moe_combine": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_void_p]),
    "fp8lin_variant_name": (c_char_p, [c_int, c_int64, c_int64, c_int64]),
    "fp8lin_set_tuning": (c_int, [c_char_p, c_int]),
    "fp8lin_read_status": (c_int, [c_void_p, c_void_p, POINTER(c_int)]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python {LIB_PATH.parent / 'build.py'}` "
            "(needs nvcc; there is no CPU fallback)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return (load().fp8lin_last_error() or b"").decode()


def raise_for(code: int, what: str) -> None:
    """Map a status code to the exception type the reference raises for the
    same condition (ValueError for bad arguments, RuntimeError for device
    problems; nanovllm/quantization/cuda_ext.py:78-79, csrc TORCH_CHECKs)."""
    if code == OK:
        return
    msg = f"{what}: {last_error()} (fp8lin status {code})"
    if code in (ERR_NULL, ERR_SHAPE, ERR_ALIGN, ERR_ARG):
        raise ValueError(msg)
    raise RuntimeError(msg)
