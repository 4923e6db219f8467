"""ctypes binding of ``libpx_b200.so`` (the C ABI declared in ``include/px_b200.h``).

There is one code path: if the library is missing, every operator of this package raises.
No CPU or torch fallback exists.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int32, c_int64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
# PX_B200_LIB names another build of the same library (e.g. one compiled with different options)
LIB_PATH = os.environ.get("PX_B200_LIB") or os.path.join(HERE, "libpx_b200.so")

PX_F32, PX_BF16, PX_F16 = 0, 1, 2

P, I32, I64, F = c_void_p, c_int32, c_int64, c_float

# name -> (restype, argtypes); mirrors include/px_b200.h declaration by declaration
SIGNATURES = {
    "px_version": (I32, []),
    "px_status_string": (c_char_p, [I32]),
    "px_ld": (I64, [I64]),
    "px_ld_mask": (I64, [I64]),
    "px_layer_norm_fwd": (I32, [P, P, P, P, P, P, I64, I64, F, I32, P]),
    "px_layer_norm_bwd": (I32, [P, P, P, P, P, P, P, P, P, I64, I64, I32, P]),
    "px_trimul_in_proj": (I32, [P, I32, P, P, P, P, P, P, P, P, P, I64, I64, I64, I32, F, P]),
    "px_trimul_contract": (I32, [P, P, P, I64, I64, I64, P]),
    "px_device_error_flags": (I32, [P]),
    "px_device_error_detail": (I32, [P, P]),
    "px_set_wait_limit_cycles": (I32, [I64]),
    "px_selftest_wait_timeout": (I32, [P, P]),
    "px_standardise_rows": (I32, [P, P, I64, F, P]),
    "px_add_update_rows": (I32, [P, P, I64, P]),
    "px_trimul_out": (I32, [P, P, P, P, I32, P, P, P, P, P, P, I64, I64, I64, I32, F, P]),
    "px_trimul_workspace_bytes": (I64, [I64]),
    "px_triangle_multiplication": (I32, [P, P, I32, P, P, P, P, P, P, P, P, P, P, P, P, I64, I64, I32, I32, F, P]),
    "px_triangle_multiplication_static": (I32, [P, P, I32, P, P, P, P, P, P, P, P, P, P, P, I64, I32, I32, F, P]),
    "px_static_max_n": (I64, []),
    "px_triatt_in_proj": (I32, [P, I32, P, P, P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I32, F, F, P]),
    "px_triatt_flash": (I32, [P, P, P, P, P, P, P, I64, I64, I64, P]),
    "px_triatt_flash_scratch_bytes": (I64, [I64, I64]),
    "px_triatt_out": (I32, [P, P, P, P, I32, P, P, P, P, I64, I64, I32, I32, F, P]),
    "px_triatt_workspace_bytes": (I64, [I64]),
    "px_triangle_attention": (I32, [P, P, I32, P, P, P, P, P, P, P, P, P, P, I64, I64, I32, I32, F, F, P]),
    "px_transition": (I32, [P, P, I32, P, P, P, P, P, I64, I32, F, P]),
    "px_pair_bias_proj": (I32, [P, I32, P, P, P, P, I64, I32, F, P]),
    "px_recycle_update": (I32, [P, P, P, I32, P, P, P, I64, F, P]),
    "px_scale_add_rowwise": (I32, [P, P, P, P, I64, I64, I64, I32, P]),
    "px_opm_outer": (I32, [P, P, P, I64, I64, I64, P]),
    "px_opm_out": (I32, [P, P, P, P, P, P, I32, I64, I64, I32, P]),
    "px_peer_alloc": (I32, [I64, P, P]),
    "px_peer_open": (I32, [P, P]),
    "px_peer_close": (I32, [P]),
    "px_peer_free": (I32, [P]),
    "px_peer_barrier": (I32, [P, I32, I32, ctypes.c_uint32, P]),
    "px_copy_2d": (I32, [P, I64, P, I64, I64, I64, P]),
    "px_copy_2d_dma": (I32, [P, I64, P, I64, I64, I64, P]),
    "px_copy_2d_batch": (I32, [P, P, I32, I64, I64, I64, I64, P]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m protenix_b200.build` "
                "(nvcc, sm_100a). This package has no fallback path."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().px_status_string(status).decode()
        raise RuntimeError(f"{what} failed: {msg} (status {status})")
