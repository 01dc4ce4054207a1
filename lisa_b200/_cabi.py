"""ctypes binding of ``liblisa_cuda.so`` (the C ABI declared in ``include/lisa_cuda.h``).

The library must have been built (``python -m lisa_b200.build``); loading fails loudly when
it is missing.  There is no CPU fallback anywhere in this package.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "liblisa_cuda.so")

# lisa_status
OK = 0
ERR_BAD_ARG = -1
ERR_UNSUPPORTED = -2
ERR_MISALIGNED = -3
ERR_OVERFLOW = -4
ERR_CUDA = -5
ERR_WORKSPACE = -6
ERR_LIMIT = -7

BF16, F16, F32 = 0, 1, 2
GGUF_Q2_K, GGUF_Q4_K, GGUF_Q5_K = 10, 12, 13

FLAG_NONE = 0
FLAG_FORCE_QMV = 1 << 0
FLAG_FORCE_QMV_SIMPLE = 1 << 1
FLAG_FORCE_QMM = 1 << 2
FLAG_PDL = 1 << 3
FLAG_FORCE_QMV_TC = 1 << 4
FLAG_FORCE_QMV_I8 = 1 << 5

_vp, _i64, _int, _sz, _u = C.c_void_p, C.c_int64, C.c_int, C.c_size_t, C.c_uint

# name -> (restype, argtypes); mirrors include/lisa_cuda.h declaration by declaration.
SIGNATURES = {
    "lisa_cuda_last_error_string": (C.c_char_p, []),
    "lisa_cuda_version": (_int, []),
    "lisa_cuda_launch_count": (C.c_uint64, []),
    "lisa_cuda_device_status": (_int, []),
    "lisa_cuda_clear_device_status": (_int, []),
    "lisa_cuda_quantized_matmul": (_int, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _i64, _int, _int, _int, _int, _vp]),
    "lisa_cuda_quantized_matmul_ex": (_int, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _i64, _int, _int, _int, _int, _vp, _u]),
    "lisa_cuda_quantized_matmul_serial_rows": (_int, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _i64, _int, _int, _int, _int, _vp]),
    "lisa_cuda_quantized_matmul_allgather": (_int, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _i64, _int, _int, _int, _int, _vp, _int, _i64, _i64, _u]),
    "lisa_cuda_quantized_matmul_siblings": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _vp, _u]),
    "lisa_cuda_quantized_matmul_siblings_allgather": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _vp, _int, _vp, _vp, _u]),
    "lisa_cuda_peer_barrier": (_int, [_vp, _int, _int, _vp, C.c_uint64]),
    "lisa_cuda_dequantize": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _int, _vp]),
    "lisa_cuda_dequantize_rows": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _int, _vp]),
    "lisa_cuda_quantize": (_int, [_vp, _vp, _i64, _i64, _int, _int, _int, _vp, _vp, _vp]),
    "lisa_cuda_gather_qmm_siblings": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _int, _int, _int,
                                             _vp, _vp, _sz]),
    "lisa_cuda_gather_qmm_workspace_bytes": (_sz, [_i64, _i64]),
    "lisa_cuda_gather_qmm": (_int, [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _int, _int, _int, _vp, _vp, _sz]),
    "lisa_cuda_gguf_packed_matvec": (_int, [_vp, _int, _vp, _i64, _i64, _vp, _i64, _vp]),
    "lisa_cuda_gguf_packed_matvec_allgather": (_int, [_vp, _int, _vp, _i64, _i64, _vp, _i64, _vp, _int, _i64, _i64]),
    "lisa_cuda_gguf_packed_matmul_workspace_bytes": (_sz, [_i64, _i64, _int]),
    "lisa_cuda_gguf_packed_matmul": (_int, [_vp, _int, _vp, _i64, _i64, _vp, _i64, _vp, _vp, _sz]),
    "lisa_cuda_gguf_expert_matvec": (_int, [_vp, _int, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _vp]),
    "lisa_cuda_moe_route": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp]),
    "lisa_cuda_moe_sort_workspace_bytes": (_sz, [_i64, _i64]),
    "lisa_cuda_moe_sort": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _sz]),
    "lisa_cuda_moe_sort_static": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "lisa_cuda_gather_rows": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "lisa_cuda_swiglu": (_int, [_vp, _vp, _vp, _i64, _int, _vp]),
    "lisa_cuda_ep_counts": (_int, [_vp, _vp, _i64, _i64, _int, _int, _vp]),
    "lisa_cuda_ep_dispatch": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp, _int]),
    "lisa_cuda_ep_return": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _int, _vp, _vp, _int]),
    "lisa_cuda_moe_combine": (_int, [_vp, _vp, _vp, _vp, _i64, _int, _i64, _int, _vp]),
    "lisa_cuda_quantized_matmul_swiglu": (_int, [_vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _i64, _int, _int, _int, _int, _vp, _vp,
                                                 C.c_uint]),
    "lisa_cuda_add_rmsnorm": (_int, [_vp, _vp, _vp, _vp, C.c_float, _i64, _i64, _int, _vp, _vp]),
    "lisa_cuda_quantized_matmul_addnorm": (_int, [_vp, _vp, _vp, _vp, C.c_float, _i64, _i64, _int, _vp, _vp, _vp, _vp, _int, _int,
                                                  _int, _int, _vp, _vp, _vp, C.c_uint]),
    "lisa_cuda_moe_gate_up_act": (_int, [_vp, _vp, _vp, _vp, _i64, _int, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp,
                                         _int, _int, _int, _vp]),
    "lisa_cuda_moe_down_combine": (_int, [_vp, _vp, _vp, _vp, _i64, _int, _i64, _i64, _i64, _vp, _vp, _vp, _int, _int, _int,
                                          _vp]),
}

_lib = None


class LisaError(RuntimeError):
    """An operator call was rejected or failed; mirrors the reference's ``Error::Msg``
    (crates/lisa-mlx/src/error.rs)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA library with `python -m lisa_b200.build` "
                "(there is no CPU fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error() -> str:
    s = lib().lisa_cuda_last_error_string()
    return s.decode() if s else ""


def check(rc: int) -> None:
    if rc != OK:
        raise LisaError(rc, last_error())
