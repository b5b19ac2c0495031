"""ctypes binding of ``oracle/_ref/libtwm_ref.so``: the reference's own CUDA
kernels, compiled unchanged by ``build_ref.py``.  TEST INFRASTRUCTURE ONLY.
Arguments are device pointers (ints)."""
from __future__ import annotations

import ctypes as C
import os

_SO = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libtwm_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(_SO)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not available():
            raise FileNotFoundError(f"{_SO} missing: run `python oracle/build_ref.py` where the reference tree is")
        _lib = C.CDLL(_SO)
        v = C.c_void_p
        _lib.twmref_gemm_tw_marlin_m1.argtypes = [v, v, v, v, C.c_uint, C.c_uint, C.c_int, C.POINTER(C.c_int), v]
        _lib.twmref_quantize_q4_0.argtypes = [v, v, C.c_uint, v]
        _lib.twmref_dequantize_q4_0.argtypes = [v, v, C.c_uint, v]
        _lib.twmref_gemm_q4_0.argtypes = [v, v, v, C.c_uint, C.c_uint, C.c_uint, v]
        _lib.twmref_dequant_q4_to_f16.argtypes = [v, v, C.c_uint, C.c_uint, v]
        u = C.c_uint
        _lib.twmref_batched_marlin_gate_up.argtypes = [v, v, v, v, v, u, u, u, u, u, v]
        _lib.twmref_batched_marlin_down_axpy.argtypes = [v, v, v, v, v, v, u, u, u, u, u, v]
        _lib.twmref_batched_marlin_split_geglu.argtypes = [v, v, u, u, v]
    return _lib


def gemm_tw_marlin_m1(c_ptr, a_ptr, packed_ptr, scales_ptr, n, k, stream=0, force_splits=0) -> int:
    """Runs the reference launcher's logic (heuristic, memset, kernel); returns the splits used."""
    used = C.c_int(0)
    rc = lib().twmref_gemm_tw_marlin_m1(c_ptr, a_ptr, packed_ptr, scales_ptr, n, k, force_splits, C.byref(used), stream)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: {rc}")
    return used.value


def quantize_q4_0(out_ptr, in_ptr, n, stream=0):
    rc = lib().twmref_quantize_q4_0(out_ptr, in_ptr, n, stream)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: {rc}")


def dequantize_q4_0(out_ptr, in_ptr, n, stream=0):
    rc = lib().twmref_dequantize_q4_0(out_ptr, in_ptr, n, stream)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: {rc}")


def gemm_q4_0(c_ptr, a_ptr, bq_ptr, m, n, k, stream=0):
    rc = lib().twmref_gemm_q4_0(c_ptr, a_ptr, bq_ptr, m, n, k, stream)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: {rc}")


def dequant_q4_to_f16(out_ptr, bq_ptr, k, n, stream=0):
    rc = lib().twmref_dequant_q4_to_f16(out_ptr, bq_ptr, k, n, stream)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: {rc}")


def batched_marlin_gate_up(c_ptr, a_ptr, packed_ptr, scales_ptr, ids_ptr, packed_bytes_per_expert, scales_per_expert, n, k,
                           top_k, stream=0):
    rc = lib().twmref_batched_marlin_gate_up(c_ptr, a_ptr, packed_ptr, scales_ptr, ids_ptr, packed_bytes_per_expert,
                                             scales_per_expert, n, k, top_k, stream)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: {rc}")


def batched_marlin_down_axpy(acc_ptr, a_ptr, packed_ptr, scales_ptr, ids_ptr, weights_ptr, packed_bytes_per_expert,
                             scales_per_expert, n, k, top_k, stream=0):
    rc = lib().twmref_batched_marlin_down_axpy(acc_ptr, a_ptr, packed_ptr, scales_ptr, ids_ptr, weights_ptr,
                                               packed_bytes_per_expert, scales_per_expert, n, k, top_k, stream)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: {rc}")


def batched_marlin_split_geglu(out_ptr, gate_up_ptr, moe_dim, top_k, stream=0):
    rc = lib().twmref_batched_marlin_split_geglu(out_ptr, gate_up_ptr, moe_dim, top_k, stream)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: {rc}")
