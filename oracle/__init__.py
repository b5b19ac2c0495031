"""ctypes binding of the CPU oracle (``twm_oracle.c``).

TEST INFRASTRUCTURE ONLY: the parity checker and the timed CPU baseline.  The
product package never imports this module; only the tests, the smoke check
and the benchmark's CPU-baseline leg do.

All arrays are numpy, C-contiguous.  fp16 values travel as ``uint16`` bit
patterns so that no numpy rounding sits between the oracle and the checker.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libtwm_oracle.so")


def build(force: bool = False) -> str:
    """Compile ``twm_oracle.c`` into ``libtwm_oracle.so`` with gcc."""
    src = os.path.join(_HERE, "twm_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "all"], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.twmo_f32_to_f16.restype = C.c_uint16
        _lib.twmo_f32_to_f16.argtypes = [C.c_float]
        _lib.twmo_f16_to_f32.restype = C.c_float
        _lib.twmo_f16_to_f32.argtypes = [C.c_uint16]
        _lib.twmo_w4a16_threaded.restype = C.c_int
        _lib.twmo_num_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def f32_to_f16_bits(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().twmo_f32_to_f16_array(_p(x), _p(out), C.c_long(x.size))
    return out


def f16_bits_to_f32(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, dtype=np.float32)
    lib().twmo_f16_to_f32_array(_p(h), _p(out), C.c_long(h.size))
    return out


def quantize_pack(w, K: int, N: int, group: int = 32, w_is_nk: bool = False):
    """-> (packed u8 [K/32, N, 16], scales u16 [K/group, N])."""
    w = _f32(w)
    assert w.size == K * N
    packed = np.empty((K // 32, N, 16), dtype=np.uint8)
    scales = np.empty((K // group, N), dtype=np.uint16)
    rc = lib().twmo_quantize_pack(_p(w), C.c_int(int(w_is_nk)), C.c_int(K), C.c_int(N),
                                  C.c_int(group), _p(packed), _p(scales))
    if rc != 0:
        raise ValueError("twmo_quantize_pack: bad shape/group")
    return packed, scales


def q4_0_roundtrip(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().twmo_q4_0_roundtrip(_p(x), _p(out), C.c_long(x.size))
    return out


def dequant_f32(packed, scales, K: int, N: int, group: int = 32) -> np.ndarray:
    out = np.empty((K, N), dtype=np.float32)
    rc = lib().twmo_dequant_f32(_p(packed), _p(scales), C.c_int(K), C.c_int(N), C.c_int(group),
                                _p(out))
    if rc != 0:
        raise ValueError("twmo_dequant_f32: bad shape/group")
    return out


def dequant_f16_bits(packed, scales, K: int, N: int, group: int = 32) -> np.ndarray:
    out = np.empty((K, N), dtype=np.uint16)
    rc = lib().twmo_dequant_f16(_p(packed), _p(scales), C.c_int(K), C.c_int(N), C.c_int(group),
                                _p(out))
    if rc != 0:
        raise ValueError("twmo_dequant_f16: bad shape/group")
    return out


def gemm_f32(a, b, M: int, N: int, K: int) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    c = np.empty((M, N), dtype=np.float32)
    lib().twmo_gemm_f32(_p(a), _p(b), _p(c), C.c_int(M), C.c_int(N), C.c_int(K))
    return c


def w4a16_literal(a, packed, scales, M: int, N: int, K: int, group: int = 32) -> np.ndarray:
    """Dequantise the whole matrix, then the naive i-j-p GEMM; one thread."""
    a = _f32(a)
    c = np.empty((M, N), dtype=np.float32)
    scratch = np.empty((K, N), dtype=np.float32)
    rc = lib().twmo_w4a16_literal(_p(a), _p(packed), _p(scales), _p(c), C.c_int(M), C.c_int(N),
                                  C.c_int(K), C.c_int(group), _p(scratch))
    if rc != 0:
        raise ValueError("twmo_w4a16_literal: bad shape/group")
    return c


def w4a16_threaded(a, packed, scales, M: int, N: int, K: int, group: int = 32):
    """Same values as :func:`w4a16_literal`, columns over all host threads.
    -> (c f32 [M,N], threads used)."""
    a = _f32(a)
    c = np.empty((M, N), dtype=np.float32)
    used = lib().twmo_w4a16_threaded(_p(a), _p(packed), _p(scales), _p(c), C.c_int(M), C.c_int(N),
                                     C.c_int(K), C.c_int(group))
    return c, int(used)


def w4a16_f64(a, packed, scales, M: int, N: int, K: int, group: int = 32, weights_f16: bool = False) -> np.ndarray:
    """f64-accumulated result.  weights_f16: the weights are first rounded to f16, the operand a
    tensor-core path multiplies with (dequant_q4_to_f16, quantize.rs:534-571)."""
    a = _f32(a)
    c = np.empty((M, N), dtype=np.float64)
    fn = lib().twmo_w4a16_f64acc_w16 if weights_f16 else lib().twmo_w4a16_f64acc
    fn(_p(a), _p(packed), _p(scales), _p(c), C.c_int(M), C.c_int(N), C.c_int(K), C.c_int(group))
    return c


def m1_kernel_order(a, packed, scales, N: int, K: int, group: int = 32, g0: int = 0,
                    g1: int | None = None) -> np.ndarray:
    """The reference M=1 CUDA kernel's operation order on the CPU (fused
    multiply-adds, per-block partial times scale)."""
    a = _f32(a)
    c = np.empty((N,), dtype=np.float32)
    lib().twmo_m1_kernel_order(_p(a), _p(packed), _p(scales), _p(c), C.c_int(N), C.c_int(group),
                               C.c_int(g0), C.c_int(K // 32 if g1 is None else g1))
    return c


def splitk_plan_ref(n: int, k: int):
    """-> (n_blocks, splits, k_blocks_per_split) of the reference heuristic."""
    nb, sp, kb = C.c_uint(), C.c_uint(), C.c_uint()
    lib().twmo_splitk_plan_ref(C.c_uint(n), C.c_uint(k), C.byref(nb), C.byref(sp), C.byref(kb))
    return nb.value, sp.value, kb.value


def fuse_n(mats, K: int, group: int = 32):
    """mats: list of (packed [K/32,n_i,16], scales [K/group,n_i]) -> fused pair."""
    ns = [int(p.shape[1]) for p, _ in mats]
    total = sum(ns)
    cnt = len(mats)
    ns_c = (C.c_int * cnt)(*ns)
    out_p = np.empty((K // 32, total, 16), dtype=np.uint8)
    out_s = np.empty((K // group, total), dtype=np.uint16)
    ptrs_p = (C.c_void_p * cnt)(*[p.ctypes.data for p, _ in mats])
    ptrs_s = (C.c_void_p * cnt)(*[s.ctypes.data for _, s in mats])
    lib().twmo_fuse_n(ptrs_p, ns_c, C.c_int(cnt), C.c_int(K // 32), C.c_int(16), _p(out_p))
    lib().twmo_fuse_n(ptrs_s, ns_c, C.c_int(cnt), C.c_int(K // group), C.c_int(2), _p(out_s))
    return out_p, out_s


def reorder_to_tw_marlin(blocks, K: int, N: int):
    """Column-major 20-byte Q4_0 blocks -> (packed u8 [K/32, N, 16], scales u16 [K/32, N]) (quantize.rs:912-956)."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    assert blocks.size == (K // 32) * N * 20
    packed = np.empty((K // 32, N, 16), dtype=np.uint8)
    scales = np.empty((K // 32, N), dtype=np.uint16)
    if lib().twmo_reorder_to_tw_marlin(_p(blocks), C.c_int(K), C.c_int(N), _p(packed), _p(scales)) != 0:
        raise ValueError("twmo_reorder_to_tw_marlin: bad shape")
    return packed, scales


def tw_marlin_to_q4_0_blocks(packed, scales, K: int, N: int) -> np.ndarray:
    """The column-major Q4_0 block form of a group-32 TW-Marlin tensor (test input builder)."""
    out = np.empty((K // 32) * N * 20, dtype=np.uint8)
    if lib().twmo_tw_marlin_to_q4_0_blocks(_p(np.ascontiguousarray(packed)), _p(np.ascontiguousarray(scales)), C.c_int(K),
                                           C.c_int(N), _p(out)) != 0:
        raise ValueError("twmo_tw_marlin_to_q4_0_blocks: bad shape")
    return out


def moe_gate_up(a, packed_base, scales_base, topk_ids, packed_bytes_per_expert: int, scales_per_expert: int,
                K: int, N: int, group: int = 32) -> np.ndarray:
    """batched_marlin_gate_up (moe_batched_marlin.rs:21-74) -> f32 [top_k, N]."""
    a, ids = _f32(a), _f32(topk_ids)
    out = np.empty((ids.size, N), dtype=np.float32)
    lib().twmo_moe_gate_up(_p(a), _p(packed_base), _p(scales_base), _p(ids), C.c_long(packed_bytes_per_expert),
                           C.c_long(scales_per_expert), C.c_int(ids.size), C.c_int(K), C.c_int(N), C.c_int(group), _p(out))
    return out


def moe_split_geglu(gate_up, moe_dim: int) -> np.ndarray:
    """batched_marlin_split_geglu (moe_batched_marlin.rs:138-152) -> f32 [top_k, moe_dim]."""
    gu = _f32(gate_up)
    top_k = gu.size // (2 * moe_dim)
    out = np.empty((top_k, moe_dim), dtype=np.float32)
    lib().twmo_moe_split_geglu(_p(gu), C.c_int(top_k), C.c_int(moe_dim), _p(out))
    return out


def moe_down_axpy(a_all, packed_base, scales_base, topk_ids, topk_weights, packed_bytes_per_expert: int,
                  scales_per_expert: int, K: int, N: int, group: int = 32, acc=None):
    """batched_marlin_down_axpy (moe_batched_marlin.rs:78-134), experts added in slot order.
    -> (acc f32 [N], the same sum accumulated in f64)."""
    a_all, ids, wts = _f32(a_all), _f32(topk_ids), _f32(topk_weights)
    out = np.zeros(N, dtype=np.float32) if acc is None else _f32(acc).copy()
    out64 = out.astype(np.float64)
    lib().twmo_moe_down_axpy(_p(a_all), C.c_long(a_all.shape[-1]), _p(packed_base), _p(scales_base), _p(ids), _p(wts),
                             C.c_long(packed_bytes_per_expert), C.c_long(scales_per_expert), C.c_int(ids.size), C.c_int(K),
                             C.c_int(N), C.c_int(group), _p(out), _p(out64))
    return out, out64


def set_threads(n: int) -> None:
    """Use `n` host threads in the threaded routines from now on."""
    lib().twmo_set_num_threads(C.c_int(int(n)))


def num_threads() -> int:
    return int(lib().twmo_num_threads())
